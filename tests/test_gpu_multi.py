"""Multi-rank GPU parity over NCCL: the row-split decode step against the reference's logits,
and the expert-parallel exchanges against one device holding every expert. One process per
GPU. The two-rank cases skip on a box with one GPU; the one-rank cases run the same code
(collectives included) everywhere."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gufo_npu_b200 import synth
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

STEP_TOL = 2e-3
# A dense model whose heads and FFN width divide over two ranks in whole 256-value blocks.
SPLIT_MODEL = dict(layers=4, hidden=256, ffn=512, vocab=512, full_attention_interval=4, heads=2, kv_heads=1,
                   head_dim=256, rope_dim=64, linear_key_heads=4, linear_value_heads=4, linear_head_dim=128)


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def _worker(rank, world, port, out):
    """Always reports: (rank, failures) or (rank, [traceback]). A rank that is stuck dumps its
    stack to stderr and exits instead of holding the box."""
    import faulthandler
    faulthandler.dump_traceback_later(200, exit=True)
    try:
        _checks(rank, world, port, out)
    except Exception:   # noqa: BLE001 - the parent prints it
        import traceback
        out.put((rank, [traceback.format_exc()]))
    # Leave without tearing the process group down: rank 0 hosts the rendezvous store, and a
    # rank that outlives it would wait on the dead store inside the teardown.
    out.close()
    out.join_thread()
    os._exit(0)


def _checks(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from gufo_npu_b200.backend import Context, CudaMoe, CudaProjections
    from gufo_npu_b200.ep import EpMoe
    from gufo_npu_b200.tp import TpDecoder
    dev = torch.device("cuda", rank)
    stream = torch.cuda.Stream()
    failures = []
    with torch.cuda.stream(stream):
        ctx = Context(rank, stream.cuda_stream)
        # Row-split decode step against the committed logits of the reference's Decoder::Step.
        cfg = synth.ModelConfig(**G.DENSE)
        tensors = synth.build_model(cfg, G.DENSE_SEED)
        # Gathers by this library's kernel over NVLink peer memory, and by NCCL: the same rows
        # travel either way, so the logits agree bit for bit; graphs replay from the third step.
        dec = TpDecoder(ctx, cfg, tensors, rank=rank, world=world, max_positions=32, collective="peer")
        by_nccl = TpDecoder(ctx, cfg, tensors, rank=rank, world=world, max_positions=32, collective="nccl")
        g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "decoder.npz"))
        for i, tok in enumerate(int(t) for t in g["decoder_dense_tokens"]):
            logits = dec.step(tok, stream).cpu().numpy()
            err = rel_l2(logits, g["decoder_dense_logits"][i])
            if err > STEP_TOL:
                failures.append(("tp logits", i, err))
            other = by_nccl.step(tok, stream).cpu().numpy()
            if not np.array_equal(logits, other):
                failures.append(("peer gather differs from NCCL's", i, rel_l2(logits, other)))
        if dec.peers is not None:
            dec.peers.status()   # raises if a wait for a peer's flag ran out
        if world > 1:
            # Product and gather in one kernel: every stage stores its rows into the peers'
            # arenas itself; the gates of the DeltaNet layers are computed in the mixer, so the
            # logits agree with the reference's within the step tolerance, not bit for bit.
            fused = TpDecoder(ctx, cfg, tensors, rank=rank, world=world, max_positions=32, collective="fused")
            for i, tok in enumerate(int(t) for t in g["decoder_dense_tokens"]):
                logits = fused.step(tok, stream).cpu().numpy()
                err = rel_l2(logits, g["decoder_dense_logits"][i])
                if err > STEP_TOL:
                    failures.append(("fused tp logits", i, err))
            fused.peers.status()
        # Heads and FFN width split over the ranks (partial sums added by the next product):
        # against the one-GPU resident decoder on a model whose slices are whole blocks.
        from gufo_npu_b200.backend import CudaDecoder
        scfg = synth.ModelConfig(**SPLIT_MODEL)
        stensors = synth.build_model(scfg, 31)
        split = TpDecoder(ctx, scfg, stensors, rank=rank, world=world, max_positions=32, collective="split")
        one = CudaDecoder(CudaProjections(ctx, scfg, stensors), stensors, max_positions=32, use_graph=False)
        for i, tok in enumerate((5, 77, 300, 12, 501, 9, 250, 64)):
            logits = split.step(tok, stream).cpu().numpy()
            want = one.Step(tok)
            err = rel_l2(logits, want)
            if err > 1e-4 or int(np.argmax(logits)) != int(np.argmax(want)):
                failures.append(("head-split logits", i, err))
        split.peers.status()
        # Expert parallelism against one device with every expert.
        mcfg = synth.ModelConfig(**G.MOE)
        mtensors = synth.build_model(mcfg, G.MOE_SEED)
        proj = CudaProjections(ctx, mcfg, mtensors)
        whole = CudaMoe(proj, max_tokens=4)
        ep = EpMoe(ctx, mcfg, mtensors, proj, rank, world, max_tokens=4)
        tokens = 3
        shared = torch.from_numpy(G.normal(93, tokens, mcfg.hidden)).to(dev)
        # Replicated tokens: the same rows on every rank.
        same = torch.from_numpy(G.normal(92, tokens, mcfg.hidden)).to(dev)
        want = torch.empty(tokens, mcfg.hidden, device=dev)
        got = torch.empty_like(want)
        whole.MoeFfn(0, same, shared, tokens, want)
        ep.moe_ffn_replicated(0, same, shared, tokens, got)
        stream.synchronize()
        if not torch.equal(got, want):
            failures.append(("ep replicated", float((got - want).abs().max())))
        # Token-sharded: every rank brings its own rows.
        own = torch.from_numpy(G.normal(192 + rank, tokens, mcfg.hidden)).to(dev)
        whole.MoeFfn(1, own, shared, tokens, want)
        ep.moe_ffn_sharded(1, own, shared, tokens, got)
        stream.synchronize()
        if not torch.equal(got, want):
            failures.append(("ep sharded", float((got - want).abs().max())))
        if float(want.abs().sum()) == 0:
            failures.append(("ep", "all-zero outputs"))
    dist.barrier()
    torch.cuda.synchronize()
    out.put((rank, failures))


def _run(world):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 33500 + os.getpid() % 2000 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    results = []
    try:
        for _ in range(world):
            results.append(out.get(timeout=240))
    except Exception:   # noqa: BLE001 - queue.Empty: a rank died or hung
        pass
    for p in procs:
        p.join(timeout=20)
        if p.is_alive():
            p.terminate()
            p.join(timeout=20)
    assert len(results) == world, f"{world - len(results)} rank(s) did not report: {results}"
    for rank, failures in results:
        assert not failures, (rank, "\n".join(str(f) for f in failures))


def test_one_rank_nccl_paths():
    _run(1)


def test_two_ranks_row_split_and_expert_parallel():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run(2)


def test_peer_gather_wait_that_runs_out_is_reported_and_the_context_lives():
    """A gather whose peer never raises its flag: a two-rank group on ONE device whose second
    arena is a plain local allocation nobody writes to. With the limit set to two milliseconds
    the kernel must return by itself, the group must report GUFO_CUDA_TIMEOUT, a later gather
    must give up at once, and after a reset the one-rank part of the work and an ordinary
    product must still run. No rank dies and no kernel traps: the wait simply runs out."""
    import ctypes as C
    import time

    from gufo_npu_b200 import _capi
    from gufo_npu_b200 import quantize as Q
    from gufo_npu_b200._capi import GufoCudaError
    from gufo_npu_b200.backend import Context
    dev = torch.device("cuda:0")
    ctx = Context(0)
    lib = ctx.lib
    floats = 1024
    nbytes = _capi.PEER_HEADER_BYTES + 4 * 2 * floats
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    silent = torch.zeros(nbytes, dtype=torch.uint8, device=dev)     # the "peer" that never answers
    arenas = (C.c_void_p * 2)(mine.data_ptr(), silent.data_ptr())
    group = C.c_void_p()
    ctx._check(lib.gufo_cuda_peer_group_create_local(ctx.handle, 0, 2, arenas, nbytes, C.byref(group)))
    ctx._check(lib.gufo_cuda_peer_group_set_limit(group, 2000))
    src = torch.arange(floats, dtype=torch.float32, device=dev)
    ctx._check(lib.gufo_cuda_peer_group_status(group))               # healthy before the first gather
    t0 = time.perf_counter()
    ctx._check(lib.gufo_cuda_peer_allgather_device(group, C.c_void_p(src.data_ptr()), _capi.PEER_HEADER_BYTES, floats))
    ctx.synchronize()
    first = time.perf_counter() - t0
    assert first < 1.0, first                                        # two milliseconds, not four seconds
    with pytest.raises(GufoCudaError) as e:
        ctx._check(lib.gufo_cuda_peer_group_status(group))
    assert e.value.status == _capi.STATUS_TIMEOUT
    # The slice still reached both arenas (rank 0's half of the full vector).
    at = _capi.PEER_HEADER_BYTES
    for arena in (mine, silent):
        got = arena[at:at + 4 * floats].view(torch.float32)
        assert torch.equal(got, src)
    # A later gather gives up at once: no second wait for the limit.
    ctx._check(lib.gufo_cuda_peer_group_set_limit(group, 30 * 1000000))
    t0 = time.perf_counter()
    ctx._check(lib.gufo_cuda_peer_allgather_device(group, C.c_void_p(src.data_ptr()), _capi.PEER_HEADER_BYTES, floats))
    ctx.synchronize()
    assert time.perf_counter() - t0 < 1.0
    # After a reset the group is healthy again, and the context still multiplies.
    ctx._check(lib.gufo_cuda_peer_group_reset(group))
    ctx._check(lib.gufo_cuda_peer_group_status(group))
    raw = Q.random_blocks(Q.GGML_Q4_K, 64, 512, seed=5).numpy()
    m = ctx.matrix_upload(Q.GGML_Q4_K, raw, 64, 512)
    y = ctx.matmul([(m, 0, 64)], np.ones((1, 512), dtype=np.float32), 1, 64)
    assert np.isfinite(y).all()
    ctx._check(lib.gufo_cuda_peer_group_destroy(group))
    ctx.close()


def test_product_that_gathers_by_itself_on_one_device():
    """gufo_cuda_matmul_gather_device with both ranks of a two-rank group on ONE device and one
    stream (two local arenas): each rank's product stores its rows into both arenas and raises
    its flags; the waits, enqueued after both products, find the flags set. Both arenas must
    then hold the whole product, equal to the ordinary entry point's, over several turns (a
    residual + norm input, a plain one, a SwiGLU one)."""
    import ctypes as C

    from gufo_npu_b200 import _capi
    from gufo_npu_b200 import quantize as Q
    from gufo_npu_b200.backend import Context
    dev = torch.device("cuda:0")
    ctx = Context(0)
    lib = ctx.lib
    rows, cols = 96, 512          # per rank: 48 rows
    local = rows // 2
    raw = Q.random_blocks(Q.GGML_Q4_K, rows, cols, seed=8).to(dev)
    torch.cuda.synchronize()
    whole = Context._parts([(ctx.matrix_from_device(Q.GGML_Q4_K, raw.data_ptr(), rows, cols), 0, rows)])
    rb = Q.row_bytes(Q.GGML_Q4_K, cols)
    halves = [Context._parts([(ctx.matrix_from_device(Q.GGML_Q4_K, raw.data_ptr() + r * local * rb, local, cols), 0,
                               local)]) for r in range(2)]
    nbytes = _capi.PEER_HEADER_BYTES + 4 * rows
    arenas_t = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(2)]
    arenas = (C.c_void_p * 2)(*(a.data_ptr() for a in arenas_t))
    groups = []
    for r in range(2):
        group = C.c_void_p()
        ctx._check(lib.gufo_cuda_peer_group_create_local(ctx.handle, r, 2, arenas, nbytes, C.byref(group)))
        groups.append(group)
    gen = torch.Generator(device=dev).manual_seed(9)
    for turn in range(5):
        kind = turn % 3
        want = torch.empty(1, rows, device=dev)
        p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
        if kind == 0:     # residual + delta through RMSNorm
            h = torch.randn(cols, device=dev, generator=gen)
            delta = torch.randn(cols, device=dev, generator=gen)
            w = 1.0 + 0.1 * torch.randn(cols, device=dev, generator=gen)
            x_full = (h + delta) * torch.rsqrt(((h + delta) ** 2).mean() + 1e-6) * w
            h_out = [torch.empty(cols, device=dev) for _ in range(2)]
            scratch = [torch.empty(cols, device=dev) for _ in range(2)]
            inputs = [_capi.FusedInput(_capi.PROLOGUE_RES_NORM, None, p(h), p(delta), p(w), 1e-6, p(h_out[r]),
                                       p(scratch[r]), None) for r in range(2)]
        elif kind == 1:   # plain rows
            x_full = torch.randn(cols, device=dev, generator=gen)
            inputs = [_capi.FusedInput(_capi.PROLOGUE_PLAIN, p(x_full), None, None, None, 0.0, None, None, None)] * 2
        else:             # SwiGLU of [gate | up]
            gate_up = torch.randn(2 * cols, device=dev, generator=gen)
            x_full = torch.nn.functional.silu(gate_up[:cols]) * gate_up[cols:]
            inputs = [_capi.FusedInput(_capi.PROLOGUE_SWIGLU, p(gate_up), None, None, None, 0.0, None, None, None)] * 2
        torch.cuda.synchronize()
        ctx.matmul_device(whole, 1, x_full.reshape(1, cols).contiguous(), 1, want)
        for r in range(2):
            ctx._check(lib.gufo_cuda_matmul_gather_device(groups[r], halves[r], 1, C.byref(inputs[r]),
                                                          _capi.PEER_HEADER_BYTES, 0, -1))
        for r in range(2):
            ctx._check(lib.gufo_cuda_peer_wait_device(groups[r], 0))
        ctx.synchronize()
        for r in range(2):
            ctx._check(lib.gufo_cuda_peer_group_status(groups[r]))
            got = arenas_t[r][_capi.PEER_HEADER_BYTES:].view(torch.float32)
            assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= 1e-5, (turn, r)
        if kind == 0:
            assert torch.allclose(h_out[0], h + delta)
    for group in groups:
        ctx._check(lib.gufo_cuda_peer_group_destroy(group))
    ctx.close()
