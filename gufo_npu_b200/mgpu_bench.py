"""Multi-GPU measurements of the two sharded paths that are not the decode step of one
sequence: the ragged verify batch with row-split projections, and the MoE layer with its
experts spread over the ranks. Called by bench.py's N > 1 arm (one process per GPU,
torch.distributed over NCCL); every function returns a dict that rank 0 prints inside the
benchmark's JSON line. All inputs are seeded synthetic tensors of the shapes named.

Row split (every output row is an independent dot product,
src/models/qwen35/gguf_projections.cpp:241-243 in the reference): rank r multiplies rows
[r * R / N, (r + 1) * R / N) of each matrix. Gate and up are cut alike, so SwiGLU stays local;
the activated rows and the down projection's rows are all-gathered; of the LM head only each
token's best (value, index) per rank travels. Expert parallelism: gufo_npu_b200/ep.py.
"""
from __future__ import annotations

from typing import Dict

import numpy as np
import torch
import torch.distributed as dist

from . import quantize as Q
from . import synth
from .backend import Context, CudaMoe, CudaProjections


def _timed(fn, steps: int, device) -> float:
    """Milliseconds per call of `fn`: `steps` calls captured into one CUDA graph (kernels, torch
    ops and NCCL collectives alike, so that the host's launch pace does not enter), replayed
    between a barrier and synchronizes, CUDA events on the current stream, the median of five
    replays, then the maximum over the ranks."""
    fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=torch.cuda.current_stream()):
        for _ in range(steps):
            fn()
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(5):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / steps)
    ms = torch.tensor([float(np.median(times))], device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    del graph
    return float(ms.item())


def _rel_l2(got: torch.Tensor, want: torch.Tensor) -> float:
    return float(torch.linalg.norm(got.double() - want.double()) / torch.linalg.norm(want.double()))


class VerifyBatch:
    """The three products of a verify pass at 4B-class shapes (hidden 2560, FFN 9728 Q4_K,
    LM head 248320 x 2560 Q6_K) for M packed token rows, rank `rank` of `world` holding its
    row runs. world = 1 is the one-GPU form of the same computation."""

    HIDDEN, FFN, VOCAB = 2560, 9728, 248320

    def __init__(self, ctx: Context, rank: int, world: int, device, seed: int = 50):
        self.ctx, self.rank, self.world, self.dev = ctx, rank, world, device
        gen = torch.Generator(device=device).manual_seed(seed)
        h, f, v = self.HIDDEN, self.FFN, self.VOCAB
        assert f % world == 0 and h % world == 0 and v % world == 0
        self._keep = []

        def rows(ggml_type, total_rows, cols):
            # The whole matrix is drawn on every rank (same seed, same values); the rank keeps its run.
            w = torch.randn(total_rows, cols, device=device, generator=gen) * 0.02
            per = total_rows // world
            raw = Q.quantize(ggml_type, w[rank * per:(rank + 1) * per].contiguous())
            del w
            self._keep.append(raw)
            return (ctx.matrix_from_device(ggml_type, raw.data_ptr(), per, cols), 0, per)
        torch.cuda.synchronize()
        self.gate_up = Context._parts([rows(Q.GGML_Q4_K, f, h), rows(Q.GGML_Q4_K, f, h)])
        self.down = Context._parts([rows(Q.GGML_Q6_K, h, f)])
        self.head = Context._parts([rows(Q.GGML_Q6_K, v, h)])
        torch.cuda.synchronize()
        self.weight_bytes = (2 * f * Q.row_bytes(Q.GGML_Q4_K, h) + h * Q.row_bytes(Q.GGML_Q6_K, f) +
                             v * Q.row_bytes(Q.GGML_Q6_K, h))

    def buffers(self, m: int):
        h, f, v, n = self.HIDDEN, self.FFN, self.VOCAB, self.world
        z = lambda *s: torch.empty(*s, device=self.dev)
        return {"ffn": z(m, 2 * f // n), "act_local": z(m, f // n), "act": z(n, m, f // n), "out_local": z(m, h // n),
                "out": z(n, m, h // n), "logits": z(m, v // n), "best": z(n, m, 2)}

    def run(self, x: torch.Tensor, b: Dict[str, torch.Tensor]):
        """x [M][hidden] -> (down-projection rows [M][hidden], chosen token ids [M])."""
        m = x.shape[0]
        n, f, h, v = self.world, self.FFN, self.HIDDEN, self.VOCAB
        self.ctx.matmul_device(self.gate_up, 2, x, m, b["ffn"])
        torch.mul(torch.nn.functional.silu(b["ffn"][:, :f // n]), b["ffn"][:, f // n:], out=b["act_local"])
        if n > 1:
            dist.all_gather_into_tensor(b["act"], b["act_local"])
            act = b["act"].permute(1, 0, 2).reshape(m, f).contiguous()
        else:
            act = b["act_local"]
        self.ctx.matmul_device(self.down, 1, act, m, b["out_local"])
        if n > 1:
            dist.all_gather_into_tensor(b["out"], b["out_local"])
            out = b["out"].permute(1, 0, 2).reshape(m, h).contiguous()
        else:
            out = b["out_local"]
        # The verify step's own input is the layer's output; here the packed rows again, so that
        # the LM head does not depend on how the down rows were rounded.
        self.ctx.matmul_device(self.head, 1, x, m, b["logits"])
        value, index = torch.max(b["logits"], dim=1)
        mine = torch.stack([value, (index + self.rank * (v // n)).float()], dim=1)
        if n > 1:
            dist.all_gather_into_tensor(b["best"], mine)
            winner = torch.argmax(b["best"][:, :, 0], dim=0)
            tokens = b["best"][winner, torch.arange(m, device=self.dev), 1].long()
        else:
            tokens = mine[:, 1].long()
        return out, tokens


def verify_batch_tp(ctx: Context, rank: int, world: int, device, steps: int, peak_gbs: float) -> dict:
    """Config 5: 32 sequences x 1-4 draft tokens packed into M rows, row-split over the ranks,
    against the same computation on one GPU (parity and time)."""
    counts = np.random.default_rng(55).integers(1, 5, size=32)
    m = int(counts.sum())
    x = torch.randn(m, VerifyBatch.HIDDEN, device=device, generator=torch.Generator(device=device).manual_seed(56))
    split = VerifyBatch(ctx, rank, world, device)
    b = split.buffers(m)
    for _ in range(3):
        out, tokens = split.run(x, b)
    ms_split = _timed(lambda: split.run(x, b), steps, device)
    out, tokens = split.run(x, b)
    out, tokens = out.clone(), tokens.clone()
    del split, b
    torch.cuda.empty_cache()
    # The same on one GPU (every rank runs its own copy at the same time; no collective).
    whole = VerifyBatch(ctx, 0, 1, device)
    bw = whole.buffers(m)
    for _ in range(3):
        want_out, want_tokens = whole.run(x, bw)
    ms_whole = _timed(lambda: whole.run(x, bw), steps, device)
    want_out, want_tokens = whole.run(x, bw)
    torch.cuda.synchronize()
    check = torch.tensor([_rel_l2(out, want_out), float((tokens != want_tokens).sum())], device=device)
    dist.all_reduce(check, op=dist.ReduceOp.MAX)
    nbytes = whole.weight_bytes
    del whole, bw
    torch.cuda.empty_cache()
    return {"workload": f"ragged verify batch: 32 sequences x 1-4 draft tokens = {m} packed rows, hidden 2560, "
                        f"gate/up 2 x 9728 x 2560 Q4_K, down 2560 x 9728 Q6_K, LM head 248320 x 2560 Q6_K",
            "rows": m, "parallelism": f"tp{world}: rows of every matrix split over the ranks; activated rows and "
                                      f"down rows all-gathered (NCCL), LM head reduced to each token's best "
                                      f"(value, index) per rank",
            "ms_per_pass": ms_split, "ms_per_pass_one_gpu": ms_whole, "speedup_over_one_gpu": ms_whole / ms_split,
            "rows_per_s": m / ms_split * 1e3,
            "weight_bytes": nbytes, "hbm_frac_of_all_gpus": nbytes / (ms_split * 1e-3) / 1e9 / (peak_gbs * world),
            "parity": {"down_rows_rel_l2_vs_one_gpu": float(check[0]), "tokens_that_differ": int(check[1]),
                       "tolerance": 1e-3}}


def moe_layer_ep(ctx: Context, rank: int, world: int, device, steps: int, peak_gbs: float) -> dict:
    """Config 4: one MoE layer at 35B-A3B-class shapes (hidden 2048, 256 experts of width 512,
    top-8, a shared expert), 1 to 4 tokens, the experts spread over the ranks: both exchanges of
    ep.py against one GPU holding every expert (parity and time). Two layers are alternated so
    that the expert rows come from HBM."""
    from .ep import EpMoe
    cfg = synth.ModelConfig(layers=2, hidden=2048, ffn=0, vocab=512, heads=2, kv_heads=1, head_dim=128, rope_dim=32,
                            linear_key_heads=2, linear_value_heads=2, linear_head_dim=128, experts=256,
                            experts_used=8, expert_ffn=512, shared_expert_ffn=512, full_attention_interval=2,
                            tied_embeddings=False)
    tensors = synth.build_model(cfg, 60, device=str(device))
    torch.cuda.synchronize()
    proj = CudaProjections(ctx, cfg, tensors)
    whole = CudaMoe(proj, max_tokens=4)
    ep = EpMoe(ctx, cfg, tensors, proj, rank, world, max_tokens=4)
    per_expert = 2 * cfg.expert_ffn * Q.row_bytes(Q.GGML_Q4_K, cfg.hidden) + cfg.hidden * Q.row_bytes(Q.GGML_Q4_K, cfg.expert_ffn)
    results = []
    gen = torch.Generator(device=device).manual_seed(61)
    for tokens in (1, 2, 4):
        same = torch.randn(tokens, cfg.hidden, device=device, generator=gen)
        shared = torch.randn(tokens, cfg.hidden, device=device, generator=gen)
        own = same + float(rank)       # token-sharded: every rank brings its own rows
        want, got = torch.empty(tokens, cfg.hidden, device=device), torch.empty(tokens, cfg.hidden, device=device)
        layer = [0]

        def step(fn, x):
            layer[0] ^= 1
            fn(layer[0], x, shared, tokens, got)
        entry = {"tokens": tokens}
        for name, fn, x in (("replicated_all_reduce", ep.moe_ffn_replicated, same),
                            ("sharded_all_to_all", ep.moe_ffn_sharded, own)):
            whole.MoeFfn(0, x, shared, tokens, want)
            fn(0, x, shared, tokens, got)
            torch.cuda.synchronize()
            equal = torch.tensor([0.0 if torch.equal(got, want) else 1.0], device=device)
            dist.all_reduce(equal, op=dist.ReduceOp.MAX)
            for _ in range(3):
                step(fn, x)
            ms = _timed(lambda: step(fn, x), steps, device)
            served = tokens * (world if name.startswith("sharded") else 1)
            entry[name] = {"us_per_layer": ms * 1e3, "tokens_served": served,
                           "bit_equal_to_one_gpu": bool(equal.item() == 0.0),
                           "hbm_frac_of_all_gpus": served * cfg.experts_used * per_expert / (ms * 1e-3) / 1e9 /
                                                   (peak_gbs * world)}

        def one(x=same):
            layer[0] ^= 1
            whole.MoeFfn(layer[0], x, shared, tokens, want)
        for _ in range(3):
            one()
        entry["one_gpu_us_per_layer"] = _timed(one, steps, device) * 1e3
        results.append(entry)
    return {"workload": "MoE layer: hidden 2048, 256 experts x (gate, up 512 x 2048; down 2048 x 512) Q4_K, top-8 of "
                        "softmax over N(0,1)-input router logits, shared expert of width 512; 1, 2 and 4 tokens",
            "parallelism": f"ep{world}: {cfg.experts // world} experts per rank, router and shared expert replicated",
            "results": results}
