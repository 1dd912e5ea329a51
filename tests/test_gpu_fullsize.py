"""Parity at the sizes the benchmark runs, and of the attention past a handful of positions.

The other GPU parity tests use small matrices and an 8-position decoder run; these close the
gap to the benchmarked configuration: the 2B-class decode step against the reference's own
Decoder::Step (the compiled reference, where it was built), LM heads of 248320 rows against the
oracle on a row sample, the decoder over 1100 positions against committed reference logits, and
the attention entry point by itself against the CPU restatement.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from gufo_npu_b200 import _capi
from gufo_npu_b200 import quantize as Q
from gufo_npu_b200 import synth
from gufo_npu_b200.backend import Context, CudaDecoder, CudaProjections
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

STEP_TOL = 2e-3      # logits relative L2 (the reference's own decoder bound, decoder_test.cpp:30-31)


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


@pytest.fixture(scope="module")
def ctx():
    c = Context(0)
    yield c
    c.close()


def test_config2_decode_step_matches_compiled_reference(ctx, reflib):
    """The benchmark's model (hidden 2048, FFN 6144, 24 layers, 248320-row tied Q6_K head):
    six tokens through gufo_cuda_decoder_step and through the reference's Decoder::Step over
    GgufProjections(kFloat); logits within the step tolerance and the same arg-max."""
    import bench
    cfg = bench.model_config()
    tensors = synth.build_model(cfg, seed=1, device="cuda:0")
    proj = CudaProjections(ctx, cfg, tensors)
    dec = CudaDecoder(proj, tensors, max_positions=64, use_graph=True)
    host = {k: synth.Tensor(t.shape, t.ggml_type, t.data.cpu()) for k, t in tensors.items()}
    image = synth.to_gguf(cfg, host)
    del host
    model = reflib.open_model(image, precision_float=True)
    del image
    model.decoder_reset()
    tokens = [int(t) for t in np.random.default_rng(17).integers(0, cfg.vocab, size=6)]
    worst = 0.0
    for i, tok in enumerate(tokens):
        got = dec.Step(tok)
        want = model.decoder_step(tok, cfg.vocab)
        err = rel_l2(got, want)
        worst = max(worst, err)
        assert err <= STEP_TOL, (i, err)
        assert int(np.argmax(got)) == int(np.argmax(want)), i
    assert worst < 2e-4, worst
    model.close()
    dec.close()


@pytest.mark.parametrize("cols", [2048, 2560])
@pytest.mark.parametrize("tokens", [1, 32])
def test_lm_head_248320_rows_against_oracle_row_sample(ctx, oracle, cols, tokens):
    """The LM heads of the benchmark and of the verify batch (248320 x 2048 and x 2560 Q6_K):
    one token on the GEMV kernel, 32 packed rows on the tcgen05 GEMM; every 97th row against
    the oracle's fused row dot."""
    rows = 248320
    dev = torch.device("cuda:0")
    gen = torch.Generator(device=dev).manual_seed(40 + cols)
    raw = Q.quantize(Q.GGML_Q6_K, torch.randn(rows, cols, device=dev, generator=gen) * 0.02)
    x = torch.randn(tokens, cols, device=dev, generator=gen)
    y = torch.empty(tokens, rows, device=dev)
    # The context has its own stream: the inputs must be ready before it rearranges the Q6_K
    # rows (matrix_from_device) and multiplies.
    torch.cuda.synchronize()
    m = ctx.matrix_from_device(Q.GGML_Q6_K, raw.data_ptr(), rows, cols)
    ctx.matmul_device(Context._parts([(m, 0, rows)]), 1, x, tokens, y)
    ctx.synchronize()
    got = y.cpu().numpy()
    sample = np.arange(0, rows, 97)
    host_rows = raw.view(rows, -1)[torch.from_numpy(sample).to(dev)].cpu().numpy()
    want = oracle.matmul([(host_rows, Q.GGML_Q6_K, 0, sample.size)], cols, x.cpu().numpy())
    tol = 1e-3
    for t in range(tokens):
        assert rel_l2(got[t, sample], want[t]) <= tol, (t, rel_l2(got[t, sample], want[t]))
    assert np.isfinite(got).all()
    ctx.matrix_free(m)


@pytest.mark.parametrize("use_graph", [False, True])
def test_decoder_1100_positions_match_reference_logits(ctx, golden, use_graph):
    """The dense test model over 1100 positions against the reference's committed logits at
    positions around its 128-position attention slices and past a thousand: the attention's
    position slices hold many positions each, of unequal length."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    dec = CudaDecoder(CudaProjections(ctx, cfg, tensors), tensors, max_positions=G.LONG_STEPS, use_graph=use_graph)
    g = golden("decoder_long")
    keep = {int(p): i for i, p in enumerate(g["positions"])}
    worst = 0.0
    for pos, tok in enumerate(G.long_tokens(cfg.vocab)):
        if pos in keep:
            got = dec.Step(int(tok))
            want = g["logits"][keep[pos]]
            err = rel_l2(got, want)
            worst = max(worst, err)
            assert err <= STEP_TOL, (pos, err)
            assert int(np.argmax(got)) == int(np.argmax(want)), pos
        else:
            dec.step_device(int(tok))
    assert worst < 5e-4, worst
    assert dec.position == G.LONG_STEPS
    dec.close()


@pytest.mark.parametrize("heads,kv_heads,head_dim,rope_dim", [(8, 2, 256, 64), (2, 1, 128, 32), (4, 4, 64, 64)])
def test_attention_device_matches_cpu_restatement(ctx, heads, kv_heads, head_dim, rope_dim):
    """gufo_cuda_attention_device by itself: tokens appended one by one at cache lengths that
    give empty, one-position, unequal and long position slices."""
    from oracle import attention as A
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(3 * heads + head_dim)
    max_positions = 1600
    kv = kv_heads * head_dim
    width = 2 * heads * head_dim + 2 * kv
    q_norm = (1.0 + 0.1 * rng.standard_normal(head_dim)).astype(np.float32)
    k_norm = (1.0 + 0.1 * rng.standard_normal(head_dim)).astype(np.float32)
    inv_freq = np.array([1.0 / (1e7 ** (2.0 * i / rope_dim)) for i in range(rope_dim // 2)], dtype=np.float32)
    keys_h = np.zeros((max_positions, kv), dtype=np.float16)
    values_h = np.zeros((max_positions, kv), dtype=np.float16)
    # A cache filled with plausible rows up to the longest length tested.
    fill = 1537
    keys_h[:fill] = (rng.standard_normal((fill, kv)) * 0.7).astype(np.float16)
    values_h[:fill] = rng.standard_normal((fill, kv)).astype(np.float16)
    t = lambda a: torch.from_numpy(a).to(dev)
    keys, values = t(keys_h.copy()), t(values_h.copy())
    qn, kn, fr = t(q_norm), t(k_norm), t(inv_freq)
    queries = torch.empty(heads * head_dim, device=dev)
    partials = torch.empty(kv_heads * 32 * (heads // kv_heads) * (head_dim + 2), device=dev)
    out = torch.empty(heads * head_dim, device=dev)
    position = torch.zeros(1, dtype=torch.int32, device=dev)
    for pos in (0, 1, 6, 7, 8, 9, 130, 1000, 1536):
        row = rng.standard_normal(width).astype(np.float32)
        x = t(row)
        position.fill_(pos)
        torch.cuda.synchronize()
        args = _capi.AttentionArgs(heads, kv_heads, head_dim, rope_dim, max_positions, 1e-6, position.data_ptr(),
                                   x.data_ptr(), qn.data_ptr(), kn.data_ptr(), fr.data_ptr(), keys.data_ptr(),
                                   values.data_ptr(), queries.data_ptr(), partials.data_ptr(), out.data_ptr())
        ctx._check(ctx.lib.gufo_cuda_attention_device(ctx.handle, C.byref(args)))
        ctx.synchronize()
        want = A.attention_step(row, pos, keys_h, values_h, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                q_norm=q_norm, k_norm=k_norm, inv_freq=inv_freq, rms_eps=1e-6)
        assert rel_l2(out.cpu().numpy(), want) <= 2e-4, (pos, rel_l2(out.cpu().numpy(), want))
        # The appended cache row, as fp16 bits (one unit in the last place for the normed key).
        got_k = keys[pos].cpu().numpy().astype(np.float32)
        assert np.allclose(got_k, keys_h[pos].astype(np.float32), rtol=2e-3, atol=1e-4), pos
        assert np.array_equal(values[pos].cpu().numpy().view(np.uint16), values_h[pos].view(np.uint16)), pos


def test_logits_into_pinned_memory_equal_copied_logits(ctx):
    """gufo_cuda_decoder_step with a pinned host buffer: once the step replays as a graph, the LM
    head writes the caller's buffer itself and no copy follows; the logits are those of a decoder
    whose logits are copied down, bit for bit, also after the caller switches buffers."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    proj = CudaProjections(ctx, cfg, tensors)
    copied = CudaDecoder(proj, tensors, max_positions=32, use_graph=True)
    direct = CudaDecoder(proj, tensors, max_positions=32, use_graph=True)
    pinned = [torch.empty(cfg.vocab, dtype=torch.float32).pin_memory() for _ in range(2)]
    for i, tok in enumerate((3, 99, 7, 250, 11, 400, 42, 17, 301, 5)):
        want = copied.Step(tok)
        buf = pinned[0] if i < 6 else pinned[1]
        buf.fill_(float("nan"))
        got = direct.Step(tok, buf.numpy())
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), i
    copied.close()
    direct.close()
