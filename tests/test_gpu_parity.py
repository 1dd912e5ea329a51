"""GPU parity: the CUDA path through the C ABI against the CPU oracle and the committed
reference outputs. Tolerances: dequantization bit-exact; GEMV / GEMM outputs <= 1e-3
relative L2 (fp32); DeltaNet state and output <= 1e-4 relative L2."""
import numpy as np
import pytest
import torch

from gufo_npu_b200 import quantize as Q
from gufo_npu_b200 import synth
from gufo_npu_b200.backend import Context, CudaDecoder, CudaMixer, CudaProjections, Stage, stage_inputs
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

GEMV_TOL = 1e-3      # relative L2, fp32 outputs
DELTA_TOL = 1e-4     # relative L2, DeltaNet state and output
TYPES = {"q4k": Q.GGML_Q4_K, "q6k": Q.GGML_Q6_K}


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.fixture(scope="module", params=["default", "general"])
def ctx(request):
    """Every test runs twice: with the kernels the dispatcher picks, and with every product
    forced through the general kernel."""
    c = Context(0)
    c.set_option("general_gemv", int(request.param == "general"))
    yield c
    c.close()


# ---- dequantization -------------------------------------------------------

@pytest.mark.parametrize("name,ggml_type", [("Q4_K", Q.GGML_Q4_K), ("Q6_K", Q.GGML_Q6_K)])
def test_dequantize_reference_fixtures_bit_exact(ctx, golden, name, ggml_type):
    raw = np.fromfile(golden.path("quant", name + ".bin"), dtype=np.uint8)
    want = np.fromfile(golden.path("quant", name + ".f32"), dtype=np.float32)
    m = ctx.matrix_upload(ggml_type, raw, 1, want.size)
    got = ctx.dequantize(m, 0, 1, want.size)
    assert np.array_equal(bits(got.ravel()), bits(want))
    ctx.matrix_free(m)


@pytest.mark.parametrize("name", ["q4k", "q6k"])
def test_dequantize_matches_oracle_bit_exact(ctx, oracle, name):
    t = TYPES[name]
    rows, cols = 37, 1024
    for raw in (Q.random_blocks(t, rows, cols, seed=21).numpy(),
                Q.quantize(t, torch.from_numpy(G.normal(22, rows, cols) * 0.02)).numpy()):
        m = ctx.matrix_upload(t, raw, rows, cols)
        got = ctx.dequantize(m, 0, rows, cols)
        want = oracle.dequantize(t, raw, rows * cols).reshape(rows, cols)
        assert np.array_equal(bits(got), bits(want))
        # A row range, as the embedding lookup reads one row.
        got = ctx.dequantize(m, 5, 2, cols)
        assert np.array_equal(bits(got), bits(want[5:7]))
        ctx.matrix_free(m)


def test_dequantize_subnormal_and_extreme_scales(ctx, oracle):
    """fp16 d / dmin that are subnormal, zero or the largest finite half."""
    for t, offs in ((Q.GGML_Q4_K, (0, 2)), (Q.GGML_Q6_K, (208,))):
        raw = Q.random_blocks(t, 1, 256 * 6, seed=31).numpy().reshape(6, -1)
        for b, half in enumerate((0x0001, 0x03FF, 0x0000, 0x7BFF, 0x8001, 0xFBFF)):
            for at in offs:
                raw[b, at] = half & 0xFF
                raw[b, at + 1] = half >> 8
        m = ctx.matrix_upload(t, raw.reshape(-1), 1, 256 * 6)
        got = ctx.dequantize(m, 0, 1, 256 * 6)
        want = oracle.dequantize(t, raw.reshape(-1), 256 * 6)
        assert np.array_equal(bits(got.ravel()), bits(want))
        ctx.matrix_free(m)


def test_dequantize_full_size_bit_exact(ctx, oracle):
    """The 6144 x 2048 Q4_K matrix of the headline GEMV: every value, bit for bit."""
    gen = torch.Generator().manual_seed(1)
    w = torch.randn(6144, 2048, generator=gen) * 0.02
    raw = Q.quantize_q4_k(w).numpy()
    m = ctx.matrix_upload(Q.GGML_Q4_K, raw, 6144, 2048)
    got = ctx.dequantize(m, 0, 6144, 2048)
    want = oracle.dequantize(Q.GGML_Q4_K, raw, 6144 * 2048).reshape(6144, 2048)
    assert np.array_equal(bits(got), bits(want))
    # The packer's codes reproduce the weights to within one quantization step.
    assert rel_l2(got, w.numpy()) < 0.1
    ctx.matrix_free(m)


# ---- GEMV / small-M GEMM ----------------------------------------------------

def test_headline_gemv_q4k_6144x2048(ctx, oracle):
    """W 6144 x 2048 from N(0, 0.02) seed 1, x N(0, 1) seed 2, batch 1."""
    w = torch.randn(6144, 2048, generator=torch.Generator().manual_seed(1)) * 0.02
    raw = Q.quantize_q4_k(w).numpy()
    x = torch.randn(2048, generator=torch.Generator().manual_seed(2)).numpy()
    m = ctx.matrix_upload(Q.GGML_Q4_K, raw, 6144, 2048)
    got = ctx.matmul([(m, 0, 6144)], x, 1, 6144)
    want = oracle.matmul([(raw, Q.GGML_Q4_K, 0, 6144)], 2048, x)
    exact = oracle.matmul([(raw, Q.GGML_Q4_K, 0, 6144)], 2048, x, exact=True)
    assert rel_l2(got, want) <= GEMV_TOL
    assert rel_l2(got, exact) < 1e-5          # fp32 accumulation sits far inside the tolerance
    ctx.matrix_free(m)


@pytest.mark.parametrize("name", ["q4k", "q6k"])
@pytest.mark.parametrize("rows,cols", [(1, 256), (16, 256), (1000, 512), (2048, 6144), (257, 2560)])
def test_gemv_shapes_random_blocks(ctx, oracle, name, rows, cols):
    """Ragged row counts and every block pattern; error bound of the reference's fused-dot
    test (2e-5 of sum |w x|, tests/models/qwen35/gguf_dot_test.cpp:114-116)."""
    t = TYPES[name]
    raw = Q.random_blocks(t, rows, cols, seed=rows + cols).numpy()
    x = G.normal(rows * 3 + cols, cols)
    m = ctx.matrix_upload(t, raw, rows, cols)
    got = ctx.matmul([(m, 0, rows)], x, 1, rows)[0]
    want = oracle.matmul([(raw, t, 0, rows)], cols, x)[0]
    assert rel_l2(got, want) <= GEMV_TOL
    wabs = np.abs(oracle.dequantize(t, raw[:64], min(rows, 64) * cols).reshape(-1, cols))
    magnitude = wabs @ np.abs(x)
    n = magnitude.size
    exact = oracle.matmul([(raw, t, 0, n)], cols, x, exact=True)[0]
    assert np.all(np.abs(got[:n] - exact) < 2e-5 * magnitude)
    ctx.matrix_free(m)


def test_activation_extremes(ctx, oracle):
    """Activations with a wide dynamic range inside one 256-value block, zero blocks, tiny and
    huge magnitudes: the fixed-point staging keeps fp32-level accuracy."""
    rows, cols = 64, 1024
    rng = np.random.default_rng(17)
    x = rng.standard_normal(cols).astype(np.float32)
    x[0:256] = 0.0                                  # an all-zero block
    x[256:512] *= 1e-30                             # tiny
    x[512:768] *= 1e20                              # huge
    x[768] = 3000.0                                 # one outlier among N(0, 1)
    x[900:1024] *= np.float32(2.0) ** rng.integers(-20, 4, 124)
    for name, t in TYPES.items():
        raw = Q.random_blocks(t, rows, cols, seed=4).numpy()
        m = ctx.matrix_upload(t, raw, rows, cols)
        got = ctx.matmul([(m, 0, rows)], x, 1, rows)[0]
        exact = oracle.matmul([(raw, t, 0, rows)], cols, x, exact=True)[0]
        wabs = np.abs(oracle.dequantize(t, raw, rows * cols).reshape(rows, cols)).astype(np.float64)
        magnitude = wabs @ np.abs(x).astype(np.float64)
        assert np.all(np.abs(got - exact) < 2e-5 * magnitude)
        # Non-finite activations give non-finite outputs, as on the CPU.
        bad = x.copy()
        bad[5] = np.inf
        assert not np.isfinite(ctx.matmul([(m, 0, rows)], bad, 1, rows)).any()
        ctx.matrix_free(m)


@pytest.mark.parametrize("ggml_type", [Q.GGML_Q4_K, Q.GGML_Q6_K])
@pytest.mark.parametrize("tokens,cols,rows", [(1, 768, 96), (2, 768, 96), (1, 2048, 3072), (1, 512, 16)])
def test_gate_up_product_activates_its_own_rows(request, ctx, oracle, ggml_type, tokens, cols, rows):
    """gufo_cuda_fused_input.epilogue = SWIGLU (the reference's npu::Epilogue::kSwiGlu,
    src/npu/gemv.hpp:64-68): the stacked gate and up rows multiplied by one launch that stores
    silu(gate) * up, against the activation of the oracle's rows; with a fused residual + norm
    input whose pending add is the sum of three vectors (delta_parts)."""
    dev = torch.device("cuda:0")
    eps = 1e-6
    gate = Q.quantize(ggml_type, torch.from_numpy(G.normal(170, rows, cols) * 0.05)).numpy()
    up_w = Q.quantize(ggml_type, torch.from_numpy(G.normal(171, rows, cols) * 0.05)).numpy()
    mg, mu = ctx.matrix_upload(ggml_type, gate, rows, cols), ctx.matrix_upload(ggml_type, up_w, rows, cols)
    parts = Context._parts([(mg, 0, rows), (mu, 0, rows)])
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev)
    x = G.normal(172, tokens, cols)
    want_rows = oracle.matmul([(gate, ggml_type, 0, rows), (up_w, ggml_type, 0, rows)], cols, x)
    g, u = want_rows[:, :rows].astype(np.float64), want_rows[:, rows:].astype(np.float64)
    want = g / (1.0 + np.exp(-g)) * u
    act = torch.empty(tokens, rows, device=dev)
    from gufo_npu_b200._capi import GufoCudaError
    if "general" in request.node.name:
        # The general kernel has no such epilogue: refused, nothing enqueued.
        with pytest.raises(GufoCudaError):
            ctx.matmul_fused_device(parts, 2, tokens, act, x=t(x), activate=True)
        ctx.matrix_free(mg)
        ctx.matrix_free(mu)
        return
    ctx.matmul_fused_device(parts, 2, tokens, act, x=t(x), activate=True)
    ctx.synchronize()
    assert rel_l2(act.cpu().numpy(), want) <= 1e-5
    if tokens == 1:
        # Residual plus three partial vectors through the norm, then the activating product.
        h, w = G.normal(173, 1, cols), G.normal(174, cols) * 0.2 + 1.0
        partials = G.normal(175, 3, cols) * 0.3
        total = (h[0] + partials[0] + partials[1] + partials[2]).astype(np.float32)
        normed = (total / np.sqrt((total.astype(np.float64) ** 2).mean() + eps) * w).astype(np.float32)
        h_out, scratch = torch.empty(1, cols, device=dev), torch.empty(1, cols, device=dev)
        ctx.matmul_fused_device(parts, 2, 1, act, residual=t(h), delta=t(partials), delta_parts=3, delta_stride=cols,
                                norm_weight=t(w), rms_eps=eps, residual_out=h_out, scratch=scratch, activate=True)
        ctx.synchronize()
        assert np.array_equal(h_out.cpu().numpy()[0], ((h[0] + partials[0]) + partials[1]) + partials[2])
        rows2 = oracle.matmul([(gate, ggml_type, 0, rows), (up_w, ggml_type, 0, rows)], cols, normed[None, :])
        g, u = rows2[:, :rows].astype(np.float64), rows2[:, rows:].astype(np.float64)
        assert rel_l2(act.cpu().numpy()[:1], g / (1.0 + np.exp(-g)) * u) <= 1e-5
    # Parts that are not whole tiles are refused and nothing runs.
    odd = Context._parts([(mg, 0, rows - 8), (mu, 0, rows - 8)])
    with pytest.raises(GufoCudaError):
        ctx.matmul_fused_device(odd, 2, tokens, act, x=t(x), activate=True)
    ctx.matrix_free(mg)
    ctx.matrix_free(mu)


@pytest.mark.parametrize("tokens", [1, 2, 3, 4, 7, 8, 9, 19])
def test_small_m_tokens_do_not_change_rows(ctx, oracle, tokens):
    """Results do not depend on how many tokens come together
    (src/models/qwen35/gguf_projections.cpp:241-243): to fp32 summation order on the GEMV kernels;
    a product that the dispatcher sends to the tcgen05 path differs by that path's fp16 rounding,
    hence the wider bound from 16 tokens on. Both are far inside the 1e-3 bound."""
    rows, cols = 96, 768
    x = G.normal(50 + tokens, tokens, cols)
    exact_tol, same_tol = (1e-5, 1e-6) if tokens < 16 else (5e-4, 5e-4)
    for name, t in TYPES.items():
        raw = Q.quantize(t, torch.from_numpy(G.normal(60, rows, cols) * 0.02)).numpy()
        m = ctx.matrix_upload(t, raw, rows, cols)
        got = ctx.matmul([(m, 0, rows)], x, tokens, rows)
        want = oracle.matmul([(raw, t, 0, rows)], cols, x)
        assert rel_l2(got, want) <= exact_tol
        single = np.stack([ctx.matmul([(m, 0, rows)], x[i], 1, rows)[0] for i in range(tokens)])
        assert rel_l2(got, single) <= same_tol
        ctx.matrix_free(m)


@pytest.mark.parametrize("tokens", [1, 2, 3, 9])
@pytest.mark.parametrize("cols", [768, 6144])
def test_fused_products_match_the_separate_steps(ctx, oracle, tokens, cols):
    """gufo_cuda_matmul_fused_device (the reference's npu::Prologue options, src/npu/gemv.hpp:58-68):
    the residual add + RMSNorm and the SwiGLU done inside the product against numpy's, the product
    against the oracle's fused row dots on those inputs. Q4_K and Q6_K parts with an F32 part
    beside them; 9 tokens take the path that materialises the rows."""
    from gufo_npu_b200._capi import GufoCudaError
    dev = torch.device("cuda:0")
    rows, eps = 80, 1e-6
    raws = {"q4": Q.quantize(Q.GGML_Q4_K, torch.from_numpy(G.normal(70, rows, cols) * 0.02)).numpy(),
            "q6": Q.quantize(Q.GGML_Q6_K, torch.from_numpy(G.normal(71, rows, cols) * 0.02)).numpy(),
            "f32": (G.normal(72, 8, cols) * 0.05).astype(np.float32)}
    types = {"q4": Q.GGML_Q4_K, "q6": Q.GGML_Q6_K, "f32": Q.GGML_F32}
    nrows = {"q4": rows, "q6": rows, "f32": 8}
    mats = {k: ctx.matrix_upload(types[k], raws[k], nrows[k], cols) for k in raws}
    listing = [(mats[k], 0, nrows[k]) for k in ("q4", "q6", "f32")]
    oracle_parts = [(raws[k].view(np.uint8) if k == "f32" else raws[k], types[k], 0, nrows[k])
                    for k in ("q4", "q6", "f32")]
    parts = Context._parts(listing)
    total = sum(nrows.values())
    up = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev)
    y = torch.empty(tokens, total, device=dev)
    scratch = torch.empty(tokens, cols, device=dev)
    # Residual + delta through RMSNorm.
    h, delta, w = G.normal(73, tokens, cols), G.normal(74, tokens, cols) * 0.3, G.normal(75, cols) * 0.2 + 1.0
    h_out = torch.empty(tokens, cols, device=dev)
    counter = torch.zeros(1, dtype=torch.int32, device=dev)
    ctx.matmul_fused_device(parts, len(listing), tokens, y, residual=up(h), delta=up(delta), norm_weight=up(w),
                            rms_eps=eps, residual_out=h_out, scratch=scratch, advance=counter)
    ctx.synchronize()
    total_h = (h + delta).astype(np.float32)
    normed = (total_h / np.sqrt((total_h.astype(np.float64) ** 2).mean(axis=1, keepdims=True) + eps) * w).astype(np.float32)
    assert np.array_equal(h_out.cpu().numpy(), total_h)
    assert rel_l2(scratch.cpu().numpy(), normed) <= 1e-6
    assert int(counter.item()) == tokens
    assert rel_l2(y.cpu().numpy(), oracle.matmul(oracle_parts, cols, normed)) <= 1e-5
    # Without a pending add the residual passes through.
    ctx.matmul_fused_device(parts, len(listing), tokens, y, residual=up(h), norm_weight=up(w), rms_eps=eps,
                            residual_out=h_out, scratch=scratch)
    ctx.synchronize()
    assert np.array_equal(h_out.cpu().numpy(), h.astype(np.float32))
    # SwiGLU of [gate | up] rows (the F32 part sends the product down the materialising path).
    gu = G.normal(76, tokens, 2 * cols)
    act = (gu[:, :cols] / (1.0 + np.exp(-gu[:, :cols].astype(np.float64))) * gu[:, cols:]).astype(np.float32)
    for picked, oparts in ((listing[:2], oracle_parts[:2]), (listing, oracle_parts)):
        width = sum(p[2] for p in picked)
        out = torch.empty(tokens, width, device=dev)
        ctx.matmul_fused_device(Context._parts(picked), len(picked), tokens, out, x=up(gu), swiglu=True, scratch=scratch)
        ctx.synchronize()
        assert rel_l2(out.cpu().numpy(), oracle.matmul(oparts, cols, act)) <= 1e-5
    # Plain rows: the same as the ordinary product.
    x = G.normal(77, tokens, cols)
    ctx.matmul_fused_device(parts, len(listing), tokens, y, x=up(x))
    ctx.synchronize()
    assert rel_l2(y.cpu().numpy(), ctx.matmul(listing, x, tokens, total)) <= 1e-6
    # Refusals: residual_out on top of residual; a missing scratch.
    same = up(h)
    with pytest.raises(GufoCudaError):
        ctx.matmul_fused_device(parts, len(listing), tokens, y, residual=same, norm_weight=up(w), rms_eps=eps,
                                residual_out=same, scratch=scratch)
    with pytest.raises(GufoCudaError):
        ctx.matmul_fused_device(parts, len(listing), tokens, y, x=up(gu), swiglu=True)
    for m in mats.values():
        ctx.matrix_free(m)


def test_empty_and_bad_products(ctx):
    from gufo_npu_b200._capi import GufoCudaError
    raw = Q.random_blocks(Q.GGML_Q4_K, 8, 256, seed=1).numpy()
    m = ctx.matrix_upload(Q.GGML_Q4_K, raw, 8, 256)
    other = ctx.matrix_upload(Q.GGML_Q4_K, Q.random_blocks(Q.GGML_Q4_K, 8, 512, seed=1).numpy(), 8, 512)
    x = np.zeros(256, dtype=np.float32)
    assert ctx.matmul([(m, 0, 8)], np.zeros((0, 256), dtype=np.float32), 0, 8).shape == (0, 8)
    for bad, status in (([(m, 4, 8)], 2), ([(m, -1, 2)], 2), ([(m, 0, 0)], 2), ([(999, 0, 1)], 1),
                        ([(m, 0, 8), (other, 0, 8)], 2), ([], 1)):
        with pytest.raises(GufoCudaError) as e:
            ctx.matmul(bad, x, 1, 8)
        assert e.value.status == status
    with pytest.raises(GufoCudaError) as e:
        ctx.matrix_upload(10, raw, 8, 256)          # Q2_K: not run by this backend
    assert e.value.status == 3
    with pytest.raises(GufoCudaError) as e:
        ctx.matrix_upload(Q.GGML_Q4_K, raw, 8, 250)
    assert e.value.status == 2
    ctx.matrix_free(m)
    ctx.matrix_free(other)
    with pytest.raises(GufoCudaError):
        ctx.matrix_free(m)


@pytest.mark.parametrize("tag,kwargs,seed", [("dense", G.DENSE, G.DENSE_SEED), ("moe", G.MOE, G.MOE_SEED)])
def test_projections_match_reference_outputs(ctx, golden, tag, kwargs, seed):
    """CudaProjections.Apply / ApplyExpert against the committed outputs of the reference's
    GgufProjections (fp32 and double) on the same synthetic models: every stage, 1 and 3 tokens."""
    cfg = synth.ModelConfig(**kwargs)
    tensors = synth.build_model(cfg, seed)
    proj = CudaProjections(ctx, cfg, tensors)
    g = golden("projections")
    worst = 0.0
    for il in range(cfg.layers):
        stages = [Stage.kMixerOut, Stage.kFfnIn, Stage.kFfnDown,
                  Stage.kAttentionIn if cfg.is_full_attention(il) else Stage.kLinearIn]
        if cfg.is_moe:
            stages.append(Stage.kRouter)
        names = {Stage.kMixerOut: "mixer_out", Stage.kFfnIn: "ffn_in", Stage.kFfnDown: "ffn_down",
                 Stage.kAttentionIn: "attention_in", Stage.kLinearIn: "linear_in", Stage.kRouter: "router"}
        for stage in stages:
            for tokens in (1, 3):
                x = G.normal(1000 + 10 * il + tokens, tokens, stage_inputs(cfg, stage, il))
                got = proj.Apply(stage, il, x, tokens)
                for prec in ("f32", "f64"):
                    err = rel_l2(got, g[f"{tag}_{prec}_{names[stage]}_{il}_{tokens}"])
                    worst = max(worst, err)
                    assert err <= GEMV_TOL, (stage, il, tokens, prec, err)
        if cfg.is_moe:
            for expert in (0, 5, cfg.experts - 1):
                for stage, name in ((Stage.kExpertIn, "expert_in"), (Stage.kExpertDown, "expert_down")):
                    x = G.normal(2000 + expert, 2, stage_inputs(cfg, stage, il))
                    got = proj.ApplyExpert(stage, il, expert, x, 2)
                    assert rel_l2(got, g[f"{tag}_f32_{name}_{il}_e{expert}"]) <= GEMV_TOL
    got = proj.Apply(Stage.kLmHead, -1, G.normal(3000, 2, cfg.hidden), 2)
    assert rel_l2(got, g[f"{tag}_f32_lm_head"]) <= GEMV_TOL
    assert worst < 1e-5
    with pytest.raises(LookupError):
        proj.Apply(Stage.kExpertIn, 0, np.zeros(cfg.hidden, dtype=np.float32), 1)
    if not cfg.is_moe:
        with pytest.raises(LookupError):
            proj.ApplyExpert(Stage.kExpertIn, 0, 0, np.zeros(cfg.hidden, dtype=np.float32), 1)


def test_mtp_layer_projections_match_reference_outputs(ctx, golden):
    """A model with an MTP layer: Stage.kMtpIn (nextn.eh_proj over [embedding | hidden]) and the
    MTP layer's attention and FFN stages at layer index `layers`, against the committed outputs
    of the reference's GgufProjections (gguf_projections.cpp:114-125,205-207)."""
    cfg = synth.ModelConfig(**G.DENSE, mtp_layers=1)
    tensors = synth.build_model(cfg, G.MTP_SEED)
    proj = CudaProjections(ctx, cfg, tensors)
    g = golden("projections_mtp")
    il = cfg.layers
    names = {Stage.kMtpIn: "mtp_in", Stage.kAttentionIn: "attention_in", Stage.kMixerOut: "mixer_out",
             Stage.kFfnIn: "ffn_in", Stage.kFfnDown: "ffn_down"}
    assert stage_inputs(cfg, Stage.kMtpIn, il) == 2 * cfg.hidden
    for stage, name in names.items():
        for tokens in (1, 3):
            x = G.normal(8000 + tokens, tokens, stage_inputs(cfg, stage, il))
            got = proj.Apply(stage, il, x, tokens)
            for prec in ("f32", "f64"):
                err = rel_l2(got, g[f"{prec}_{name}_{tokens}"])
                assert err <= 1e-5, (stage, tokens, prec, err)
    # The decoder layers have no such stage; a model without the layer has no such layer.
    with pytest.raises(LookupError):
        proj.Apply(Stage.kMtpIn, 0, np.zeros(2 * cfg.hidden, dtype=np.float32), 1)
    plain = CudaProjections(ctx, synth.ModelConfig(**G.DENSE), synth.build_model(synth.ModelConfig(**G.DENSE), G.DENSE_SEED))
    with pytest.raises(IndexError):
        plain.Apply(Stage.kMtpIn, il, np.zeros(2 * cfg.hidden, dtype=np.float32), 1)


def test_projection_shape_check_at_construction(ctx):
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    bad = dict(tensors)
    t = bad["blk.0.ffn_down.weight"]
    bad["blk.0.ffn_down.weight"] = synth.Tensor((t.shape[1], t.shape[0]), t.ggml_type, t.data)
    with pytest.raises(RuntimeError, match="has shape"):
        CudaProjections(ctx, cfg, bad)


# ---- Gated DeltaNet -----------------------------------------------------------

def _delta_inputs(seed, hk, hv, dk):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((hk, dk)).astype(np.float32)
    k = rng.standard_normal((hk, dk)).astype(np.float32)
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    k /= np.linalg.norm(k, axis=1, keepdims=True)
    v = rng.standard_normal((hv, dk)).astype(np.float32)
    beta = (1.0 / (1.0 + np.exp(-rng.standard_normal(hv)))).astype(np.float32)
    g = rng.standard_normal(hv)
    decay = np.exp(-np.log1p(np.exp(g))).astype(np.float32)
    return q, k, v, decay, beta


@pytest.mark.parametrize("hk,hv,dk", [(16, 16, 128), (2, 4, 128), (1, 2, 64), (2, 2, 32)])
def test_delta_rule_matches_oracle_over_steps(ctx, oracle, hk, hv, dk):
    """8 sequences of ragged context lengths: each state is advanced by its own number of
    steps; state and output are checked after step 1, mid-way and after the last step."""
    dev = torch.device("cuda:0")
    nseq = 8
    lengths = np.random.default_rng(7).integers(1, 25, size=nseq)
    states = torch.zeros(nseq, hv, dk, dk, device=dev)
    ref_states = np.zeros((nseq, hv, dk, dk), dtype=np.float32)
    checked = 0
    for step in range(int(lengths.max())):
        live = [s for s in range(nseq) if step < lengths[s]]
        bufs, seqs = [], []
        for s in live:
            q, k, v, decay, beta = _delta_inputs(1000 * s + step, hk, hv, dk)
            d = {n: torch.from_numpy(a).to(dev) for n, a in
                 (("q", q), ("k", k), ("v", v), ("decay", decay), ("beta", beta))}
            d["y"] = torch.empty(hv, dk, device=dev)
            d["state"] = states[s]
            bufs.append((s, d, (q, k, v, decay, beta)))
            seqs.append(d)
        torch.cuda.synchronize()
        ctx.delta_rule_device(seqs, hk, hv, dk)
        ctx.synchronize()
        for s, d, (q, k, v, decay, beta) in bufs:
            want_y = np.empty((hv, dk), dtype=np.float32)
            for h in range(hv):
                ref_states[s, h], want_y[h] = oracle.delta_rule(ref_states[s, h], k[h % hk], q[h % hk], v[h],
                                                                float(decay[h]), float(beta[h]))
            if step in (0, lengths[s] // 2, lengths[s] - 1):
                assert rel_l2(d["y"].cpu().numpy(), want_y) <= DELTA_TOL
                assert rel_l2(states[s].cpu().numpy(), ref_states[s]) <= DELTA_TOL
                checked += 1
    assert checked >= nseq


def test_delta_rule_config3_context_lengths(ctx, oracle):
    """Config 3 as BASELINE states it: 16 heads of 128 x 128, 8 sequences whose states have seen
    a seeded draw of 1 to 4096 steps each. All heads run on the device; two heads of every
    sequence are followed on the CPU and compared after the first, a middle and the last step."""
    dev = torch.device("cuda:0")
    hk = hv = 16
    dk, nseq = 128, 8
    lengths = np.random.default_rng(33).integers(1, 4097, size=nseq)
    watched = (0, 9)
    gen = torch.Generator(device=dev).manual_seed(34)
    states = torch.zeros(nseq, hv, dk, dk, device=dev)
    y = torch.empty(nseq, hv, dk, device=dev)
    ref = np.zeros((nseq, len(watched), dk, dk), dtype=np.float32)
    worst = 0.0
    for step in range(int(lengths.max())):
        live = [s for s in range(nseq) if step < lengths[s]]
        n = len(live)
        q = torch.nn.functional.normalize(torch.randn(n, hk, dk, device=dev, generator=gen), dim=-1)
        k = torch.nn.functional.normalize(torch.randn(n, hk, dk, device=dev, generator=gen), dim=-1)
        v = torch.randn(n, hv, dk, device=dev, generator=gen)
        beta = torch.sigmoid(torch.randn(n, hv, device=dev, generator=gen))
        decay = torch.exp(-torch.nn.functional.softplus(torch.randn(n, hv, device=dev, generator=gen)))
        seqs = [{"q": q[i], "k": k[i], "v": v[i], "decay": decay[i], "beta": beta[i], "y": y[s], "state": states[s]}
                for i, s in enumerate(live)]
        torch.cuda.synchronize()
        ctx.delta_rule_device(seqs, hk, hv, dk)
        ctx.synchronize()
        qc, kc, vc, bc, dc = (t.cpu().numpy() for t in (q, k, v, beta, decay))
        for i, s in enumerate(live):
            for j, h in enumerate(watched):
                ref[s, j], want_y = oracle.delta_rule(ref[s, j], kc[i, h], qc[i, h], vc[i, h], float(dc[i, h]),
                                                      float(bc[i, h]))
                if step in (0, lengths[s] // 2, lengths[s] - 1):
                    err = max(rel_l2(y[s, h].cpu().numpy(), want_y), rel_l2(states[s, h].cpu().numpy(), ref[s, j]))
                    worst = max(worst, err)
                    assert err <= DELTA_TOL, (s, h, step, err)
    assert worst > 0.0


def test_delta_rule_alternate_output_leaves_state(ctx, oracle):
    dev = torch.device("cuda:0")
    hk = hv = 4
    dk = 128
    state = torch.randn(hv, dk, dk, device=dev, generator=torch.Generator(device=dev).manual_seed(3))
    before = state.clone()
    out = torch.zeros_like(state)
    q, k, v, decay, beta = _delta_inputs(5, hk, hv, dk)
    d = {n: torch.from_numpy(a).to(dev) for n, a in (("q", q), ("k", k), ("v", v), ("decay", decay), ("beta", beta))}
    d.update(state=state, state_out=out, y=torch.empty(hv, dk, device=dev))
    torch.cuda.synchronize()
    ctx.delta_rule_device([d], hk, hv, dk)
    ctx.synchronize()
    assert torch.equal(state, before)
    for h in range(hv):
        want, want_y = oracle.delta_rule(before[h].cpu().numpy(), k[h], q[h], v[h], float(decay[h]), float(beta[h]))
        assert rel_l2(out[h].cpu().numpy(), want) <= DELTA_TOL
        assert rel_l2(d["y"][h].cpu().numpy(), want_y) <= DELTA_TOL


def test_deltanet_linear_matches_reference_outputs(ctx, golden):
    """Mixer::Linear over 12 steps with speculative states kept or dropped, against the
    committed outputs of the reference (tests/golden/deltanet.npz)."""
    dev = torch.device("cuda:0")
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    mixer = CudaMixer(ctx, cfg, tensors)
    g = golden("deltanet")
    width = cfg.conv_channels + cfg.value_dim + 2 * cfg.linear_value_heads
    conv = [torch.zeros(mixer.conv_values(), device=dev), torch.zeros(mixer.conv_values(), device=dev)]
    ssm = torch.zeros(mixer.ssm_values(), device=dev)
    spec = torch.zeros_like(ssm)
    y = torch.empty(cfg.value_dim, device=dev)
    cur = 0
    for step in range(12):
        x_in = torch.from_numpy(G.normal(4000 + step, width)).to(dev)
        speculative = step % 4 == 3
        torch.cuda.synchronize()
        mixer.Linear(0, [{"in": x_in, "conv_in": conv[cur], "conv_out": conv[1 - cur], "ssm": ssm,
                          "ssm_out": spec if speculative else None, "y": y}])
        ctx.synchronize()
        cur = 1 - cur
        assert rel_l2(y.cpu().numpy(), g["linear_y"][step]) <= DELTA_TOL, step
        if speculative:
            assert rel_l2(spec.cpu().numpy()[::G.SAMPLE], g[f"linear_spec_{step}"]) <= DELTA_TOL
            if step % 8 == 3:
                ssm.copy_(spec)
    assert np.array_equal(bits(conv[cur].cpu().numpy()), bits(g["linear_conv"]))   # copies of inputs: exact
    assert rel_l2(ssm.cpu().numpy(), g["linear_ssm"]) <= DELTA_TOL


def test_deltanet_run_matches_reference_outputs(ctx, golden):
    """DeltaNetStep::Run (1 or 2 tokens, gates from the residual stream, draft state and saved
    window) over 6 steps, against the committed outputs of the reference's fused step; the draft
    is kept on even steps and dropped on odd ones, as when the goldens were made."""
    dev = torch.device("cuda:0")
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    mixer = CudaMixer(ctx, cfg, tensors)
    g = golden("deltanet")
    rows = cfg.conv_channels + cfg.value_dim
    width = rows + 2 * cfg.linear_value_heads
    conv = torch.zeros(mixer.conv_values(), device=dev)
    ssm = torch.zeros(mixer.ssm_values(), device=dev)
    for step in range(6):
        count = 1 if step % 3 == 0 else 2
        x_in = torch.from_numpy(G.normal(5000 + step, count, width)).to(dev)
        x_in[:, rows:] = float("nan")            # the alpha / beta slots of the rows are not read
        h = torch.from_numpy(4.0 * G.normal(6000 + step, count, cfg.hidden)).to(dev)
        conv_out, saved = torch.zeros_like(conv), torch.zeros_like(conv)
        spec = torch.zeros_like(ssm)
        y = torch.empty(count, cfg.value_dim, device=dev)
        torch.cuda.synchronize()
        mixer.Run(0, [{"n_tokens": count, "in": x_in, "h": h, "conv_in": conv, "conv_out": conv_out,
                       "conv_saved": saved if count == 2 else None, "ssm": ssm,
                       "ssm_spec": spec if count == 2 else None, "y": y}])
        ctx.synchronize()
        assert rel_l2(y.cpu().numpy(), g[f"fused_y_{step}"]) <= DELTA_TOL, step
        conv = conv_out
        if count == 2:
            assert rel_l2(spec.cpu().numpy()[::G.SAMPLE], g[f"fused_spec_{step}"]) <= DELTA_TOL
            assert np.array_equal(bits(saved.cpu().numpy()[::7]), bits(g[f"fused_saved_{step}"]))
            if step % 2 == 0:
                ssm = spec.clone()
            else:
                conv = saved.clone()
    assert np.array_equal(bits(conv.cpu().numpy()), bits(g["fused_conv"]))
    assert rel_l2(ssm.cpu().numpy(), g["fused_ssm"]) <= DELTA_TOL


def test_deltanet_run_ragged_token_counts(ctx):
    """Sequences of 1 to 4 tokens in one call equal the same tokens one call at a time: the
    tokens before the last advance the state, the last of several is a draft."""
    dev = torch.device("cuda:0")
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    mixer = CudaMixer(ctx, cfg, tensors)
    width = cfg.conv_channels + cfg.value_dim + 2 * cfg.linear_value_heads
    counts = [3, 1, 4, 2, 1]
    gen = torch.Generator(device=dev).manual_seed(10)
    z = lambda *shape: torch.zeros(*shape, device=dev)
    x_in = [torch.randn(n, width, device=dev, generator=gen) for n in counts]
    h = [torch.randn(n, cfg.hidden, device=dev, generator=gen) * 3 for n in counts]
    conv0 = [torch.randn(mixer.conv_values(), device=dev, generator=gen) for _ in counts]
    ssm0 = [torch.randn(mixer.ssm_values(), device=dev, generator=gen) * 0.1 for _ in counts]

    def seq(s, n, x, hh, conv_in, ssm):
        return {"n_tokens": n, "in": x, "h": hh, "conv_in": conv_in, "conv_out": z(mixer.conv_values()),
                "conv_saved": z(mixer.conv_values()), "ssm": ssm, "ssm_spec": z(mixer.ssm_values()),
                "y": z(n, cfg.value_dim)}
    together = [seq(s, n, x_in[s], h[s], conv0[s], ssm0[s].clone()) for s, n in enumerate(counts)]
    torch.cuda.synchronize()
    mixer.Run(0, together)
    ctx.synchronize()
    for s, n in enumerate(counts):
        conv, ssm = conv0[s], ssm0[s].clone()
        for t in range(n):
            last_of_many = n >= 2 and t == n - 1
            one = seq(s, 1, x_in[s][t:t + 1], h[s][t:t + 1], conv, ssm)
            before = ssm.clone()
            torch.cuda.synchronize()
            mixer.Run(0, [one])
            ctx.synchronize()
            assert torch.equal(one["y"][0], together[s]["y"][t]), (s, t)
            if last_of_many:
                assert torch.equal(conv, together[s]["conv_saved"])
                assert torch.equal(ssm, together[s]["ssm_spec"])       # the draft state
                assert torch.equal(before, together[s]["ssm"])         # ssm kept the state before it
            conv = one["conv_out"]
        assert torch.equal(conv, together[s]["conv_out"])
        if n == 1:
            assert torch.equal(ssm, together[s]["ssm"])


def test_deltanet_linear_batched_sequences(ctx, oracle):
    """Several sequences in one launch equal the same sequences one by one."""
    dev = torch.device("cuda:0")
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    mixer = CudaMixer(ctx, cfg, tensors)
    width = cfg.conv_channels + cfg.value_dim + 2 * cfg.linear_value_heads
    nseq = 19                                    # more than one launch's worth of descriptors
    gen = torch.Generator(device=dev).manual_seed(9)
    x_in = torch.randn(nseq, width, device=dev, generator=gen)
    conv_in = torch.randn(nseq, mixer.conv_values(), device=dev, generator=gen)
    ssm0 = torch.randn(nseq, mixer.ssm_values(), device=dev, generator=gen) * 0.1

    def run(batched):
        conv_out = torch.zeros_like(conv_in)
        ssm = ssm0.clone()
        y = torch.zeros(nseq, cfg.value_dim, device=dev)
        seqs = [{"in": x_in[s], "conv_in": conv_in[s], "conv_out": conv_out[s], "ssm": ssm[s], "y": y[s]}
                for s in range(nseq)]
        torch.cuda.synchronize()
        if batched:
            mixer.Linear(0, seqs)
        else:
            for s in seqs:
                mixer.Linear(0, [s])
        ctx.synchronize()
        return conv_out, ssm, y
    a, b = run(True), run(False)
    for got, want in zip(a, b):
        assert torch.equal(got, want)
    # And against the oracle for one of them.
    from tests.test_oracle import _deltanet_cfg, _deltanet_weights
    s = 7
    conv = conv_in[s].cpu().numpy().copy()
    ssm = ssm0[s].cpu().numpy().copy()
    want_y, _ = oracle.deltanet_linear(_deltanet_cfg(cfg), _deltanet_weights(cfg, tensors, 0),
                                       x_in[s].cpu().numpy(), conv, ssm)
    assert rel_l2(a[2][s].cpu().numpy(), want_y) <= DELTA_TOL
    assert rel_l2(a[1][s].cpu().numpy(), ssm) <= DELTA_TOL
    assert np.array_equal(bits(a[0][s].cpu().numpy()), bits(conv))


# ---- the decode step ------------------------------------------------------------

STEP_TOL = 2e-3      # logits relative L2: the reference's own bound between its decoder and its
                     # oracle (tests/models/qwen35_2b/decoder_test.cpp:30-31)


@pytest.mark.parametrize("use_graph", [False, True])
def test_decoder_step_matches_reference_logits(ctx, golden, use_graph):
    """CudaDecoder.Step against the committed logits of the reference's Decoder::Step on the
    same synthetic dense model (3 DeltaNet layers + 1 attention layer), 8 tokens."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    proj = CudaProjections(ctx, cfg, tensors)
    dec = CudaDecoder(proj, tensors, max_positions=64, use_graph=use_graph)
    g = golden("decoder")
    tokens = [int(t) for t in g["decoder_dense_tokens"]]
    worst = 0.0
    for i, tok in enumerate(tokens):
        logits = dec.Step(tok)
        want = g["decoder_dense_logits"][i]
        err = rel_l2(logits, want)
        worst = max(worst, err)
        assert err <= STEP_TOL, (i, err)
        assert int(np.argmax(logits)) == int(np.argmax(want))
    assert worst < 1e-4
    assert dec.position == len(tokens)
    # A second sequence after Reset reproduces the first.
    dec.Reset()
    again = dec.Step(tokens[0])
    assert rel_l2(again, g["decoder_dense_logits"][0]) <= STEP_TOL
    from gufo_npu_b200._capi import GufoCudaError
    with pytest.raises(GufoCudaError):
        dec.Step(cfg.vocab)
    dec.close()


def check_pair_steps(dec, cfg, tokens, want_logits):
    """Walks `tokens` with two-token steps whose drafts are kept or rolled back
    (NpuDecoder::Step / Resolve, src/models/qwen35_2b/npu_decoder.hpp:57-68); every row of
    logits must be the one-token decoder's at that position (`want_logits`)."""
    def check(row, i):
        err = rel_l2(row, want_logits[i])
        assert err <= STEP_TOL, (i, err)
        assert int(np.argmax(row)) == int(np.argmax(want_logits[i]))
        return err
    worst = 0.0
    wrong = lambda tok: (tok + 7) % cfg.vocab
    # (0, 1) kept; (2, wrong) rolled back; (3, 4) kept; 5 alone; (6, wrong) rolled back; 7 alone.
    both = dec.StepTokens(tokens[0:2])
    assert both.shape == (2, cfg.vocab)
    worst = max(worst, check(both[0], 0), check(both[1], 1))
    with pytest.raises(Exception):
        dec.Step(tokens[2])              # a pair awaits Resolve
    dec.Resolve(True)
    assert dec.position == 2
    both = dec.StepTokens([tokens[2], wrong(tokens[3])])
    worst = max(worst, check(both[0], 2))
    dec.Resolve(False)
    assert dec.position == 3
    both = dec.StepTokens(tokens[3:5])
    worst = max(worst, check(both[0], 3), check(both[1], 4))
    dec.Resolve(True)
    worst = max(worst, check(dec.Step(tokens[5]), 5))
    both = dec.StepTokens([tokens[6], wrong(tokens[7])])
    worst = max(worst, check(both[0], 6))
    dec.Resolve(False)
    worst = max(worst, check(dec.StepTokens([tokens[7]])[0], 7))
    assert dec.position == 8
    with pytest.raises(Exception):
        dec.Resolve(True)                # nothing to resolve after a one-token step
    return worst


@pytest.mark.parametrize("use_graph", [False, True])
def test_decoder_pair_steps_and_resolve(ctx, golden, use_graph):
    """Two-token steps with kept and rolled-back drafts against the committed logits of the
    reference's Decoder::Step; three passes, so that the replayed graphs are covered."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    dec = CudaDecoder(CudaProjections(ctx, cfg, tensors), tensors, max_positions=64, use_graph=use_graph)
    g = golden("decoder")
    tokens = [int(t) for t in g["decoder_dense_tokens"]]
    for _ in range(3):
        dec.Reset()
        assert check_pair_steps(dec, cfg, tokens, g["decoder_dense_logits"]) < 1e-4
    # Prompt passes without logits, then the final residual and the next token's logits.
    dec.Reset()
    assert dec.StepTokens(tokens[0:2], logits=False) is None
    dec.Resolve(True)
    assert dec.StepTokens(tokens[2:3], logits=False) is None
    hidden_quiet = dec.hidden(0)
    assert rel_l2(dec.Step(tokens[3]), g["decoder_dense_logits"][3]) <= STEP_TOL
    dec.Reset()
    for tok in tokens[:3]:
        dec.Step(tok)
    assert rel_l2(hidden_quiet, dec.hidden(0)) <= 1e-4
    pair = CudaDecoder(CudaProjections(ctx, cfg, tensors), tensors, max_positions=64, use_graph=False)
    pair.StepTokens(tokens[0:2])
    pair.Resolve(True)
    pair.StepTokens(tokens[2:4])
    assert rel_l2(pair.hidden(0), hidden_quiet) <= 1e-4
    pair.close()
    dec.close()


def test_decoder_steps_enqueued_without_waits_keep_their_tokens(ctx, golden):
    """Steps that leave their logits on the device return before the device has run them; each
    must still see its own token id (the host side stages ids in slots it reuses only after
    the copy that read them has run)."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    dec = CudaDecoder(CudaProjections(ctx, cfg, tensors), tensors, max_positions=64, use_graph=True)
    g = golden("decoder")
    tokens = [int(t) for t in g["decoder_dense_tokens"]]
    for _ in range(4):
        dec.Reset()
        for tok in tokens[:7]:
            dec.step_device(tok)
        assert rel_l2(dec.Step(tokens[7]), g["decoder_dense_logits"][7]) <= STEP_TOL
    dec.close()


def test_decoder_cache_capacity(ctx):
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    dec = CudaDecoder(CudaProjections(ctx, cfg, tensors), tensors, max_positions=3, use_graph=False)
    for tok in (1, 2, 3):
        dec.Step(tok)
    from gufo_npu_b200._capi import GufoCudaError
    with pytest.raises(GufoCudaError) as e:
        dec.Step(4)
    assert e.value.status == 7
    dec.close()


def test_row_split_decoder_single_rank_matches_reference_logits(golden):
    """The tensor-parallel decode loop (host-side steps over the C ABI's small operations) with
    one rank: same logits as the reference's Decoder::Step, eager and graph-replayed."""
    from gufo_npu_b200.tp import TpDecoder
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        c = Context(0, stream.cuda_stream)
        cfg = synth.ModelConfig(**G.DENSE)
        tensors = synth.build_model(cfg, G.DENSE_SEED)
        dec = TpDecoder(c, cfg, tensors, rank=0, world=1, max_positions=32)
        g = golden("decoder")
        for i, tok in enumerate(int(t) for t in g["decoder_dense_tokens"]):
            logits = dec.step(tok, stream).cpu().numpy()
            assert rel_l2(logits, g["decoder_dense_logits"][i]) <= STEP_TOL, i
        assert dec.graphs and dec.kernels_per_step > 0
    torch.cuda.synchronize()
    c.close()


@pytest.mark.parametrize("tag,kwargs,seed", [("dense", G.DENSE, G.DENSE_SEED), ("moe", G.MOE, G.MOE_SEED),
                                             ("mtp", dict(G.DENSE, mtp_layers=1), G.MTP_SEED)])
def test_reference_decoder_with_cuda_adapter(tmp_path, tag, kwargs, seed):
    """Drop-in at step level: the reference's own Decoder::Step (its mixers, norms, routing)
    with the C++ adapter over this library plugged in behind qwen35::Projections, against the
    same decoder over its GgufProjections. Dense and MoE (ApplyExpert through Route) models.
    Runs the binary oracle/Makefile builds where the reference tree is mounted."""
    import os
    import subprocess
    binary = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref",
                          "adapter_parity")
    if not os.path.exists(binary):
        pytest.skip("oracle/_ref/adapter_parity was not built (no reference tree here)")
    cfg = synth.ModelConfig(**kwargs)
    image = synth.to_gguf(cfg, synth.build_model(cfg, seed))
    path = tmp_path / f"{tag}.gguf"
    image.tofile(path)
    run = subprocess.run([binary, str(path), "6"], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "PASS" in run.stdout


# ---- the other row formats of real files: Q8_0, Q5_K (products and dequantization), F16, BF16 ----

@pytest.mark.parametrize("name,ggml_type", [("Q5_K", Q.GGML_Q5_K), ("Q8_0", Q.GGML_Q8_0), ("BF16", Q.GGML_BF16)])
def test_dequantize_other_reference_fixtures_bit_exact(ctx, golden, name, ggml_type):
    raw = np.fromfile(golden.path("quant", name + ".bin"), dtype=np.uint8)
    want = np.fromfile(golden.path("quant", name + ".f32"), dtype=np.float32)
    m = ctx.matrix_upload(ggml_type, raw, 1, want.size)
    got = ctx.dequantize(m, 0, 1, want.size)
    assert np.array_equal(bits(got.ravel()), bits(want))
    ctx.matrix_free(m)


@pytest.mark.parametrize("ggml_type", [Q.GGML_Q5_K, Q.GGML_Q8_0, Q.GGML_F16, Q.GGML_BF16])
def test_dequantize_other_types_match_oracle_bit_exact(ctx, oracle, ggml_type):
    rows, cols = 19, 768
    if ggml_type in (Q.GGML_F16, Q.GGML_BF16):
        # Every 16-bit pattern once (NaN payloads included: compared as bits).
        raw = np.arange(65536, dtype=np.uint16).view(np.uint8)
        rows, cols = 64, 1024
    else:
        raw = Q.random_blocks(ggml_type, rows, cols, seed=23).numpy()
    m = ctx.matrix_upload(ggml_type, raw, rows, cols)
    got = ctx.dequantize(m, 0, rows, cols)
    want = oracle.dequantize(ggml_type, raw, rows * cols).reshape(rows, cols)
    assert np.array_equal(bits(got), bits(want))
    ctx.matrix_free(m)


@pytest.mark.parametrize("ggml_type", [Q.GGML_Q5_K, Q.GGML_Q8_0])
@pytest.mark.parametrize("tokens", [1, 3, 9])
def test_gemv_other_types_match_oracle(ctx, oracle, ggml_type, tokens):
    """Q5_K and Q8_0 rows on the general kernel against the oracle's fused row dots, alone and
    stacked beside a Q4_K part."""
    rows, cols = 77, 1024
    raw = Q.random_blocks(ggml_type, rows, cols, seed=24).numpy()
    other = Q.random_blocks(Q.GGML_Q4_K, 40, cols, seed=25).numpy()
    x = G.normal(26 + tokens, tokens, cols)
    m = ctx.matrix_upload(ggml_type, raw, rows, cols)
    mo = ctx.matrix_upload(Q.GGML_Q4_K, other, 40, cols)
    got = ctx.matmul([(mo, 0, 40), (m, 5, 70)], x, tokens, 110)
    want = oracle.matmul([(other, Q.GGML_Q4_K, 0, 40), (raw, ggml_type, 5, 70)], cols, x)
    exact = oracle.matmul([(other, Q.GGML_Q4_K, 0, 40), (raw, ggml_type, 5, 70)], cols, x, exact=True)
    assert rel_l2(got, want) <= 1e-5
    assert rel_l2(got, exact) <= 1e-5
    ctx.matrix_free(m)
    ctx.matrix_free(mo)


def test_half_rows_are_not_multiplied(ctx):
    from gufo_npu_b200._capi import GufoCudaError
    raw = np.zeros(8 * 256 * 2, dtype=np.uint8)
    m = ctx.matrix_upload(Q.GGML_F16, raw, 8, 256)
    with pytest.raises(GufoCudaError) as e:
        ctx.matmul([(m, 0, 8)], np.zeros((1, 256), dtype=np.float32), 1, 8)
    assert e.value.status == 3
    ctx.matrix_free(m)
