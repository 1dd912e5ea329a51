"""GPU parity of the routed-expert path: Route / SharedExpertScale on the device, the grouped
expert FFN, the weighted sum, and Decoder::Step on a MoE model. Indices are compared exactly;
weights to one fp32 ulp (the device's double exp may differ from the host's in the last bit);
products <= 1e-3 relative L2."""
import numpy as np
import pytest
import torch

from gufo_npu_b200 import _capi
from gufo_npu_b200 import quantize as Q
from gufo_npu_b200 import synth
from gufo_npu_b200.backend import Context, CudaDecoder, CudaMoe, CudaProjections, Stage
from tests.golden import make_golden as G

pytestmark = pytest.mark.gpu

GEMV_TOL = 1e-3
STEP_TOL = 2e-3


def rel_l2(got, want):
    got = np.asarray(got, dtype=np.float64).ravel()
    want = np.asarray(want, dtype=np.float64).ravel()
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


@pytest.fixture(scope="module", params=["default", "general"])
def ctx(request):
    c = Context(0)
    c.set_option("general_gemv", int(request.param == "general"))
    yield c
    c.close()


def _route(ctx, rows: np.ndarray, experts: int, k: int):
    tokens, stride = rows.shape
    dev = torch.device("cuda:0")
    router = torch.from_numpy(rows).to(dev)
    chosen = torch.full((tokens, k), -7, dtype=torch.int32, device=dev)
    weights = torch.zeros(tokens, k, dtype=torch.float32, device=dev)
    scale = torch.zeros(tokens, dtype=torch.float32, device=dev)
    ctx.route_device(router, stride, tokens, experts, k, chosen, weights, scale if stride > experts else None)
    ctx.synchronize()
    return chosen.cpu().numpy(), weights.cpu().numpy(), scale.cpu().numpy()


def test_route_matches_reference_goldens(ctx, golden, oracle):
    """The committed outputs of the reference's Route on 8 rows of 256 logits (one exact tie,
    one all-equal row), k = 8, plus its SharedExpertScale."""
    g = golden("routing")
    logits = g["route_logits"]
    shared = np.array([-30.0, -1.5, 0.0, 0.25, 12.0, 3.0, -0.75, 88.0], dtype=np.float32)
    rows = np.concatenate([logits, shared[:, None]], axis=1).astype(np.float32)
    chosen, weights, scale = _route(ctx, rows, 256, 8)
    assert np.array_equal(chosen, g["route_chosen"])
    np.testing.assert_allclose(weights, g["route_weights"], rtol=1.2e-7, atol=0)
    np.testing.assert_allclose(scale[:5], g["shared_scale"], rtol=1.2e-7, atol=0)
    want = np.array([oracle.shared_expert_scale(float(v)) for v in shared], dtype=np.float32)
    np.testing.assert_allclose(scale, want, rtol=1.2e-7, atol=0)


def test_route_edge_cases_match_oracle(ctx, oracle):
    """Underflowing probabilities (ties at zero go to the lower id), huge logits, k = 1, k =
    experts, an expert count that is not a multiple of the block size."""
    rng = np.random.default_rng(5)
    cases = []
    a = rng.standard_normal((3, 100)).astype(np.float32)
    a[0, 10:] = -2000.0          # only ten live experts for k = 16
    a[1] *= 300.0
    a[2, ::2] = a[2, 1::2]       # pairs of equal logits
    cases.append((a, 100, 16))
    cases.append((rng.standard_normal((2, 7)).astype(np.float32), 7, 7))
    cases.append((rng.standard_normal((2, 1000)).astype(np.float32) * 5, 1000, 1))
    for rows, experts, k in cases:
        chosen, weights, _ = _route(ctx, rows, experts, k)
        for t in range(rows.shape[0]):
            want_c, want_w = oracle.route(rows[t], k)
            assert np.array_equal(chosen[t], want_c), (experts, k, t)
            np.testing.assert_allclose(weights[t], want_w, rtol=1.2e-7, atol=1e-45)


def test_route_rejects_bad_counts(ctx):
    rows = np.zeros((1, 8), dtype=np.float32)
    with pytest.raises(_capi.GufoCudaError):
        _route(ctx, rows, 8, 9)


def _moe_model(ctx, **over):
    kwargs = dict(G.MOE)
    kwargs.update(over)
    cfg = synth.ModelConfig(**kwargs)
    tensors = synth.build_model(cfg, G.MOE_SEED)
    return cfg, tensors, CudaProjections(ctx, cfg, tensors)


@pytest.mark.parametrize("proj_type", [Q.GGML_Q4_K, Q.GGML_Q6_K])
def test_grouped_expert_ffn_matches_per_expert_products(ctx, proj_type):
    """The two grouped launches against ApplyExpert(kExpertIn) -> SwiGLU -> ApplyExpert(kExpertDown)
    one expert at a time (itself pinned to the reference's outputs); a skipped pair stays untouched."""
    cfg, _, proj = _moe_model(ctx, proj_type=proj_type)
    dev = torch.device("cuda:0")
    moe = CudaMoe(proj, max_tokens=2)
    ids = [3, -1, cfg.experts - 1, 0, 3]
    x = G.normal(91, len(ids), cfg.hidden)
    for shared_input in (False, True):
        xd = torch.from_numpy(x).to(dev)
        ffn = torch.empty(len(ids), 2 * cfg.expert_ffn, device=dev)
        act = torch.empty(len(ids), cfg.expert_ffn, device=dev)
        y = torch.full((len(ids), cfg.hidden), 7.0, device=dev)
        ctx.expert_ffn_device(moe.banks[1], torch.tensor(ids, dtype=torch.int32, device=dev), len(ids), xd,
                              0 if shared_input else cfg.hidden, ffn, act, y)
        ctx.synchronize()
        got = y.cpu().numpy()
        for p, e in enumerate(ids):
            if e < 0:
                assert np.all(got[p] == 7.0)
                continue
            xin = x[0] if shared_input else x[p]
            mid = proj.ApplyExpert(Stage.kExpertIn, 1, e, xin, 1)[0]
            gate, up = mid[:cfg.expert_ffn], mid[cfg.expert_ffn:]
            act_host = (gate / (1.0 + np.exp(-gate.astype(np.float64)))).astype(np.float32) * up
            want = proj.ApplyExpert(Stage.kExpertDown, 1, e, act_host, 1)[0]
            assert rel_l2(got[p], want) <= 1e-5, (p, e)


def test_moe_ffn_matches_oracle_route_and_per_expert_sum(ctx, oracle):
    """CudaMoe.MoeFfn for 3 tokens against Decoder::MoeFfn's recipe on the host: oracle Route on the
    same router outputs, experts in slot order, fp32 sum onto the scaled shared output."""
    cfg, _, proj = _moe_model(ctx)
    dev = torch.device("cuda:0")
    tokens, k = 3, cfg.experts_used
    normed = G.normal(92, tokens, cfg.hidden)
    shared = G.normal(93, tokens, cfg.hidden)
    nd, sd = torch.from_numpy(normed).to(dev), torch.from_numpy(shared).to(dev)
    out = torch.empty(tokens, cfg.hidden, device=dev)
    moe = CudaMoe(proj, max_tokens=4)
    moe.MoeFfn(0, nd, sd, tokens, out)
    ctx.synchronize()
    got = out.cpu().numpy()
    router = proj.Apply(Stage.kRouter, 0, normed, tokens)
    for t in range(tokens):
        chosen, weights = oracle.route(router[t, :cfg.experts], k)
        assert np.array_equal(moe.chosen[t].cpu().numpy(), chosen)
        want = shared[t] * np.float32(oracle.shared_expert_scale(float(router[t, cfg.experts])))
        for slot in range(k):
            mid = proj.ApplyExpert(Stage.kExpertIn, 0, int(chosen[slot]), normed[t], 1)[0]
            gate, up = mid[:cfg.expert_ffn], mid[cfg.expert_ffn:]
            act = (gate / (1.0 + np.exp(-gate.astype(np.float64)))).astype(np.float32) * up
            want = want + weights[slot] * proj.ApplyExpert(Stage.kExpertDown, 0, int(chosen[slot]), act, 1)[0]
        assert rel_l2(got[t], want) <= 1e-5, t


def test_expert_parallel_halves_add_up_to_the_whole():
    """Expert parallelism on one device: two CudaMoe, each holding half of the experts, compute
    their own pairs; the rows add up (only zeros are added) to the single-device rows, bit for
    bit. torch ops sit between the kernels here, so the context shares torch's stream."""
    stream = torch.cuda.Stream()
    ctx = Context(0, stream.cuda_stream)
    with torch.cuda.stream(stream):
        cfg, _, proj = _moe_model(ctx)
        dev = torch.device("cuda:0")
        tokens = 3
        nd = torch.from_numpy(G.normal(92, tokens, cfg.hidden)).to(dev)
        whole = CudaMoe(proj, max_tokens=4)
        whole.route(0, nd, tokens)
        whole.experts(0, nd, tokens)
        half = cfg.experts // 2
        parts = []
        for first in (0, half):
            part = CudaMoe(proj, max_tokens=4, expert_range=(first, half))
            part.route(0, nd, tokens)
            part.experts(0, nd, tokens)
            parts.append(part)
        total = parts[0].expert_out + parts[1].expert_out
        stream.synchronize()
        assert torch.equal(total[:tokens], whole.expert_out[:tokens])
        assert float(whole.expert_out[:tokens].abs().sum()) > 0
    ctx.close()


@pytest.mark.parametrize("use_graph", [False, True])
def test_moe_decoder_step_matches_reference_logits(ctx, golden, use_graph):
    """CudaDecoder.Step on the synthetic MoE model (router, top-k and experts on the device)
    against the committed logits of the reference's Decoder::Step, 8 tokens."""
    cfg, tensors, proj = _moe_model(ctx)
    dec = CudaDecoder(proj, tensors, max_positions=64, use_graph=use_graph)
    g = golden("decoder")
    tokens = [int(t) for t in g["decoder_moe_tokens"]]
    worst = 0.0
    for i, tok in enumerate(tokens):
        logits = dec.Step(tok)
        want = g["decoder_moe_logits"][i]
        err = rel_l2(logits, want)
        worst = max(worst, err)
        assert err <= STEP_TOL, (i, err)
        assert int(np.argmax(logits)) == int(np.argmax(want))
    assert worst < 1e-4
    dec.close()


@pytest.mark.parametrize("use_graph", [False, True])
def test_moe_decoder_pair_steps_and_resolve(ctx, golden, use_graph):
    """Two-token steps on the MoE model: both rows route on the device and run their experts in
    one grouped launch; kept and rolled-back drafts against the reference's one-token logits."""
    from tests.test_gpu_parity import check_pair_steps
    cfg, tensors, proj = _moe_model(ctx)
    dec = CudaDecoder(proj, tensors, max_positions=64, use_graph=use_graph)
    g = golden("decoder")
    tokens = [int(t) for t in g["decoder_moe_tokens"]]
    for _ in range(3):
        dec.Reset()
        assert check_pair_steps(dec, cfg, tokens, g["decoder_moe_logits"]) < 1e-4
    dec.close()


def test_config4_shaped_experts(ctx, oracle):
    """Config-4 shapes (hidden 2048, expert FFN 512, Q4_K, top-8) on a bank of 32 experts: the
    grouped path against the oracle's fused row dots for two of the chosen experts."""
    hidden, ef, experts, k = 2048, 512, 32, 8
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(31)
    mats = {}
    raws = {}
    for name, rows, cols in (("gate", ef, hidden), ("up", ef, hidden), ("down", hidden, ef)):
        w = torch.randn(experts * rows, cols, generator=gen) * 0.02
        raw = Q.quantize(Q.GGML_Q4_K, w).numpy()
        raws[name] = raw.reshape(experts * rows, -1)
        mats[name] = ctx.matrix_upload(Q.GGML_Q4_K, raw, experts * rows, cols)
    bank = _capi.ExpertBank(mats["gate"], mats["up"], mats["down"], experts, ef, hidden)
    logits = G.normal(32, 1, experts)
    chosen, weights, _ = _route(ctx, logits, experts, k)
    x = G.normal(33, hidden)
    xd = torch.from_numpy(x).to(dev)
    ffn = torch.empty(k, 2 * ef, device=dev)
    act = torch.empty(k, ef, device=dev)
    y = torch.empty(k, hidden, device=dev)
    ctx.expert_ffn_device(bank, torch.from_numpy(chosen[0]).to(dev), k, xd, 0, ffn, act, y)
    ctx.synchronize()
    got = y.cpu().numpy()
    for slot in (0, k - 1):
        e = int(chosen[0, slot])
        mid = oracle.matmul([(raws["gate"], Q.GGML_Q4_K, e * ef, ef), (raws["up"], Q.GGML_Q4_K, e * ef, ef)],
                            hidden, x)[0]
        gate, up = mid[:ef], mid[ef:]
        a = (gate / (1.0 + np.exp(-gate.astype(np.float64)))).astype(np.float32) * up
        want = oracle.matmul([(raws["down"], Q.GGML_Q4_K, e * hidden, hidden)], ef, a)[0]
        assert rel_l2(got[slot], want) <= GEMV_TOL, slot
    for m in mats.values():
        ctx.matrix_free(m)


@pytest.mark.parametrize("tokens", [1, 3])
def test_moe_ffn_in_one_call_equals_expert_ffn_then_combine(ctx, tokens):
    """gufo_cuda_moe_ffn_device (config-4 shapes: the down rows of a token's experts and the
    weighted sum in one launch) against gufo_cuda_expert_ffn_device + gufo_cuda_moe_combine_device
    on the same routing, one slot of the second token's ids set to -1 (adds nothing)."""
    hidden, ef, experts, k = 2048, 512, 32, 8
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(41)
    mats = {}
    for name, rows, cols in (("gate", ef, hidden), ("up", ef, hidden), ("down", hidden, ef)):
        w = torch.randn(experts * rows, cols, generator=gen) * 0.02
        raw = Q.quantize(Q.GGML_Q4_K, w).numpy()
        mats[name] = ctx.matrix_upload(Q.GGML_Q4_K, raw, experts * rows, cols)
    bank = _capi.ExpertBank(mats["gate"], mats["up"], mats["down"], experts, ef, hidden)
    logits = torch.from_numpy(G.normal(42, tokens, experts + 1)).to(dev)
    chosen = torch.empty(tokens, k, dtype=torch.int32, device=dev)
    weights = torch.empty(tokens, k, device=dev)
    scale = torch.empty(tokens, device=dev)
    ctx.route_device(logits, experts + 1, tokens, experts, k, chosen, weights, scale)
    ctx.synchronize()
    if tokens > 1:
        chosen[1, 2] = -1
        torch.cuda.synchronize()
    x = torch.from_numpy(G.normal(43, tokens, hidden)).to(dev)
    shared = torch.from_numpy(G.normal(44, tokens, hidden)).to(dev)
    ffn = torch.empty(tokens * k, 2 * ef, device=dev)
    act = torch.empty(tokens * k, ef, device=dev)
    rows_out = torch.zeros(tokens, k, hidden, device=dev)   # a skipped pair's rows stay zero
    want = torch.empty(tokens, hidden, device=dev)
    ctx.expert_ffn_device(bank, chosen, tokens * k, x, hidden, ffn, act, rows_out, pairs_per_input=k)
    ctx.moe_combine_device(shared, scale, weights, rows_out, tokens, k, hidden, want)
    got = torch.empty(tokens, hidden, device=dev)
    ctx.moe_ffn_device(bank, chosen, weights, scale, tokens, k, x, hidden, shared, ffn, act, rows_out, got)
    ctx.synchronize()
    assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= 1e-6
    # In place over the shared expert's output, as the decoder calls it.
    ctx.moe_ffn_device(bank, chosen, weights, scale, tokens, k, x, hidden, shared, ffn, act, rows_out, shared)
    ctx.synchronize()
    assert rel_l2(shared.cpu().numpy(), want.cpu().numpy()) <= 1e-6
    for m in mats.values():
        ctx.matrix_free(m)
