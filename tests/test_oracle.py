"""Pins the CPU oracle (oracle/gufo_oracle.c) to the reference.

Three rings, all on the CPU:
  1. the reference's own dequantization fixtures (tests/fixtures/quant in its
     tree, copied to tests/golden/quant) and its fp16 known answers
     (tests/core/quant_test.cpp:51-70), bit for bit;
  2. committed outputs of the reference's compiled sources on seeded inputs
     (tests/golden/*.npz, made by tests/golden/make_golden.py);
  3. where oracle/_ref/libgufo_ref.so exists, the same comparisons live.
"""
import numpy as np
import pytest
import torch

from gufo_npu_b200 import quantize as Q
from gufo_npu_b200 import synth
from tests.golden import make_golden as G

TYPES = {"q4k": Q.GGML_Q4_K, "q6k": Q.GGML_Q6_K}


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("name,ggml_type", [("Q4_K", Q.GGML_Q4_K), ("Q6_K", Q.GGML_Q6_K),
                                            ("Q5_K", Q.GGML_Q5_K), ("Q8_0", Q.GGML_Q8_0),
                                            ("BF16", Q.GGML_BF16)])
def test_dequantize_matches_reference_fixtures(oracle, golden, name, ggml_type):
    raw = np.fromfile(golden.path("quant", name + ".bin"), dtype=np.uint8)
    want = np.fromfile(golden.path("quant", name + ".f32"), dtype=np.float32)
    assert oracle.row_bytes(ggml_type, want.size) == raw.size
    got = oracle.dequantize(ggml_type, raw, want.size)
    assert np.array_equal(bits(got), bits(want))


def test_half_known_answers(oracle):
    cases = {0x0000: 0.0, 0x3C00: 1.0, 0xC000: -2.0, 0x3555: 0.333251953125,
             0x0001: 5.96046448e-08, 0x7BFF: 65504.0}
    for h, value in cases.items():
        assert oracle.half_to_float(h) == np.float32(value)
    # Every finite half against numpy's conversion.
    halves = np.arange(0, 0x7C00, dtype=np.uint16)
    want = halves.view(np.float16).astype(np.float32)
    got = np.array([oracle.half_to_float(int(h)) for h in halves[::7]], dtype=np.float32)
    assert np.array_equal(got, want[::7])


def test_partial_block_rejected(oracle):
    with pytest.raises(ValueError):
        oracle.dequantize(Q.GGML_Q4_K, np.zeros(144, dtype=np.uint8), 255)
    assert oracle.row_bytes(Q.GGML_Q6_K, 100) == 0


@pytest.mark.parametrize("name", ["q4k", "q6k"])
@pytest.mark.parametrize("n", [256, 512, 2048])
def test_fused_dots_match_reference_bit_for_bit(oracle, golden, name, n):
    t = TYPES[name]
    g = golden("dots")
    rows = Q.random_blocks(t, 24, n, seed=100 + n).numpy()
    x = G.normal(200 + n, 24, n)
    got = np.array([oracle.dot(t, rows[i], x[i]) for i in range(24)], dtype=np.float32)
    assert np.array_equal(bits(got), bits(g[f"dot_{name}_random_{n}"]))
    packed = Q.quantize(t, torch.from_numpy(G.normal(300 + n, 24, n) * 0.02)).numpy()
    got = np.array([oracle.dot(t, packed[i], x[i]) for i in range(24)], dtype=np.float32)
    assert np.array_equal(bits(got), bits(g[f"dot_{name}_packed_{n}"]))
    if n == 512:
        assert np.array_equal(bits(oracle.dequantize(t, packed[:8], 8 * n)), bits(g[f"dequant_{name}_packed_{n}"]))
        assert np.array_equal(bits(oracle.dequantize(t, rows[:8], 8 * n)), bits(g[f"dequant_{name}_random_{n}"]))


@pytest.mark.parametrize("name", ["q4k", "q6k"])
def test_fused_dot_close_to_double_sum(oracle, name):
    """The reference's own bound: error < 2e-5 of sum |w x| (tests/models/qwen35/gguf_dot_test.cpp:114-116)."""
    t = TYPES[name]
    rows = Q.random_blocks(t, 50, 2048, seed=5).numpy()
    x = G.normal(6, 50, 2048)
    for i in range(50):
        w = oracle.dequantize(t, rows[i], 2048).astype(np.float64)
        want = float(np.dot(w, x[i].astype(np.float64)))
        magnitude = float(np.abs(w * x[i]).sum())
        assert abs(oracle.dot(t, rows[i], x[i]) - want) < 2e-5 * magnitude


def _model_parts(cfg, tensors, stage, il):
    """(bytes 2-D, type, first, rows) lists as GgufProjections stacks them
    (src/models/qwen35/gguf_projections.cpp:100-175, 219-237)."""
    p = f"blk.{il}."
    suffix = "_shexp.weight" if cfg.is_moe else ".weight"
    names = {
        "linear_in": [p + "attn_qkv.weight", p + "attn_gate.weight", p + "ssm_alpha.weight", p + "ssm_beta.weight"],
        "attention_in": [p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"],
        "mixer_out": [p + ("attn_output.weight" if cfg.is_full_attention(il) else "ssm_out.weight")],
        "ffn_in": [p + "ffn_gate" + suffix, p + "ffn_up" + suffix],
        "ffn_down": [p + "ffn_down" + suffix],
        "router": [p + "ffn_gate_inp.weight", p + "ffn_gate_inp_shexp.weight"],
        "lm_head": ["token_embd.weight" if cfg.tied_embeddings else "output.weight"],
    }[stage]
    parts = []
    for name in names:
        t = tensors[name]
        data = t.data.numpy().reshape(t.rows, -1)
        parts.append((data, t.ggml_type, 0, t.rows))
    return parts, tensors[names[0]].cols


@pytest.mark.parametrize("tag,kwargs,seed", [("dense", G.DENSE, G.DENSE_SEED), ("moe", G.MOE, G.MOE_SEED)])
def test_matmul_matches_reference_projections(oracle, golden, tag, kwargs, seed):
    cfg = synth.ModelConfig(**kwargs)
    tensors = synth.build_model(cfg, seed)
    g = golden("projections")
    checked = 0
    for il in range(cfg.layers):
        stages = ["mixer_out", "ffn_in", "ffn_down", "attention_in" if cfg.is_full_attention(il) else "linear_in"]
        if cfg.is_moe:
            stages.append("router")
        for stage in stages:
            parts, cols = _model_parts(cfg, tensors, stage, il)
            for tokens in (1, 3):
                x = G.normal(1000 + 10 * il + tokens, tokens, cols)
                got = oracle.matmul(parts, cols, x)
                assert np.array_equal(bits(got), bits(g[f"{tag}_f32_{stage}_{il}_{tokens}"])), (stage, il, tokens)
                exact = oracle.matmul(parts, cols, x, exact=True)
                assert np.array_equal(bits(exact), bits(g[f"{tag}_f64_{stage}_{il}_{tokens}"])), (stage, il)
                checked += 1
        if cfg.is_moe:
            p = f"blk.{il}."
            for expert in (0, 5, cfg.experts - 1):
                gate, up, down = (tensors[p + n] for n in ("ffn_gate_exps.weight", "ffn_up_exps.weight",
                                                           "ffn_down_exps.weight"))
                x = G.normal(2000 + expert, 2, cfg.hidden)
                parts = [(t.data.numpy().reshape(t.rows, -1), t.ggml_type, expert * cfg.expert_ffn, cfg.expert_ffn)
                         for t in (gate, up)]
                assert np.array_equal(bits(oracle.matmul(parts, cfg.hidden, x)),
                                      bits(g[f"{tag}_f32_expert_in_{il}_e{expert}"]))
                x = G.normal(2000 + expert, 2, cfg.expert_ffn)
                parts = [(down.data.numpy().reshape(down.rows, -1), down.ggml_type, expert * cfg.hidden, cfg.hidden)]
                assert np.array_equal(bits(oracle.matmul(parts, cfg.expert_ffn, x)),
                                      bits(g[f"{tag}_f32_expert_down_{il}_e{expert}"]))
    parts, cols = _model_parts(cfg, tensors, "lm_head", -1)
    assert np.array_equal(bits(oracle.matmul(parts, cols, G.normal(3000, 2, cfg.hidden))), bits(g[f"{tag}_f32_lm_head"]))
    assert checked > 0


def _deltanet_weights(cfg, tensors, il):
    p = f"blk.{il}."

    def f32(name):
        return tensors[p + name].data.numpy().view(np.float32).copy()
    return {"conv": f32("ssm_conv1d.weight"), "ssm_a": f32("ssm_a"), "dt_bias": f32("ssm_dt.bias"),
            "ssm_norm": f32("ssm_norm.weight")}


def _deltanet_cfg(cfg):
    return {"key_heads": cfg.linear_key_heads, "value_heads": cfg.linear_value_heads,
            "head_dim": cfg.linear_head_dim, "conv_kernel": cfg.conv_kernel, "rms_eps": cfg.rms_eps}


def test_deltanet_linear_matches_reference(oracle, golden):
    """Mixer::Linear over 12 steps with speculative states kept or dropped: bit for bit."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    g = golden("deltanet")
    weights = _deltanet_weights(cfg, tensors, 0)
    width = cfg.conv_channels + cfg.value_dim + 2 * cfg.linear_value_heads
    conv = np.zeros((cfg.conv_kernel - 1) * cfg.conv_channels, dtype=np.float32)
    ssm = np.zeros(cfg.linear_value_heads * cfg.linear_head_dim ** 2, dtype=np.float32)
    for step in range(12):
        x_in = G.normal(4000 + step, width)
        speculative = step % 4 == 3
        y, spec = oracle.deltanet_linear(_deltanet_cfg(cfg), weights, x_in, conv, ssm, speculative)
        assert np.array_equal(bits(y), bits(g["linear_y"][step])), step
        if speculative:
            assert np.array_equal(bits(spec[::G.SAMPLE]), bits(g[f"linear_spec_{step}"]))
            if step % 8 == 3:
                ssm[:] = spec
    assert np.array_equal(bits(conv), bits(g["linear_conv"]))
    assert np.array_equal(bits(ssm), bits(g["linear_ssm"]))


def test_fused_deltanet_step_matches_reference(oracle, golden):
    """DeltaNetStep::Run (1 or 2 tokens, alpha/beta rows from the residual) restated as
    RMSNorm + two F32 row dots + Mixer::Linear per token (src/models/qwen35_2b/deltanet.cpp:358-392)."""
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    g = golden("deltanet")
    weights = _deltanet_weights(cfg, tensors, 0)
    p = "blk.0."
    attn_norm = tensors[p + "attn_norm.weight"].data.numpy().view(np.float32).copy()
    ab = [(tensors[p + n].data.numpy().reshape(cfg.linear_value_heads, -1), Q.GGML_F32, 0, cfg.linear_value_heads)
          for n in ("ssm_alpha.weight", "ssm_beta.weight")]
    rows = cfg.conv_channels + cfg.value_dim
    width = rows + 2 * cfg.linear_value_heads
    conv = np.zeros((cfg.conv_kernel - 1) * cfg.conv_channels, dtype=np.float32)
    ssm = np.zeros(cfg.linear_value_heads * cfg.linear_head_dim ** 2, dtype=np.float32)
    for step in range(6):
        count = 1 if step % 3 == 0 else 2
        x_in = G.normal(5000 + step, count, width)
        h = 4.0 * G.normal(6000 + step, count, cfg.hidden)
        saved = None
        spec = None
        for t in range(count):
            normed = oracle.rms_norm(h[t].copy(), attn_norm, cfg.rms_eps)
            full = np.concatenate([x_in[t, :rows], oracle.matmul(ab, cfg.hidden, normed)[0]]).astype(np.float32)
            if count == 2 and t == 1:
                saved = conv.copy()
            y, out = oracle.deltanet_linear(_deltanet_cfg(cfg), weights, full, conv, ssm, count == 2 and t == 1)
            if out is not None:
                spec = out
            assert np.array_equal(bits(y), bits(g[f"fused_y_{step}"][t])), (step, t)
        if count == 2:
            assert np.array_equal(bits(spec[::G.SAMPLE]), bits(g[f"fused_spec_{step}"]))
            assert np.array_equal(bits(saved[::7]), bits(g[f"fused_saved_{step}"]))
            if step % 2 == 0:
                ssm[:] = spec
            else:
                conv[:] = saved
    assert np.array_equal(bits(conv), bits(g["fused_conv"]))
    assert np.array_equal(bits(ssm), bits(g["fused_ssm"]))


def test_route_matches_reference(oracle, golden):
    g = golden("routing")
    logits = g["route_logits"]
    for i in range(logits.shape[0]):
        chosen, weights = oracle.route(logits[i], 8)
        assert np.array_equal(chosen, g["route_chosen"][i])
        assert np.array_equal(bits(weights), bits(g["route_weights"][i]))
    # Ties go to the lower id; all-equal logits pick ids 0..7 at weight 1/8.
    assert list(g["route_chosen"][4]) == list(range(8))
    scales = [oracle.shared_expert_scale(v) for v in (-30.0, -1.5, 0.0, 0.25, 12.0)]
    assert np.array_equal(bits(np.array(scales, dtype=np.float32)), bits(g["shared_scale"]))


def test_delta_rule_equals_closed_form(oracle):
    """S' = a S (I - b k k^T) + b v k^T and o = S' q in the [key][value] layout, in float64."""
    rng = np.random.default_rng(3)
    dk = 128
    s = rng.standard_normal((dk, dk)).astype(np.float32)
    k = rng.standard_normal(dk).astype(np.float32)
    k /= np.linalg.norm(k)
    q = rng.standard_normal(dk).astype(np.float32)
    q /= np.linalg.norm(q)
    v = rng.standard_normal(dk).astype(np.float32)
    decay, beta = 0.9, 0.6
    out, y = oracle.delta_rule(s, k, q, v, decay, beta)
    s64 = s.astype(np.float64).T                       # [value][key]
    want = decay * s64 @ (np.eye(dk) - beta * np.outer(k, k)) + beta * np.outer(v, k)
    assert np.allclose(out.T, want, atol=1e-5)
    assert np.allclose(y, want @ q, atol=1e-5)


def test_live_reference_agrees_with_committed_goldens(reflib, golden):
    """Where the compiled reference travels, it must still produce the committed goldens."""
    g = golden("dots")
    for name, t in TYPES.items():
        rows = Q.random_blocks(t, 24, 512, seed=100 + 512).numpy()
        x = G.normal(200 + 512, 24, 512)
        got = np.array([reflib.dot(t, rows[i], x[i]) for i in range(24)], dtype=np.float32)
        assert np.array_equal(bits(got), bits(g[f"dot_{name}_random_512"]))
    assert reflib.usable_cpus() >= 1


def test_oracle_decoder_and_attention_match_reference_logits(oracle, golden):
    """The Python restatement of Decoder::Step (oracle/decoder.py, with the attention of
    oracle/attention.py) against the reference's committed logits: the 8-token run, and the
    1100-position run up to position 256 (two of the reference's 128-position slices)."""
    from oracle.decoder import OracleDecoder
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    g = golden("decoder")
    dec = OracleDecoder(oracle, cfg, tensors, 8)
    for i, tok in enumerate(int(t) for t in g["decoder_dense_tokens"]):
        got = dec.step(tok)
        want = g["decoder_dense_logits"][i]
        err = np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want)
        assert err < 2e-5, (i, err)
    long = golden("decoder_long")
    keep = {int(p): i for i, p in enumerate(long["positions"])}
    dec = OracleDecoder(oracle, cfg, tensors, 257)
    for pos, tok in enumerate(G.long_tokens(cfg.vocab)[:257]):
        got = dec.step(int(tok))
        if pos in keep:
            want = long["logits"][keep[pos]]
            err = np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want)
            assert err < 5e-5, (pos, err)


def test_oracle_mtp_layer_projections_match_reference(oracle, golden):
    """Stage::kMtpIn and the MTP layer's stages: the oracle's fused dots over the same rows the
    reference stacks (gguf_projections.cpp:114-125), bit for bit in fp32."""
    cfg = synth.ModelConfig(**G.DENSE, mtp_layers=1)
    tensors = synth.build_model(cfg, G.MTP_SEED)
    g = golden("projections_mtp")
    p = f"blk.{cfg.layers}."
    stages = {"mtp_in": ["nextn.eh_proj.weight"], "attention_in": ["attn_q.weight", "attn_k.weight", "attn_v.weight"],
              "mixer_out": ["attn_output.weight"], "ffn_in": ["ffn_gate.weight", "ffn_up.weight"],
              "ffn_down": ["ffn_down.weight"]}
    for name, parts in stages.items():
        rows = [(tensors[p + n].data.numpy().reshape(tensors[p + n].rows, -1), tensors[p + n].ggml_type, 0,
                 tensors[p + n].rows) for n in parts]
        cols = tensors[p + parts[0]].cols
        for tokens in (1, 3):
            x = G.normal(8000 + tokens, tokens, cols)
            got = oracle.matmul(rows, cols, x)
            assert np.array_equal(bits(got), bits(g[f"f32_{name}_{tokens}"])), (name, tokens)
            exact = oracle.matmul(rows, cols, x, exact=True)
            assert np.array_equal(bits(exact), bits(g[f"f64_{name}_{tokens}"])), (name, tokens)
