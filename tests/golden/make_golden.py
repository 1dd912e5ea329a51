#!/usr/bin/env python3
"""Generates tests/golden/*.npz from the reference's own code.

Run where the reference tree is mounted (oracle/Makefile builds oracle/_ref/
libgufo_ref.so from its unmodified sources). Every array here is an output of
the reference on seeded synthetic inputs built by this project's own packers;
the inputs are regenerated from the seeds by the tests, so only outputs (and a
few small inputs) are stored. The quant/ directory beside this file holds the
reference's own dequantization fixtures (tests/fixtures/quant in its tree),
copied unchanged.

    python tests/golden/make_golden.py [name ...]
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from gufo_npu_b200 import quantize as Q  # noqa: E402
from gufo_npu_b200 import synth  # noqa: E402
from oracle import binding  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# Shared with tests/test_oracle.py: the tiny models the goldens were made on.
DENSE = dict(layers=4, hidden=256, ffn=512, vocab=512, heads=2, kv_heads=1, head_dim=128, rope_dim=32,
             linear_key_heads=2, linear_value_heads=4, linear_head_dim=128)
MOE = dict(layers=2, hidden=256, ffn=0, vocab=512, heads=2, kv_heads=1, head_dim=128, rope_dim=32,
           linear_key_heads=2, linear_value_heads=2, linear_head_dim=128, experts=16, experts_used=4,
           expert_ffn=256, shared_expert_ffn=256, full_attention_interval=2, tied_embeddings=False)
DENSE_SEED = 11
# Intermediate DeltaNet states are stored as every SAMPLE-th value; final states whole.
SAMPLE = 37
MOE_SEED = 12


def normal(seed: int, *shape) -> np.ndarray:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float32).numpy()


def dots(ref: binding.RefLib) -> dict:
    """Fused row dots on random-bit rows and on packed N(0, 0.02) rows."""
    out = {}
    for name, t in (("q4k", Q.GGML_Q4_K), ("q6k", Q.GGML_Q6_K)):
        for n in (256, 512, 2048):
            rows = Q.random_blocks(t, 24, n, seed=100 + n).numpy()
            x = normal(200 + n, 24, n)
            out[f"dot_{name}_random_{n}"] = np.array(
                [ref.dot(t, rows[i], x[i]) for i in range(24)], dtype=np.float32)
            w = torch.from_numpy(normal(300 + n, 24, n) * 0.02)
            packed = Q.quantize(t, w).numpy()
            out[f"dot_{name}_packed_{n}"] = np.array(
                [ref.dot(t, packed[i], x[i]) for i in range(24)], dtype=np.float32)
            if n == 512:
                out[f"dequant_{name}_packed_{n}"] = ref.dequantize(t, packed[:8], 8 * n)
                out[f"dequant_{name}_random_{n}"] = ref.dequantize(t, rows[:8], 8 * n)
    return out


def projections(ref: binding.RefLib) -> dict:
    """GgufProjections (fp32 and double) on the dense and MoE models."""
    out = {}
    for tag, kwargs, seed in (("dense", DENSE, DENSE_SEED), ("moe", MOE, MOE_SEED)):
        cfg = synth.ModelConfig(**kwargs)
        image = synth.to_gguf(cfg, synth.build_model(cfg, seed))
        for prec, flt in (("f32", True), ("f64", False)):
            model = ref.open_model(image, precision_float=flt)
            for il in range(cfg.layers):
                stages = ["mixer_out", "ffn_in", "ffn_down"]
                stages.append("attention_in" if cfg.is_full_attention(il) else "linear_in")
                if cfg.is_moe:
                    stages.append("router")
                for stage in stages:
                    for tokens in (1, 3):
                        x = normal(1000 + 10 * il + tokens, tokens, model.stage_inputs(stage, il))
                        out[f"{tag}_{prec}_{stage}_{il}_{tokens}"] = model.apply(stage, il, x)
                if cfg.is_moe:
                    for expert in (0, 5, cfg.experts - 1):
                        for stage in ("expert_in", "expert_down"):
                            x = normal(2000 + expert, 2, model.stage_inputs(stage, il))
                            out[f"{tag}_{prec}_{stage}_{il}_e{expert}"] = model.apply_expert(stage, il, expert, x)
            x = normal(3000, 2, cfg.hidden)
            out[f"{tag}_{prec}_lm_head"] = model.apply("lm_head", -1, x)
            model.close()
    return out


def deltanet(ref: binding.RefLib) -> dict:
    """Mixer::Linear and DeltaNetStep::Run over a run of steps on the dense model."""
    out = {}
    cfg = synth.ModelConfig(**DENSE)
    image = synth.to_gguf(cfg, synth.build_model(cfg, DENSE_SEED))
    model = ref.open_model(image)
    width = model.stage_outputs("linear_in", 0)
    conv = np.zeros((cfg.conv_kernel - 1) * cfg.conv_channels, dtype=np.float32)
    ssm = np.zeros(cfg.linear_value_heads * cfg.linear_head_dim ** 2, dtype=np.float32)
    ys = []
    for step in range(12):
        x_in = normal(4000 + step, width)
        speculative = step % 4 == 3
        y, spec = model.linear(0, x_in, conv, ssm, cfg.value_dim, speculative=speculative)
        if speculative:
            out[f"linear_spec_{step}"] = spec[::SAMPLE].copy()
            if step % 8 == 3:
                ssm[:] = spec          # keep the draft
        ys.append(y)
    out["linear_y"] = np.stack(ys)
    out["linear_conv"] = conv
    out["linear_ssm"] = ssm

    # The fused step (1 or 2 tokens, alpha/beta rows from the residual).
    conv = np.zeros_like(conv)
    ssm = np.zeros_like(ssm)
    for step in range(6):
        count = 1 if step % 3 == 0 else 2
        x_in = normal(5000 + step, count, width)
        h = 4.0 * normal(6000 + step, count, cfg.hidden)
        y, spec, saved = model.deltanet_run(0, count, x_in, h, conv, ssm, cfg.value_dim)
        out[f"fused_y_{step}"] = y
        if count == 2:
            out[f"fused_spec_{step}"] = spec[::SAMPLE].copy()
            out[f"fused_saved_{step}"] = saved[::7].copy()
            if step % 2 == 0:
                ssm[:] = spec
            else:
                conv[:] = saved
    out["fused_conv"] = conv
    out["fused_ssm"] = ssm
    model.close()
    return out


def routing(ref: binding.RefLib) -> dict:
    out = {}
    logits = normal(7000, 8, 256)
    logits[3, 17] = logits[3, 5]       # an exact tie: the lower id wins
    logits[4, :] = 0.0                 # all equal
    out["route_logits"] = logits
    chosen, weights = zip(*(ref.route(logits[i], 8) for i in range(8)))
    out["route_chosen"] = np.stack(chosen)
    out["route_weights"] = np.stack(weights)
    out["shared_scale"] = np.array([ref.shared_expert_scale(float(v)) for v in (-30.0, -1.5, 0.0, 0.25, 12.0)],
                                   dtype=np.float32)
    return out


def decoder(ref: binding.RefLib) -> dict:
    """Decoder::Step logits over a few tokens on both models."""
    out = {}
    for tag, kwargs, seed in (("dense", DENSE, DENSE_SEED), ("moe", MOE, MOE_SEED)):
        cfg = synth.ModelConfig(**kwargs)
        image = synth.to_gguf(cfg, synth.build_model(cfg, seed))
        model = ref.open_model(image)
        model.decoder_reset()
        tokens = [3, 77, 200, 5, 77, 311, 42, 9]
        out[f"decoder_{tag}_tokens"] = np.array(tokens, dtype=np.int32)
        out[f"decoder_{tag}_logits"] = np.stack([model.decoder_step(tok, cfg.vocab) for tok in tokens])
        model.close()
    return out


MTP_SEED = 13


def projections_mtp(ref: binding.RefLib) -> dict:
    """GgufProjections on a dense model with an MTP layer: Stage::kMtpIn (nextn.eh_proj over
    [embedding | hidden]) and the MTP layer's own attention and FFN stages at layer index
    `layers` (gguf_projections.cpp:114-125,205-207)."""
    out = {}
    cfg = synth.ModelConfig(**DENSE, mtp_layers=1)
    image = synth.to_gguf(cfg, synth.build_model(cfg, MTP_SEED))
    il = cfg.layers
    for prec, flt in (("f32", True), ("f64", False)):
        model = ref.open_model(image, precision_float=flt)
        for stage in ("mtp_in", "attention_in", "mixer_out", "ffn_in", "ffn_down"):
            for tokens in (1, 3):
                x = normal(8000 + tokens, tokens, model.stage_inputs(stage, il))
                out[f"{prec}_{stage}_{tokens}"] = model.apply(stage, il, x)
        model.close()
    return out


# Positions whose logits decoder_long keeps: around the 128-position slices the reference's
# attention cuts the cache into (decoder.cpp:326-333) and past a thousand positions.
LONG_STEPS = 1100
LONG_KEEP = (0, 7, 8, 63, 127, 128, 129, 255, 256, 511, 777, 1023, 1024, 1099)
LONG_TOKEN_SEED = 31


def long_tokens(vocab: int) -> np.ndarray:
    return np.random.default_rng(LONG_TOKEN_SEED).integers(0, vocab, size=LONG_STEPS).astype(np.int32)


def decoder_long(ref: binding.RefLib) -> dict:
    """Decoder::Step logits of the dense model over 1100 positions, a few of them kept."""
    cfg = synth.ModelConfig(**DENSE)
    image = synth.to_gguf(cfg, synth.build_model(cfg, DENSE_SEED))
    model = ref.open_model(image)
    model.decoder_reset()
    kept = []
    for i, tok in enumerate(long_tokens(cfg.vocab)):
        if i in LONG_KEEP:
            kept.append(model.decoder_step(int(tok), cfg.vocab))
        else:
            model.decoder_step_discard(int(tok))
    model.close()
    return {"positions": np.array(LONG_KEEP, dtype=np.int32), "logits": np.stack(kept)}


def main() -> int:
    binding.build()
    if not binding.RefLib.available():
        print("the reference tree is not mounted: cannot regenerate goldens")
        return 1
    ref = binding.RefLib()
    only = set(sys.argv[1:])   # e.g. `make_golden.py decoder_long` regenerates that file alone
    for name, fn in (("dots", dots), ("projections", projections), ("deltanet", deltanet),
                     ("routing", routing), ("decoder", decoder), ("decoder_long", decoder_long),
                     ("projections_mtp", projections_mtp)):
        if only and name not in only:
            continue
        arrays = fn(ref)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **arrays)
        print(f"{name}: {len(arrays)} arrays, {os.path.getsize(path)} bytes")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
