#!/usr/bin/env python3
"""Benchmark of the decode hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step (one token through every projection, the Gated DeltaNet and
attention mixers and the LM head) of a synthetic 2B-class dense model: hidden 2048, FFN 6144,
24 layers (18 Gated DeltaNet + 6 gated attention with 8 query / 2 KV heads of 256), Q4_K
projections, Q6_K down projections and a tied Q6_K LM head of 248320 rows. Weights are
N(0, 0.02) values packed by this project's quantizers from a seed; nothing is downloaded.

Prints ONE JSON line: decode-step tok/s with the state resident on the device (`value`), the
same through the host-facing call with the token uploaded and the logits downloaded every step
(`e2e`), the HBM roofline of the metric's kernel (the 6144 x 2048 Q4_K GEMV) measured live
(`roofline`; other kernels under `roofline_more`), the logits' agreement with the reference on
the same model and tokens (`parity`), and the reference's own CPU decoder timed on the host
cores (`cpu_baseline`). `--impl reference` times only the latter. With --gpus N > 1 (torchrun)
the projections are row-split over N GPUs with an all-gather after each product; the line then
also carries the row-split verify batch and the expert-parallel MoE layer.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np
import torch

from gufo_npu_b200 import quantize as Q
from gufo_npu_b200 import synth

METRIC = "decode_step_tokens_per_s"
UNIT = "tok/s"
WORKLOAD = "decode step, 2B-class dense (hidden 2048, ffn 6144, 18 DeltaNet + 6 attention layers, " \
           "Q4_K projections, Q6_K down + LM head 248320x2048), batch 1"


def model_config() -> synth.ModelConfig:
    return synth.ModelConfig(layers=24, hidden=2048, ffn=6144, vocab=248320, rms_eps=1e-6,
                             full_attention_interval=4, heads=8, kv_heads=2, head_dim=256, rope_dim=64,
                             rope_theta=1e7, conv_kernel=4, linear_key_heads=16, linear_value_heads=16,
                             linear_head_dim=128, tied_embeddings=True)


def weight_bytes(tensors) -> int:
    return int(sum(t.data.numel() for name, t in tensors.items() if t.ggml_type != Q.GGML_F32 or t.rows > 1))


def measured_peaks():
    from gufo_npu_b200.bench_support import measured_hbm_peak
    return measured_hbm_peak()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, device: int):
        self.device = device
        self.samples = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        mhz, top, reasons = [], 0.0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                top = max(top, float(s[1]))
            except ValueError:
                continue
            for name, flag in zip(names, s[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": top or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def time_on_stream(fn, iters: int) -> float:
    """Milliseconds per call of fn over `iters` calls, by CUDA events on the current stream."""
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for i in range(iters):
        fn(i)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters


# ---- reference arm / CPU baseline ---------------------------------------------

PARITY_TOKENS = (11, 4242, 98765, 7)   # the steps compared with the reference before the CPU timing


def cpu_decode(tensors_host, cfg, steps: int, warmup: int, budget_s: float = 25.0, gpu_step=None):
    """Times the reference's own CPU decoder (Decoder::Step over GgufProjections, fp32) on the
    host cores, where oracle/_ref was built; else this project's C restatement on a sample.
    `gpu_step(token) -> logits`, when given, is run beside the reference's first steps and the
    logits compared (the returned dict then carries "parity")."""
    from oracle import binding
    if binding.RefLib.available():
        ref = binding.RefLib()
        image = synth.to_gguf(cfg, tensors_host)
        model = ref.open_model(image, precision_float=True)
        del image
        model.decoder_reset()
        parity = None
        if gpu_step is not None:
            worst, same = 0.0, True
            for tok in PARITY_TOKENS:
                want = model.decoder_step(tok % cfg.vocab, cfg.vocab).astype(np.float64)
                got = np.asarray(gpu_step(tok % cfg.vocab), dtype=np.float64)
                worst = max(worst, float(np.linalg.norm(got - want) / np.linalg.norm(want)))
                same = same and int(np.argmax(got)) == int(np.argmax(want))
            parity = {"config2_logits_rel_l2": worst, "same_argmax": same, "tokens": len(PARITY_TOKENS),
                      "tolerance": 2e-3, "against": "the reference's Decoder::Step over GgufProjections(kFloat), "
                                                    "compiled from its sources, same model and tokens"}
            if worst > 2e-3 or not same:
                raise SystemExit(f"parity with the reference failed at the benchmarked configuration: {parity}")
            model.decoder_reset()
        rng = np.random.default_rng(5)
        for _ in range(max(warmup, 1)):
            model.decoder_step_discard(int(rng.integers(0, cfg.vocab)))
        times = []
        begin = time.perf_counter()
        for _ in range(steps):
            t0 = time.perf_counter()
            model.decoder_step_discard(int(rng.integers(0, cfg.vocab)))
            times.append(time.perf_counter() - t0)
            if time.perf_counter() - begin > budget_s:
                break
        # The reference's own kernels on two of the configurations, for the probes' rooflines:
        # GgufProjections::MatMul over gate | up (2 x 6144 x 2048 Q4_K, rotating over the layers so
        # that rows come from memory) and Mixer::Linear (16 heads of 128 x 128 state).
        more = {}
        x = rng.standard_normal(cfg.hidden).astype(np.float32)
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < 2.0:
            model.apply("ffn_in", n % cfg.layers, x)
            n += 1
        us = (time.perf_counter() - t0) / n * 1e6
        nbytes = 2 * cfg.ffn * Q.row_bytes(Q.GGML_Q4_K, cfg.hidden)
        more["q4k_matmul_2x6144x2048"] = {"us": us, "GB/s": nbytes / us / 1e3}
        linear_layers = [il for il in range(cfg.layers) if not cfg.is_full_attention(il)]
        width = cfg.conv_channels + cfg.value_dim + 2 * cfg.linear_value_heads
        conv = np.zeros((cfg.conv_kernel - 1) * cfg.conv_channels, dtype=np.float32)
        ssm = (rng.standard_normal(cfg.linear_value_heads * cfg.linear_head_dim ** 2) * 0.1).astype(np.float32)
        x_in = rng.standard_normal(width).astype(np.float32)
        t0 = time.perf_counter()
        n = 0
        while time.perf_counter() - t0 < 1.0:
            model.linear(linear_layers[n % len(linear_layers)], x_in, conv, ssm, cfg.value_dim)
            n += 1
        us = (time.perf_counter() - t0) / n * 1e6
        more["deltanet_linear_16_heads_one_sequence"] = {"us": us, "GB/s": 2130048 / us / 1e3,
                                                         "note": "the binding copies the 1 MiB state in and out per call"}
        model.close()
        ms = 1e3 * float(np.mean(times))
        out = {"value": 1e3 / ms, "unit": UNIT, "cores": ref.usable_cpus(), "kind": "reference",
               "threads": f"{ref.projection_threads()} projection threads (HalfCpuWorkers + caller) and the mixers' pool, "
                          f"the reference's defaults on {ref.usable_cpus()} usable CPUs; the reference sizes its pools "
                          f"itself (src/core/cpus.hpp:53-55) and offers no all-cores setting",
               "sample": f"{len(times)} whole decode steps of the same model through the reference's "
                         f"Decoder::Step + GgufProjections(kFloat), compiled from its sources",
               "ms_per_step": ms, "kernels": more}
        if parity is not None:
            out["parity"] = parity
        return out
    # Port: one layer's projections and 1/64 of the LM head through the single-threaded C
    # restatement, scaled to a step (the mixers' share is under 3 % of a step's bytes).
    oracle = binding.Oracle()
    x = np.random.default_rng(5).standard_normal(cfg.hidden).astype(np.float32)
    t0 = time.perf_counter()
    total = 0.0
    for name, scale in (("blk.0.attn_qkv.weight", 18), ("blk.0.attn_gate.weight", 18), ("blk.0.ssm_out.weight", 18),
                        ("blk.3.attn_q.weight", 6), ("blk.3.attn_output.weight", 6),
                        ("blk.0.ffn_gate.weight", 24), ("blk.0.ffn_up.weight", 24)):
        t = tensors_host[name]
        data = t.data.numpy().reshape(t.rows, -1)
        t1 = time.perf_counter()
        oracle.matmul([(data, t.ggml_type, 0, t.rows)], t.cols, x[:t.cols] if t.cols <= x.size else np.resize(x, t.cols))
        total += (time.perf_counter() - t1) * scale
    t = tensors_host["blk.0.ffn_down.weight"]
    t1 = time.perf_counter()
    oracle.matmul([(t.data.numpy().reshape(t.rows, -1), t.ggml_type, 0, t.rows)], t.cols, np.resize(x, t.cols))
    total += (time.perf_counter() - t1) * 24
    t = tensors_host["token_embd.weight"]
    rows = t.rows // 64
    t1 = time.perf_counter()
    oracle.matmul([(t.data.numpy().reshape(t.rows, -1), t.ggml_type, 0, rows)], t.cols, x)
    total += (time.perf_counter() - t1) * 64
    del t0
    return {"value": 1.0 / total, "unit": UNIT, "cores": 1, "kind": "port",
            "sample": "one layer of each kind and 1/64 of the LM head through the single-threaded C restatement, "
                      "scaled to a step", "ms_per_step": 1e3 * total}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = model_config()
    tensors = synth.build_model(cfg, seed=1, device="cuda" if torch.cuda.is_available() else "cpu")
    host = {k: synth.Tensor(t.shape, t.ggml_type, t.data.cpu()) for k, t in tensors.items()}
    del tensors
    base = cpu_decode(host, cfg, steps=args.steps, warmup=args.warmup, budget_s=120.0)
    line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "seed": 1}, "cpu_baseline": base,
            "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ---- our arm ----------------------------------------------------------------------

def roofline_probes(ctx, proj, cfg, stream, peak):
    """HBM rooflines measured live with CUDA events on the launching stream: the LM-head Q6_K
    GEMV (the step's dominant kernel), the 6144 x 2048 Q4_K GEMV and the 16-head DeltaNet step."""
    from gufo_npu_b200 import _capi
    from gufo_npu_b200.backend import Context
    dev = torch.device("cuda", ctx.device)
    out = {}
    # LM head: 417 MB, larger than L2, so every launch streams from HBM.
    x = torch.randn(1, cfg.hidden, device=dev)
    y = torch.empty(1, cfg.vocab, device=dev)
    parts = Context._parts(proj.lm_head)
    for i in range(3):
        ctx.matmul_device(parts, 1, x, 1, y)
    ms = time_on_stream(lambda i: ctx.matmul_device(parts, 1, x, 1, y), 20)
    lm_bytes = cfg.vocab * Q.row_bytes(Q.GGML_Q6_K, cfg.hidden) + 4 * cfg.hidden + 4 * cfg.vocab
    out["lm_head"] = {"kernel": "GemvMma<Q6_K, 1 token>", "shape": f"{cfg.vocab}x{cfg.hidden} Q6_K, 1 token",
                      "bytes": lm_bytes, "us": ms * 1e3, "achieved": lm_bytes / ms / 1e6,
                      "frac": lm_bytes / ms / 1e6 / peak}
    # 6144 x 2048 Q4_K: rotate over the 24 layers' gate matrices (170 MB > L2), graph-replayed.
    mats = [Context._parts([proj.layers[il][3][0]]) for il in range(cfg.layers)]   # Stage.kFfnIn, gate
    yg = torch.empty(1, cfg.ffn, device=dev)
    # One launch per product, as the decode step runs it: the kernel converts x by itself
    # (gufo_cuda_matmul_fused_device, plain input). Beside it the two-launch form of
    # gufo_cuda_matmul_device (a staging kernel, then the GEMV against the staged image).
    def replay_us(enqueue):
        g = torch.cuda.CUDAGraph()
        for m in mats[:3]:
            enqueue(m)
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=stream):
            for m in mats:
                enqueue(m)
        g.replay()
        return time_on_stream(lambda i: g.replay(), 20) / len(mats)
    ms = replay_us(lambda m: ctx.matmul_fused_device(m, 1, 1, yg, x=x))
    ms_staged = replay_us(lambda m: ctx.matmul_device(m, 1, x, 1, yg))
    b = cfg.ffn * Q.row_bytes(Q.GGML_Q4_K, cfg.hidden) + 4 * cfg.hidden + 4 * cfg.ffn
    out["q4k_gemv"] = {"kernel": "GemvMma<Q4_K, 1 token>", "shape": f"{cfg.ffn}x{cfg.hidden} Q4_K, 1 token",
                       "bytes": b, "us": ms * 1e3, "achieved": b / ms / 1e6, "frac": b / ms / 1e6 / peak,
                       "note": "24 distinct matrices per graph replay (170 MB, larger than L2), one launch per "
                               f"product; with x staged by a kernel of its own first: {ms_staged * 1e3:.2f} us"}
    # The same Q4_K kernel on a product large enough to run at its sustained rate (262144 x 2048,
    # 302 MB): what the kernel streams once the per-launch ramp and tail are amortised.
    big_rows = 262144
    gen = torch.Generator(device=dev).manual_seed(9)
    raw = Q.quantize(Q.GGML_Q4_K, torch.randn(big_rows, cfg.hidden, device=dev, generator=gen) * 0.02)
    big = Context._parts([(ctx.matrix_from_device(Q.GGML_Q4_K, raw.data_ptr(), big_rows, cfg.hidden), 0, big_rows)])
    yb = torch.empty(1, big_rows, device=dev)
    for i in range(3):
        ctx.matmul_device(big, 1, x, 1, yb)
    ms = time_on_stream(lambda i: ctx.matmul_device(big, 1, x, 1, yb), 20)
    b = big_rows * Q.row_bytes(Q.GGML_Q4_K, cfg.hidden) + 4 * cfg.hidden + 4 * big_rows
    out["q4k_gemv_sustained"] = {"kernel": "GemvMma<Q4_K, 1 token>", "shape": f"{big_rows}x{cfg.hidden} Q4_K, 1 token",
                                 "bytes": b, "us": ms * 1e3, "achieved": b / ms / 1e6, "frac": b / ms / 1e6 / peak}
    torch.cuda.synchronize()
    del raw, yb
    # DeltaNet step: 8 sequences x 16 heads x 128 x 128 fp32, 12 state sets (192 MB) rotated.
    hv, dk, nseq, sets = 16, 128, 8, 12
    st = torch.randn(sets, nseq, hv, dk, dk, device=dev) * 0.1
    q = torch.nn.functional.normalize(torch.randn(nseq, hv, dk, device=dev), dim=-1)
    k = torch.nn.functional.normalize(torch.randn(nseq, hv, dk, device=dev), dim=-1)
    v = torch.randn(nseq, hv, dk, device=dev)
    decay = torch.exp(-torch.nn.functional.softplus(torch.randn(nseq, hv, device=dev)))
    beta = torch.sigmoid(torch.randn(nseq, hv, device=dev))
    yd = torch.empty(nseq, hv, dk, device=dev)
    arrs = []
    for c in range(sets):
        arr = (_capi.DeltaSeq * nseq)()
        for s in range(nseq):
            arr[s] = _capi.DeltaSeq(st[c, s].data_ptr(), 0, q[s].data_ptr(), k[s].data_ptr(), v[s].data_ptr(),
                                    decay[s].data_ptr(), beta[s].data_ptr(), yd[s].data_ptr())
        arrs.append(arr)
    run = lambda c: ctx._check(ctx.lib.gufo_cuda_delta_rule_device(ctx.handle, arrs[c], nseq, hv, hv, dk))
    # Each state set is touched once per 12 launches, so the kernels may request their state
    # ahead of the previous launch's completion.
    ctx.set_option("deltanet_early_state", 1)
    for c in range(3):
        run(c)
    torch.cuda.synchronize()
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=stream):
        for c in range(sets):
            run(c)
    g2.replay()
    ms = time_on_stream(lambda i: g2.replay(), 20) / sets
    ctx.set_option("deltanet_early_state", 0)
    b = 17040384
    out["deltanet"] = {"kernel": "DeltaRuleKernel", "shape": "8 sequences x 16 heads x 128x128 fp32", "bytes": b,
                       "us": ms * 1e3, "achieved": b / ms / 1e6, "frac": b / ms / 1e6 / peak,
                       "note": "12 state sets (192 MB) per graph replay"}
    del st
    return out


def run_ours(args):
    from gufo_npu_b200.backend import Context, CudaDecoder, CudaProjections
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        from gufo_npu_b200 import tp
        return tp.run_bench(args, model_config(), METRIC, UNIT, WORKLOAD)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    cfg = model_config()
    tensors = synth.build_model(cfg, seed=1, device=str(dev))
    total_bytes = weight_bytes(tensors)
    ctx = Context(local, stream.cuda_stream)
    proj = CudaProjections(ctx, cfg, tensors)
    dec = CudaDecoder(proj, tensors, max_positions=max(4096, 16 * (args.steps + args.warmup) + 256), use_graph=True)
    peak, peak_kind = measured_peaks()
    rng = np.random.default_rng(7)
    tokens = rng.integers(0, cfg.vocab, size=16 * (args.steps + args.warmup) + 256).tolist()
    cursor = iter(tokens)
    logits_host = torch.empty(cfg.vocab, dtype=torch.float32).pin_memory()

    # Warm-up (also captures the two step graphs).
    for _ in range(max(args.warmup, 3)):
        dec.step_device(next(cursor))
    torch.cuda.synchronize()
    repeats = 5
    with ClockSampler(local) as clocks:
        # K steps timed `repeats` times over (each between synchronizes, CUDA events on the
        # launching stream); the median is reported, every repeat is listed.
        launches0 = ctx.launch_count()
        resident_ms = [time_on_stream(lambda i: dec.step_device(next(cursor)), args.steps) for _ in range(repeats)]
        launches = (ctx.launch_count() - launches0) // repeats
        ms_resident = float(np.median(resident_ms))
        # End to end: token id up (4 bytes, pinned), logits down (vocab fp32, pinned) every step.
        for _ in range(2):
            dec.Step(next(cursor), logits_host.numpy())
        e2e_ms = [time_on_stream(lambda i: dec.Step(next(cursor), logits_host.numpy()), args.steps)
                  for _ in range(repeats)]
        ms_e2e = float(np.median(e2e_ms))
        probes = roofline_probes(ctx, proj, cfg, stream, peak)
        # Two-token steps (a token and a draft, the weights read once for both), drafts kept
        # or rolled back: what speculative decoding pays per step on this path.
        pair_ms = {}
        for keep in (True, False):
            def pair_step(i, keep=keep):
                dec.step_tokens_device([next(cursor), next(cursor)])
                dec.Resolve(keep)
            for _ in range(3):
                pair_step(0)
            pair_ms[keep] = time_on_stream(pair_step, max(args.steps // 2, 8))
    assert np.isfinite(logits_host.numpy()).all()
    host = {k: synth.Tensor(t.shape, t.ggml_type, t.data.cpu()) for k, t in tensors.items()}
    del tensors
    # The benchmarked decoder against the reference on the same first tokens, then the
    # reference's own timing on the host cores.
    dec.Reset()
    base = cpu_decode(host, cfg, steps=200, warmup=2, budget_s=20.0, gpu_step=lambda tok: dec.Step(tok))
    parity = base.pop("parity", None)
    gemv = probes["q4k_gemv"]
    line = {
        "metric": METRIC, "value": 1e3 / ms_resident, "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_resident, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32 (int8 tensor-core code dots, 24-bit fixed-point activations)",
        "data": "synthetic",
        "config": {"workload": WORKLOAD, "seed": 1},
        "notes": {"weight_bytes_per_step": total_bytes,
                  "l2": "weights read per step (1.15 GB) exceed L2 (126 MB); no flush needed",
                  "step_hbm_frac": total_bytes / (ms_resident * 1e-3) / 1e9 / peak,
                  "launch": "CUDA graph per step parity, programmatic dependent launch",
                  "timing": f"median of {repeats} repeats of {args.steps} steps",
                  "ms_per_step_repeats": resident_ms, "e2e_ms_per_step_repeats": e2e_ms},
        "parity": parity,
        "e2e": {"value": 1e3 / ms_e2e, "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": cfg.vocab * 4,
                "ms_per_step": ms_e2e,
                "note": "gufo_cuda_decoder_step per token: the id is copied up, the step runs, the logits land in the "
                        "caller's pinned buffer (written there over PCIe by the LM head's own stores while it "
                        "runs; a pageable buffer gets a copy after the step) and the call returns after a "
                        "stream synchronize"},
        "gpu_launches": int(launches),
        # The metric's kernel: the 6144 x 2048 Q4_K GEMV, one launch per product, 24 distinct
        # matrices back to back. `traffic` is the DRAM traffic of one launch from an ncu capture of
        # the same shape (the algorithmic bytes plus 0.6 %).
        "roofline": {"bound": "hbm", "achieved": gemv["achieved"], "peak": peak, "unit": "GB/s",
                     "frac": gemv["frac"], "traffic": Q4K_GEMV_TRAFFIC_BYTES,
                     "traffic_source": "ncu capture of the same launch (bench.py --probe q4k)", "peak_kind": peak_kind,
                     "kernel": gemv["kernel"], "shape": gemv["shape"], "bytes_per_launch": gemv["bytes"],
                     "us_per_launch": gemv["us"], "note": gemv["note"]},
        "roofline_more": {k: v for k, v in probes.items() if k != "q4k_gemv"},
        "pair_step": {"ms_kept": pair_ms[True], "ms_rolled_back": pair_ms[False],
                      "tok_s_all_kept": 2e3 / pair_ms[True], "tok_s_all_rolled_back": 1e3 / pair_ms[False],
                      "note": "NpuDecoder::Step(tokens, 2) + Resolve through gufo_cuda_decoder_step_tokens; "
                              "not the headline metric"},
        "cpu_baseline": base,
        "clocks": clocks.summary(),
    }
    print(json.dumps(line))


# DRAM traffic of one 6144 x 2048 Q4_K GEMV launch: dram__bytes_read.sum + dram__bytes_write.sum
# of the kernel from one ncu capture of `bench.py --probe q4k` (7 159 040 B read, none written:
# the 24 KB of outputs are still in L2 when the kernel ends).
Q4K_GEMV_TRAFFIC_BYTES = 7159040


def run_probe(which: str) -> None:
    """A handful of launches of one kernel family on a small case (a few hundred MB on the
    device, inputs larger than L2): the program that `ncu` is pointed at."""
    from gufo_npu_b200 import _capi
    from gufo_npu_b200.backend import Context
    dev = torch.device("cuda:0")
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    ctx = Context(0, stream.cuda_stream)
    gen = torch.Generator(device=dev).manual_seed(1)
    if which in ("q4k", "q6k", "q4k_big"):
        t = Q.GGML_Q6_K if which == "q6k" else Q.GGML_Q4_K
        rows, cols, copies = {"q4k": (6144, 2048, 24), "q6k": (131072, 2048, 1), "q4k_big": (262144, 2048, 1)}[which]
        raw = Q.quantize(t, torch.randn(rows, cols, device=dev, generator=gen) * 0.02)
        keep = [raw.clone() for _ in range(copies)]
        mats = [Context._parts([(ctx.matrix_from_device(t, r.data_ptr(), rows, cols), 0, rows)]) for r in keep]
        x = torch.randn(1, cols, device=dev, generator=gen)
        y = torch.empty(1, rows, device=dev)
        for i in range(8):
            ctx.matmul_fused_device(mats[i % copies], 1, 1, y, x=x)   # one launch per product
    elif which == "step_kernel":
        # The config-2 decode step as one cooperative kernel (context option "step_kernel").
        from gufo_npu_b200.backend import CudaDecoder, CudaProjections
        ctx.set_option("step_kernel", 1)
        cfg = model_config()
        tensors = synth.build_model(cfg, seed=1, device=str(dev))
        dec = CudaDecoder(CudaProjections(ctx, cfg, tensors), tensors, max_positions=64, use_graph=False)
        for t in range(6):
            dec.step_device(t + 1)
        torch.cuda.synchronize()
        dec.status()
    elif which == "gemm":
        return probe_gemm(ctx, stream, dev, gen)
    elif which == "moe":
        return probe_moe(ctx, stream, dev, gen)
    else:
        hv, dk, nseq, sets = 16, 128, 8, 12
        st = torch.randn(sets, nseq, hv, dk, dk, device=dev, generator=gen) * 0.1
        q = torch.nn.functional.normalize(torch.randn(nseq, hv, dk, device=dev, generator=gen), dim=-1)
        k = torch.nn.functional.normalize(torch.randn(nseq, hv, dk, device=dev, generator=gen), dim=-1)
        v = torch.randn(nseq, hv, dk, device=dev, generator=gen)
        decay, beta = torch.rand(nseq, hv, device=dev, generator=gen), torch.rand(nseq, hv, device=dev, generator=gen)
        y = torch.empty(nseq, hv, dk, device=dev)
        for c in range(8):
            arr = (_capi.DeltaSeq * nseq)()
            for s in range(nseq):
                arr[s] = _capi.DeltaSeq(st[c, s].data_ptr(), 0, q[s].data_ptr(), k[s].data_ptr(), v[s].data_ptr(),
                                        decay[s].data_ptr(), beta[s].data_ptr(), y[s].data_ptr())
            ctx._check(ctx.lib.gufo_cuda_delta_rule_device(ctx.handle, arr, nseq, hv, hv, dk))
    torch.cuda.synchronize()
    print(json.dumps({"probe": which, "launches": ctx.launch_count()}))


def graph_us(stream, enqueue, rounds: int = 5) -> float:
    """Device microseconds of one replay of the work `enqueue()` puts on `stream`, captured
    into a CUDA graph (so that host launch time does not pace the kernels), median of rounds."""
    enqueue()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        enqueue()
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(rounds):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)
    return float(np.median(times))


def probe_gemm(ctx, stream, dev, gen) -> None:
    """The verify batch's FFN input product at 4B-class shapes: gate and up 9728 x 2560 Q4_K
    stacked, M = 32 / 64 / 128 packed token rows, rotating over 6 weight copies (168 MB, larger
    than L2). Prints device time per product with its HBM and tensor-core rates."""
    from gufo_npu_b200.backend import Context
    rows, cols, copies = 9728, 2560, 6
    peak, _ = measured_peaks()
    sets = []
    keep = []
    for _ in range(copies):
        parts = []
        for _ in range(2):
            raw = Q.quantize(Q.GGML_Q4_K, torch.randn(rows, cols, device=dev, generator=gen) * 0.02)
            keep.append(raw)
            parts.append((ctx.matrix_from_device(Q.GGML_Q4_K, raw.data_ptr(), rows, cols), 0, rows))
        sets.append(Context._parts(parts))
    weight_bytes = 2 * rows * Q.row_bytes(Q.GGML_Q4_K, cols)
    out = {"probe": "gemm", "shape": f"2 x {rows} x {cols} Q4_K", "results": []}
    for m in (32, 64, 128):
        x = torch.randn(m, cols, device=dev, generator=gen)
        y = torch.empty(m, 2 * rows, device=dev)

        def enqueue():
            for c in range(copies):
                ctx.matmul_device(sets[c], 2, x, m, y)
        us = graph_us(stream, enqueue) / copies
        algorithmic = weight_bytes + 4 * m * cols + 4 * m * 2 * rows
        out["results"].append({"tokens": m, "us": us, "GB/s": algorithmic / us / 1e3,
                               "hbm_frac": algorithmic / us / 1e3 / peak,
                               "TFLOP/s": 2.0 * m * 2 * rows * cols / us / 1e6})
    # The verify batch's LM head at 4B-class shapes: 248320 x 2560 Q6_K (521 MB, one copy: larger
    # than L2 by itself).
    del sets, keep
    rows = 248320
    raw = Q.quantize(Q.GGML_Q6_K, torch.randn(rows, cols, device=dev, generator=gen) * 0.02)
    head = Context._parts([(ctx.matrix_from_device(Q.GGML_Q6_K, raw.data_ptr(), rows, cols), 0, rows)])
    weight_bytes = rows * Q.row_bytes(Q.GGML_Q6_K, cols)
    out["lm_head"] = {"shape": f"{rows} x {cols} Q6_K", "results": []}
    for m in (32, 128):
        x = torch.randn(m, cols, device=dev, generator=gen)
        y = torch.empty(m, rows, device=dev)
        us = graph_us(stream, lambda: ctx.matmul_device(head, 1, x, m, y))
        algorithmic = weight_bytes + 4 * m * cols + 4 * m * rows
        out["lm_head"]["results"].append({"tokens": m, "us": us, "GB/s": algorithmic / us / 1e3,
                                          "hbm_frac": algorithmic / us / 1e3 / peak,
                                          "TFLOP/s": 2.0 * m * rows * cols / us / 1e6})
    ctx.synchronize()
    out["launches"] = ctx.launch_count()
    print(json.dumps(out))


def probe_moe(ctx, stream, dev, gen) -> None:
    """One MoE token-layer at 35B-A3B-class shapes: hidden 2048, 256 experts of width 512 (Q4_K,
    453 MB per bank, two banks alternated), top-8 routing of N(0,1) router logits on the device,
    grouped expert products, weighted sum; 1 to 4 tokens."""
    from gufo_npu_b200 import _capi
    hidden, ef, experts, k, banks = 2048, 512, 256, 8, 2
    peak, _ = measured_peaks()
    keep, handles = [], []
    for _ in range(banks):
        ids = []
        for rows, cols in ((ef, hidden), (ef, hidden), (hidden, ef)):
            raw = Q.quantize(Q.GGML_Q4_K, torch.randn(experts * rows, cols, device=dev, generator=gen) * 0.02)
            keep.append(raw)
            ids.append(ctx.matrix_from_device(Q.GGML_Q4_K, raw.data_ptr(), experts * rows, cols))
        handles.append(_capi.ExpertBank(*ids, experts, ef, hidden))
    per_expert = 2 * ef * Q.row_bytes(Q.GGML_Q4_K, hidden) + hidden * Q.row_bytes(Q.GGML_Q4_K, ef)
    out = {"probe": "moe", "shape": f"{experts} experts x (2 x {ef} x {hidden} + {hidden} x {ef}) Q4_K, top-{k}",
           "results": []}
    rounds = 6
    for tokens in (1, 2, 4):
        logits = torch.randn(rounds, tokens, experts + 1, device=dev, generator=gen)
        x = torch.randn(tokens, hidden, device=dev, generator=gen)
        shared = torch.randn(tokens, hidden, device=dev, generator=gen)
        chosen = torch.empty(tokens, k, dtype=torch.int32, device=dev)
        weights = torch.empty(tokens, k, device=dev)
        scale = torch.empty(tokens, device=dev)
        ffn = torch.empty(tokens * k, 2 * ef, device=dev)
        act = torch.empty(tokens * k, ef, device=dev)
        rows_out = torch.empty(tokens, k, hidden, device=dev)
        y = torch.empty(tokens, hidden, device=dev)

        def enqueue():
            for r in range(rounds):
                ctx.route_device(logits[r], experts + 1, tokens, experts, k, chosen, weights, scale)
                ctx.moe_ffn_device(handles[r % banks], chosen, weights, scale, tokens, k, x, hidden, shared, ffn, act,
                                   rows_out, y)
        us = graph_us(stream, enqueue) / rounds
        algorithmic = tokens * k * per_expert
        out["results"].append({"tokens": tokens, "us": us, "GB/s": algorithmic / us / 1e3,
                               "hbm_frac": algorithmic / us / 1e3 / peak})
    ctx.synchronize()
    out["launches"] = ctx.launch_count()
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--probe", default=None, choices=["q4k", "q4k_big", "q6k", "deltanet", "gemm", "moe", "step_kernel"],
                    help="run a few launches of one kernel on a small case (for ncu) and exit")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    if args.probe:
        return run_probe(args.probe)
    if args.impl == "reference":
        return run_reference(args)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU path")
    run_ours(args)


if __name__ == "__main__":
    main()
