"""CPU restatement of the reference's gated decode attention over an fp16 cache.

Test infrastructure only: the product path never imports this. It follows
Mixer::Attention (src/models/qwen35/decoder.cpp:267-412 in the reference): q / k RMSNorm,
rotary embedding on the first rope_dim values of a head (pairs i, i + rope_dim / 2, angle =
position * inv_freq[i] taken in double), k and v appended to the cache as fp16, scores
q . k / sqrt(head_dim) over every cached position, softmax, weighted fp16 values, then the
output gate sigmoid(gate) read from the same input row. The reference cuts the positions into
slices and merges partial softmaxes (lines 326-411); a softmax is independent of that split
up to rounding, so this restatement takes it in one piece in double.

Pinned through the decoder: tests/golden/decoder_long.npz holds the reference's own logits
after more than a thousand positions of a model with an attention layer, and the CUDA
attention that passes that check is compared with this function on the same inputs.
"""
from __future__ import annotations

import numpy as np


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """vec::RmsNorm (src/core/vec.hpp:57-63) in fp32."""
    x = x.astype(np.float32)
    inv = np.float32(1.0) / np.sqrt(np.float32(np.sum(x.astype(np.float64) ** 2) / x.size) + np.float32(eps))
    return (x * inv * w.astype(np.float32)).astype(np.float32)


def rope(x: np.ndarray, position: int, inv_freq: np.ndarray) -> np.ndarray:
    """decoder.cpp:283-302: rotates (x[i], x[i + half]) by position * inv_freq[i]."""
    half = inv_freq.size
    angle = float(position) * inv_freq.astype(np.float64)
    cs, sn = np.cos(angle).astype(np.float32), np.sin(angle).astype(np.float32)
    out = x.astype(np.float32).copy()
    a, b = x[:half].astype(np.float32), x[half:2 * half].astype(np.float32)
    out[:half] = a * cs - b * sn
    out[half:2 * half] = a * sn + b * cs
    return out


def attention_step(row: np.ndarray, position: int, keys: np.ndarray, values: np.ndarray, *, heads: int,
                   kv_heads: int, head_dim: int, q_norm: np.ndarray, k_norm: np.ndarray, inv_freq: np.ndarray,
                   rms_eps: float) -> np.ndarray:
    """One token at `position`. `row` = [per query head: q | gate] + k + v (the kAttentionIn
    product's output). `keys` / `values` are fp16 [max_positions][kv_heads * head_dim] holding
    rows 0 .. position - 1; row `position` is written. Returns ctx [heads * head_dim]."""
    hd = head_dim
    kv = kv_heads * hd
    group = heads // kv_heads
    k = row[2 * heads * hd: 2 * heads * hd + kv]
    v = row[2 * heads * hd + kv: 2 * heads * hd + 2 * kv]
    for kh in range(kv_heads):
        head = rope(rms_norm(k[kh * hd:(kh + 1) * hd], k_norm, rms_eps), position, inv_freq)
        keys[position, kh * hd:(kh + 1) * hd] = head.astype(np.float16)
    values[position] = v.astype(np.float16)
    length = position + 1
    out = np.zeros(heads * hd, dtype=np.float32)
    scale = 1.0 / np.sqrt(float(hd))
    for qh in range(heads):
        kh = qh // group
        q = rope(rms_norm(row[qh * 2 * hd: qh * 2 * hd + hd], q_norm, rms_eps), position, inv_freq)
        gate = row[qh * 2 * hd + hd: (qh + 1) * 2 * hd].astype(np.float64)
        kk = keys[:length, kh * hd:(kh + 1) * hd].astype(np.float64)
        vv = values[:length, kh * hd:(kh + 1) * hd].astype(np.float64)
        s = kk @ q.astype(np.float64) * scale
        p = np.exp(s - s.max())
        ctx = (p / p.sum()) @ vv
        out[qh * hd:(qh + 1) * hd] = (ctx / (1.0 + np.exp(-gate))).astype(np.float32)
    return out
