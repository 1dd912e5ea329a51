"""Deterministic GGUF Q4_K / Q6_K quantizers for synthetic weights.

The reference ships only dequantizers for these types (src/core/quant.cpp:33-59,
98-125), so synthetic matrices for tests and benchmarks are packed here. These
are plain min/max fits written for this project: quality does not matter for
parity (both sides consume the same bytes); the output only has to be a valid
block stream with finite fp16 scales that exercises every code value.

Everything is torch, so the same code packs small test matrices on the CPU and
benchmark-sized ones on the GPU. Inputs are fp32 [rows, cols], cols % 256 == 0;
outputs are uint8 [rows, cols // 256 * block_bytes], row-major like a GGUF
tensor (src/core/quant.cpp:202-219 for the block sizes).
"""
from __future__ import annotations

import torch

GGML_F32 = 0
GGML_F16 = 1
GGML_Q8_0 = 8
GGML_Q4_K = 12
GGML_Q5_K = 13
GGML_Q6_K = 14
GGML_BF16 = 30

BLOCK_ELEMENTS = {GGML_F32: 1, GGML_F16: 1, GGML_BF16: 1, GGML_Q8_0: 32,
                  GGML_Q4_K: 256, GGML_Q5_K: 256, GGML_Q6_K: 256}
BLOCK_BYTES = {GGML_F32: 4, GGML_F16: 2, GGML_BF16: 2, GGML_Q8_0: 34,
               GGML_Q4_K: 144, GGML_Q5_K: 176, GGML_Q6_K: 210}


def row_bytes(ggml_type: int, cols: int) -> int:
    per = BLOCK_ELEMENTS[ggml_type]
    if cols % per:
        raise ValueError("row is not a whole number of blocks")
    return cols // per * BLOCK_BYTES[ggml_type]


def _half_bytes(x: torch.Tensor) -> torch.Tensor:
    """fp32 [...] -> the two little-endian bytes of its fp16 rounding, [..., 2]."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def _round_half_up(x: torch.Tensor) -> torch.Tensor:
    return torch.floor(x + 0.5)


def quantize_q4_k(w: torch.Tensor) -> torch.Tensor:
    """Min/max fit per 32-value sub-block: w ~ d*sc_j*q - dmin*m_j."""
    rows, cols = w.shape
    if cols % 256:
        raise ValueError("Q4_K rows must be a multiple of 256 values")
    nb = cols // 256
    sub = w.reshape(rows, nb, 8, 32).float()
    low = torch.clamp(sub.amin(dim=-1), max=0.0)          # <= 0
    high = sub.amax(dim=-1)
    step = (high - low) / 15.0                            # per sub-block
    offset = -low                                         # >= 0
    # Super-block fp16 scales so that the 6-bit fields reach 63 at the extreme.
    d = (step.amax(dim=-1) / 63.0).to(torch.float16)
    dmin = (offset.amax(dim=-1) / 63.0).to(torch.float16)
    d32 = d.float().unsqueeze(-1)
    dmin32 = dmin.float().unsqueeze(-1)
    sc = torch.where(d32 > 0, _round_half_up(step / d32.clamp_min(1e-30)), torch.zeros_like(step))
    sc = sc.clamp(0, 63)
    m = torch.where(dmin32 > 0, _round_half_up(offset / dmin32.clamp_min(1e-30)), torch.zeros_like(offset))
    m = m.clamp(0, 63)
    eff = (d32 * sc).unsqueeze(-1)                        # d * sc_j
    off = (dmin32 * m).unsqueeze(-1)                      # dmin * m_j
    q = torch.where(eff > 0, _round_half_up((sub + off) / eff.clamp_min(1e-30)), torch.zeros_like(sub))
    q = q.clamp(0, 15).to(torch.uint8)                    # [rows, nb, 8, 32]
    sc = sc.to(torch.uint8)
    m = m.to(torch.uint8)

    out = torch.empty(rows, nb, 144, dtype=torch.uint8, device=w.device)
    out[..., 0:2] = _half_bytes(d.float())
    out[..., 2:4] = _half_bytes(dmin.float())
    # 12 scale bytes: the inverse of quant::ScaleMinK4 (src/core/quant.cpp:158-167).
    out[..., 4:8] = sc[..., 0:4] | ((sc[..., 4:8] >> 4) << 6)
    out[..., 8:12] = m[..., 0:4] | ((m[..., 4:8] >> 4) << 6)
    out[..., 12:16] = (sc[..., 4:8] & 0x0F) | ((m[..., 4:8] & 0x0F) << 4)
    # Byte l of pair p: low nibble = sub-block 2p, high nibble = sub-block 2p+1.
    pairs = q.reshape(rows, nb, 4, 2, 32)
    out[..., 16:144] = (pairs[..., 0, :] | (pairs[..., 1, :] << 4)).reshape(rows, nb, 128)
    return out.reshape(rows, nb * 144)


def quantize_q6_k(w: torch.Tensor) -> torch.Tensor:
    """Signed fit per 16-value group: w ~ d*sc_g*(q - 32), q in [0, 63]."""
    rows, cols = w.shape
    if cols % 256:
        raise ValueError("Q6_K rows must be a multiple of 256 values")
    nb = cols // 256
    grp = w.reshape(rows, nb, 16, 16).float()
    # The element of largest magnitude lands on code -32, so the group's scale
    # carries its sign (exercises negative int8 scales).
    idx = grp.abs().argmax(dim=-1, keepdim=True)
    extreme = torch.gather(grp, -1, idx).squeeze(-1)
    scale = -extreme / 32.0
    d = (scale.abs().amax(dim=-1) / 127.0).to(torch.float16)
    d32 = d.float().unsqueeze(-1)
    sc = torch.where(d32 > 0, torch.round(scale / d32.clamp_min(1e-30)), torch.zeros_like(scale))
    sc = sc.clamp(-127, 127)
    eff = (d32 * sc).unsqueeze(-1)
    safe = torch.where(eff == 0, torch.ones_like(eff), eff)
    q = torch.where(eff != 0, torch.round(grp / safe), torch.zeros_like(grp))
    q = (q.clamp(-32, 31) + 32).to(torch.uint8).reshape(rows, nb, 2, 4, 32)  # [half][k][l]

    out = torch.empty(rows, nb, 210, dtype=torch.uint8, device=w.device)
    lo = q & 0x0F
    hi = q >> 4
    ql = torch.empty(rows, nb, 2, 64, dtype=torch.uint8, device=w.device)
    ql[..., 0:32] = lo[..., 0, :] | (lo[..., 2, :] << 4)
    ql[..., 32:64] = lo[..., 1, :] | (lo[..., 3, :] << 4)
    qh = hi[..., 0, :] | (hi[..., 1, :] << 2) | (hi[..., 2, :] << 4) | (hi[..., 3, :] << 6)
    out[..., 0:128] = ql.reshape(rows, nb, 128)
    out[..., 128:192] = qh.reshape(rows, nb, 64)
    out[..., 192:208] = sc.to(torch.int8).view(torch.uint8)
    out[..., 208:210] = _half_bytes(d.float())
    return out.reshape(rows, nb * 210)


def quantize(ggml_type: int, w: torch.Tensor) -> torch.Tensor:
    """fp32 [rows, cols] -> row-major block bytes of `ggml_type` (uint8 2-D)."""
    if ggml_type == GGML_Q4_K:
        return quantize_q4_k(w)
    if ggml_type == GGML_Q6_K:
        return quantize_q6_k(w)
    if ggml_type == GGML_F32:
        return w.float().contiguous().view(torch.uint8).reshape(w.shape[0], -1)
    raise ValueError(f"no quantizer for ggml type {ggml_type}")


def random_blocks(ggml_type: int, rows: int, cols: int, seed: int) -> torch.Tensor:
    """Random block bytes with normal fp16 scales of magnitude 2^-10 .. 2^-1.

    Every bit pattern of codes, 6-bit scales/mins and int8 scales occurs; the
    construction follows the reference's fused-dot test
    (tests/models/qwen35/gguf_dot_test.cpp:24-72).
    """
    g = torch.Generator().manual_seed(seed)
    nb = cols // BLOCK_ELEMENTS[ggml_type]
    bb = BLOCK_BYTES[ggml_type]
    raw = torch.randint(0, 256, (rows, nb, bb), generator=g, dtype=torch.uint8)
    offsets = {GGML_Q4_K: (0, 2), GGML_Q5_K: (0, 2), GGML_Q6_K: (208,), GGML_Q8_0: (0,)}[ggml_type]
    for at in offsets:
        sign = torch.randint(0, 2, (rows, nb), generator=g, dtype=torch.int32) << 15
        exponent = (5 + torch.randint(0, 10, (rows, nb), generator=g, dtype=torch.int32)) << 10
        mantissa = torch.randint(0, 1024, (rows, nb), generator=g, dtype=torch.int32)
        half = sign | exponent | mantissa
        raw[..., at] = (half & 0xFF).to(torch.uint8)
        raw[..., at + 1] = (half >> 8).to(torch.uint8)
    return raw.reshape(rows, nb * bb)
