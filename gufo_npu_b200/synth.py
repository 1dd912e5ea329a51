"""Synthetic Qwen3.5-shaped models: seeded tensors and their GGUF v3 image.

No model weights ship with this project, so tests and benchmarks build models
whose shapes follow the reference's Config (src/models/qwen35/config.hpp:13-62)
and whose tensor names, shapes and types are the ones the reference's loaders
check (src/models/qwen35/gguf_projections.cpp:100-175, decoder.cpp:67-98,
441-455). Projection matrices are N(0, 0.02) values packed as Q4_K or Q6_K;
the small per-layer vectors stay F32. The GGUF image lets the reference's own
`gguf::File::FromBytes` (src/core/gguf.cpp:209-216) open the same bytes the
CUDA backend uploads.
"""
from __future__ import annotations

import dataclasses
import struct
from typing import Dict, List, Tuple

import numpy as np
import torch

from . import quantize as Q


@dataclasses.dataclass
class ModelConfig:
    """Mirror of the reference's qwen35::Config (src/models/qwen35/config.hpp:13-62)."""
    layers: int = 4
    hidden: int = 256
    ffn: int = 512                 # dense FFN width (0 for MoE)
    vocab: int = 512
    rms_eps: float = 1e-6
    full_attention_interval: int = 4
    heads: int = 2
    kv_heads: int = 1
    head_dim: int = 64
    rope_dim: int = 16
    rope_theta: float = 1e7
    conv_kernel: int = 4
    linear_key_heads: int = 2
    linear_value_heads: int = 2
    linear_head_dim: int = 128
    experts: int = 0
    experts_used: int = 0
    expert_ffn: int = 0
    shared_expert_ffn: int = 0
    tied_embeddings: bool = True
    # MTP (next-token prediction) layers stored after the decoder layers: blk.<layers> holds
    # nextn.eh_proj and a full-attention layer (src/models/qwen35/config.cpp:25-26,74-78).
    mtp_layers: int = 0
    # Types of the stored matrices.
    proj_type: int = Q.GGML_Q4_K
    down_type: int = Q.GGML_Q6_K
    embed_type: int = Q.GGML_Q6_K

    @property
    def is_moe(self) -> bool:
        return self.experts > 0

    @property
    def ffn_width(self) -> int:
        return self.shared_expert_ffn if self.is_moe else self.ffn

    def is_full_attention(self, layer: int) -> bool:
        if layer >= self.layers:
            return True   # the MTP layer (Config::IsFullAttention, config.hpp:52-54)
        return layer >= self.layers or (layer + 1) % self.full_attention_interval == 0

    @property
    def key_dim(self) -> int:
        return self.linear_key_heads * self.linear_head_dim

    @property
    def value_dim(self) -> int:
        return self.linear_value_heads * self.linear_head_dim

    @property
    def conv_channels(self) -> int:
        return 2 * self.key_dim + self.value_dim

    @property
    def architecture(self) -> str:
        return "qwen35moe" if self.is_moe else "qwen35"


@dataclasses.dataclass
class Tensor:
    """A GGUF tensor: ggml shape (contiguous dimension first) and its raw bytes."""
    shape: Tuple[int, ...]
    ggml_type: int
    data: torch.Tensor  # uint8, 1-D, on any device

    @property
    def cols(self) -> int:
        return self.shape[0]

    @property
    def rows(self) -> int:
        n = 1
        for d in self.shape[1:]:
            n *= d
        return n


def _matrix(gen: torch.Generator, rows: int, cols: int, ggml_type: int, device, std: float = 0.02,
            chunk_rows: int = 16384) -> torch.Tensor:
    """N(0, std) fp32 [rows, cols] packed as `ggml_type`, generated in row chunks."""
    parts = []
    for r0 in range(0, rows, chunk_rows):
        n = min(chunk_rows, rows - r0)
        w = torch.randn(n, cols, generator=gen, device=device, dtype=torch.float32) * std
        parts.append(Q.quantize(ggml_type, w).reshape(-1))
    return torch.cat(parts) if len(parts) > 1 else parts[0]


def _f32(values: torch.Tensor) -> torch.Tensor:
    return values.float().contiguous().view(torch.uint8).reshape(-1)


def build_model(cfg: ModelConfig, seed: int = 1, device: str = "cpu") -> Dict[str, Tensor]:
    """Seeded tensors of a dense (`qwen35`) or MoE (`qwen35moe`) model."""
    gen = torch.Generator(device=device).manual_seed(seed)
    t: Dict[str, Tensor] = {}

    def mat(name: str, cols: int, rows: int, ggml_type: int, experts: int = 0):
        data = _matrix(gen, rows * max(experts, 1), cols, ggml_type, device)
        shape = (cols, rows, experts) if experts else (cols, rows)
        t[name] = Tensor(shape, ggml_type, data)

    def vec(name: str, values: torch.Tensor, shape=None):
        t[name] = Tensor(tuple(shape) if shape else (values.numel(),), Q.GGML_F32, _f32(values))

    def rand(*shape, std=1.0):
        return torch.randn(*shape, generator=gen, device=device, dtype=torch.float32) * std

    c = cfg
    mat("token_embd.weight", c.hidden, c.vocab, c.embed_type)
    if not c.tied_embeddings:
        mat("output.weight", c.hidden, c.vocab, c.embed_type)
    vec("output_norm.weight", 1.0 + rand(c.hidden, std=0.1))
    attn_dim = c.heads * c.head_dim
    kv_dim = c.kv_heads * c.head_dim
    for il in range(c.layers):
        p = f"blk.{il}."
        vec(p + "attn_norm.weight", 1.0 + rand(c.hidden, std=0.1))
        vec(p + "post_attention_norm.weight", 1.0 + rand(c.hidden, std=0.1))
        if c.is_full_attention(il):
            mat(p + "attn_q.weight", c.hidden, 2 * attn_dim, c.proj_type)
            mat(p + "attn_k.weight", c.hidden, kv_dim, c.proj_type)
            mat(p + "attn_v.weight", c.hidden, kv_dim, c.proj_type)
            mat(p + "attn_output.weight", attn_dim, c.hidden, c.proj_type)
            vec(p + "attn_q_norm.weight", 1.0 + rand(c.head_dim, std=0.1))
            vec(p + "attn_k_norm.weight", 1.0 + rand(c.head_dim, std=0.1))
        else:
            mat(p + "attn_qkv.weight", c.hidden, c.conv_channels, c.proj_type)
            mat(p + "attn_gate.weight", c.hidden, c.value_dim, c.proj_type)
            vec(p + "ssm_alpha.weight", rand(c.linear_value_heads, c.hidden, std=0.02),
                (c.hidden, c.linear_value_heads))
            vec(p + "ssm_beta.weight", rand(c.linear_value_heads, c.hidden, std=0.02),
                (c.hidden, c.linear_value_heads))
            mat(p + "ssm_out.weight", c.value_dim, c.hidden, c.proj_type)
            vec(p + "ssm_conv1d.weight", rand(c.conv_channels, c.conv_kernel, std=0.4),
                (c.conv_kernel, c.conv_channels))
            # ssm_a = -exp(A_log): negative, order one.
            vec(p + "ssm_a", -torch.exp(rand(c.linear_value_heads, std=0.5)))
            vec(p + "ssm_dt.bias", rand(c.linear_value_heads))
            vec(p + "ssm_norm.weight", 1.0 + rand(c.linear_head_dim, std=0.1))
        suffix = "_shexp.weight" if c.is_moe else ".weight"
        mat(p + "ffn_gate" + suffix, c.hidden, c.ffn_width, c.proj_type)
        mat(p + "ffn_up" + suffix, c.hidden, c.ffn_width, c.proj_type)
        mat(p + "ffn_down" + suffix, c.ffn_width, c.hidden, c.down_type)
        if c.is_moe:
            vec(p + "ffn_gate_inp.weight", rand(c.experts, c.hidden, std=0.05), (c.hidden, c.experts))
            vec(p + "ffn_gate_inp_shexp.weight", rand(c.hidden, std=0.05), (c.hidden,))
            mat(p + "ffn_gate_exps.weight", c.hidden, c.expert_ffn, c.proj_type, c.experts)
            mat(p + "ffn_up_exps.weight", c.hidden, c.expert_ffn, c.proj_type, c.experts)
            mat(p + "ffn_down_exps.weight", c.expert_ffn, c.hidden, c.proj_type, c.experts)
    if c.mtp_layers > 0:
        # The MTP layer, drawn after everything else so that models without one keep their
        # tensors: eh_proj over [embedding | hidden], its norms, a full-attention layer, an FFN.
        p = f"blk.{c.layers}."
        mat(p + "nextn.eh_proj.weight", 2 * c.hidden, c.hidden, c.proj_type)
        for name in ("nextn.enorm.weight", "nextn.hnorm.weight", "nextn.shared_head_norm.weight",
                     "attn_norm.weight", "post_attention_norm.weight"):
            vec(p + name, 1.0 + rand(c.hidden, std=0.1))
        mat(p + "attn_q.weight", c.hidden, 2 * attn_dim, c.proj_type)
        mat(p + "attn_k.weight", c.hidden, kv_dim, c.proj_type)
        mat(p + "attn_v.weight", c.hidden, kv_dim, c.proj_type)
        mat(p + "attn_output.weight", attn_dim, c.hidden, c.proj_type)
        vec(p + "attn_q_norm.weight", 1.0 + rand(c.head_dim, std=0.1))
        vec(p + "attn_k_norm.weight", 1.0 + rand(c.head_dim, std=0.1))
        suffix = "_shexp.weight" if c.is_moe else ".weight"
        mat(p + "ffn_gate" + suffix, c.hidden, c.ffn_width, c.proj_type)
        mat(p + "ffn_up" + suffix, c.hidden, c.ffn_width, c.proj_type)
        mat(p + "ffn_down" + suffix, c.ffn_width, c.hidden, c.down_type)
        if c.is_moe:
            vec(p + "ffn_gate_inp.weight", rand(c.experts, c.hidden, std=0.05), (c.hidden, c.experts))
            vec(p + "ffn_gate_inp_shexp.weight", rand(c.hidden, std=0.05), (c.hidden,))
            mat(p + "ffn_gate_exps.weight", c.hidden, c.expert_ffn, c.proj_type, c.experts)
            mat(p + "ffn_up_exps.weight", c.hidden, c.expert_ffn, c.proj_type, c.experts)
            mat(p + "ffn_down_exps.weight", c.expert_ffn, c.hidden, c.proj_type, c.experts)
    return t


def metadata(cfg: ModelConfig) -> List[Tuple[str, object]]:
    """The keys qwen35::ReadConfig needs (src/models/qwen35/config.cpp:18-58)."""
    a = cfg.architecture + "."
    keys: List[Tuple[str, object]] = [
        ("general.architecture", cfg.architecture),
        (a + "block_count", cfg.layers + cfg.mtp_layers),
        (a + "embedding_length", cfg.hidden),
        (a + "attention.layer_norm_rms_epsilon", float(cfg.rms_eps)),
        (a + "full_attention_interval", cfg.full_attention_interval),
        (a + "attention.head_count", cfg.heads),
        (a + "attention.head_count_kv", cfg.kv_heads),
        (a + "attention.key_length", cfg.head_dim),
        (a + "attention.value_length", cfg.head_dim),
        (a + "rope.dimension_count", cfg.rope_dim),
        (a + "rope.freq_base", float(cfg.rope_theta)),
        (a + "ssm.conv_kernel", cfg.conv_kernel),
        (a + "ssm.state_size", cfg.linear_head_dim),
        (a + "ssm.group_count", cfg.linear_key_heads),
        (a + "ssm.time_step_rank", cfg.linear_value_heads),
        (a + "ssm.inner_size", cfg.value_dim),
    ]
    if cfg.mtp_layers > 0:
        keys.append((a + "nextn_predict_layers", cfg.mtp_layers))
    if cfg.is_moe:
        keys += [(a + "expert_count", cfg.experts), (a + "expert_used_count", cfg.experts_used),
                 (a + "expert_feed_forward_length", cfg.expert_ffn),
                 (a + "expert_shared_feed_forward_length", cfg.shared_expert_ffn)]
    else:
        keys.append((a + "feed_forward_length", cfg.ffn))
    return keys


def to_gguf(cfg: ModelConfig, tensors: Dict[str, Tensor]) -> np.ndarray:
    """A GGUF v3 image (uint8 array) of `tensors` with `cfg`'s metadata.

    Layout as the reference's reader expects (src/core/gguf.cpp:224-282): header,
    key/values (uint32 = 4, float32 = 6, string = 8), tensor infos, then the data
    section aligned to 32 bytes with each tensor on a 32-byte boundary.
    """
    out = bytearray()

    def put_string(s: str):
        raw = s.encode()
        out.extend(struct.pack("<Q", len(raw)))
        out.extend(raw)

    keys = metadata(cfg)
    out.extend(struct.pack("<IIQQ", 0x46554747, 3, len(tensors), len(keys)))
    for name, value in keys:
        put_string(name)
        if isinstance(value, str):
            out.extend(struct.pack("<I", 8))
            put_string(value)
        elif isinstance(value, float):
            out.extend(struct.pack("<If", 6, value))
        else:
            out.extend(struct.pack("<II", 4, int(value)))
    offset = 0
    offsets = {}
    for name, tensor in tensors.items():
        put_string(name)
        out.extend(struct.pack("<I", len(tensor.shape)))
        for dim in tensor.shape:
            out.extend(struct.pack("<Q", dim))
        out.extend(struct.pack("<IQ", tensor.ggml_type, offset))
        offsets[name] = offset
        offset += (tensor.data.numel() + 31) // 32 * 32
    start = (len(out) + 31) // 32 * 32
    image = np.zeros(start + offset, dtype=np.uint8)
    image[:len(out)] = np.frombuffer(bytes(out), dtype=np.uint8)
    for name, tensor in tensors.items():
        at = start + offsets[name]
        image[at:at + tensor.data.numel()] = tensor.data.cpu().numpy()
    return image
