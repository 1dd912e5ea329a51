"""CPU restatement of Decoder::Step for dense models, over the C oracle's pieces.

Test infrastructure only. Follows src/models/qwen35/decoder.cpp:478-528 in the reference:
embedding row, then per layer RMSNorm -> input product -> mixer (Mixer::Linear through the C
oracle, Mixer::Attention through oracle/attention.py) -> output product -> residual add ->
RMSNorm -> gate/up product -> SwiGLU -> down product -> residual add; output norm; LM head.
tests/test_oracle.py pins it (and with it the attention restatement) to the reference's own
logits in tests/golden/decoder.npz and decoder_long.npz.
"""
from __future__ import annotations

import numpy as np

from . import attention


class OracleDecoder:
    def __init__(self, oracle, cfg, tensors, max_positions: int):
        self.o, self.c = oracle, cfg
        self.t = {k: v for k, v in tensors.items()}
        c = cfg
        self.position = 0
        self.conv = {}
        self.ssm = {}
        self.keys = {}
        self.values = {}
        for il in range(c.layers):
            if c.is_full_attention(il):
                kv = c.kv_heads * c.head_dim
                self.keys[il] = np.zeros((max_positions, kv), dtype=np.float16)
                self.values[il] = np.zeros((max_positions, kv), dtype=np.float16)
            else:
                self.conv[il] = np.zeros((c.conv_kernel - 1) * c.conv_channels, dtype=np.float32)
                self.ssm[il] = np.zeros(c.linear_value_heads * c.linear_head_dim ** 2, dtype=np.float32)
        # The reference's table (decoder.cpp:85-90).
        self.inv_freq = np.array([1.0 / (c.rope_theta ** (2.0 * i / c.rope_dim)) for i in range(c.rope_dim // 2)],
                                 dtype=np.float32)

    def _f32(self, name):
        return self.t[name].data.numpy().view(np.float32).copy()

    def _rows(self, names):
        return [(self.t[n].data.numpy().reshape(self.t[n].rows, -1), self.t[n].ggml_type, 0, self.t[n].rows)
                for n in names]

    def _product(self, names, x):
        t = self.t[names[0]]
        return self.o.matmul(self._rows(names), t.cols, np.ascontiguousarray(x, dtype=np.float32))[0]

    def step(self, token: int) -> np.ndarray:
        c, o = self.c, self.o
        embed = self.t["token_embd.weight"]
        row = embed.data.numpy().reshape(embed.rows, -1)[token]
        h = o.dequantize(embed.ggml_type, row, c.hidden).astype(np.float32)
        for il in range(c.layers):
            p = f"blk.{il}."
            normed = o.rms_norm(h.copy(), self._f32(p + "attn_norm.weight"), c.rms_eps)
            if c.is_full_attention(il):
                x_in = self._product([p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"], normed)
                mixed = attention.attention_step(
                    x_in, self.position, self.keys[il], self.values[il], heads=c.heads, kv_heads=c.kv_heads,
                    head_dim=c.head_dim, q_norm=self._f32(p + "attn_q_norm.weight"),
                    k_norm=self._f32(p + "attn_k_norm.weight"), inv_freq=self.inv_freq, rms_eps=c.rms_eps)
                out = self._product([p + "attn_output.weight"], mixed)
            else:
                x_in = self._product([p + "attn_qkv.weight", p + "attn_gate.weight", p + "ssm_alpha.weight",
                                      p + "ssm_beta.weight"], normed)
                cfg = {"key_heads": c.linear_key_heads, "value_heads": c.linear_value_heads,
                       "head_dim": c.linear_head_dim, "conv_kernel": c.conv_kernel, "rms_eps": c.rms_eps}
                weights = {"conv": self._f32(p + "ssm_conv1d.weight"), "ssm_a": self._f32(p + "ssm_a"),
                           "dt_bias": self._f32(p + "ssm_dt.bias"), "ssm_norm": self._f32(p + "ssm_norm.weight")}
                mixed, _ = o.deltanet_linear(cfg, weights, x_in, self.conv[il], self.ssm[il])
                out = self._product([p + "ssm_out.weight"], mixed)
            h = (h + out).astype(np.float32)
            normed = o.rms_norm(h.copy(), self._f32(p + "post_attention_norm.weight"), c.rms_eps)
            ffn = self._product([p + "ffn_gate.weight", p + "ffn_up.weight"], normed)
            f = c.ffn_width
            gate = ffn[:f].astype(np.float32)
            act = (gate / (np.float32(1.0) + np.exp(-gate)) * ffn[f:]).astype(np.float32)
            h = (h + self._product([p + "ffn_down.weight"], act)).astype(np.float32)
        self.position += 1
        normed = o.rms_norm(h.copy(), self._f32("output_norm.weight"), c.rms_eps)
        head = "token_embd.weight" if c.tied_embeddings else "output.weight"
        return self._product([head], normed)
