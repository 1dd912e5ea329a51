"""ctypes binding of libgufo_cuda.so, the C ABI declared in include/gufo_cuda.h.

There is no fallback: if the library is missing or no sm_100 device is usable,
loading or context creation raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libgufo_cuda.so")

OK = 0
STATUS_TIMEOUT = 6
STATUS_UNSUPPORTED_TYPE = 3
STATUS_NAMES = {1: "bad argument", 2: "shape", 3: "unsupported type", 4: "CUDA runtime",
                5: "out of memory", 6: "timeout", 7: "too large"}

_f32p = C.POINTER(C.c_float)


class GufoCudaError(RuntimeError):
    def __init__(self, status: int, text: str):
        super().__init__(f"gufo_cuda status {status} ({STATUS_NAMES.get(status, '?')}): {text}")
        self.status = status


class Rows(C.Structure):
    """gufo_cuda_rows: rows [first, first + rows) of a matrix handle."""
    _fields_ = [("w", C.c_int64), ("first", C.c_int64), ("rows", C.c_int64)]


class DeltaSeq(C.Structure):
    _fields_ = [("state", C.c_void_p), ("state_out", C.c_void_p), ("q", C.c_void_p), ("k", C.c_void_p),
                ("v", C.c_void_p), ("decay", C.c_void_p), ("beta", C.c_void_p), ("y", C.c_void_p)]


class LinearSeq(C.Structure):
    _fields_ = [("in_", C.c_void_p), ("conv_in", C.c_void_p), ("conv_out", C.c_void_p),
                ("ssm", C.c_void_p), ("ssm_out", C.c_void_p), ("y", C.c_void_p)]


class DeltaNetStepSeq(C.Structure):
    _fields_ = [("n_tokens", C.c_int), ("in_", C.c_void_p), ("in_stride", C.c_int64), ("h", C.c_void_p),
                ("h_stride", C.c_int64), ("conv_in", C.c_void_p), ("conv_out", C.c_void_p),
                ("conv_saved", C.c_void_p), ("ssm", C.c_void_p), ("ssm_spec", C.c_void_p), ("y", C.c_void_p),
                ("y_stride", C.c_int64)]


class DeltaNetParams(C.Structure):
    _fields_ = [("key_heads", C.c_int), ("value_heads", C.c_int), ("head_dim", C.c_int),
                ("conv_kernel", C.c_int), ("rms_eps", C.c_float), ("conv", _f32p), ("ssm_a", _f32p),
                ("dt_bias", _f32p), ("ssm_norm", _f32p)]


class AttentionArgs(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("heads", "kv_heads", "head_dim", "rope_dim", "max_positions")] + \
               [("rms_eps", C.c_float)] + \
               [(n, C.c_void_p) for n in ("position", "in_", "q_norm", "k_norm", "inv_freq", "keys", "values",
                                          "queries", "partials", "ctx_out")]


class FusedInput(C.Structure):
    """gufo_cuda_fused_input."""
    _fields_ = [("prologue", C.c_int), ("x", C.c_void_p), ("residual", C.c_void_p), ("delta", C.c_void_p),
                ("norm_weight", C.c_void_p), ("rms_eps", C.c_float), ("residual_out", C.c_void_p),
                ("scratch", C.c_void_p), ("advance", C.c_void_p), ("delta_parts", C.c_int), ("delta_stride", C.c_int),
                ("epilogue", C.c_int)]


PROLOGUE_PLAIN, PROLOGUE_RES_NORM, PROLOGUE_SWIGLU = 0, 1, 2
EPILOGUE_NONE, EPILOGUE_SWIGLU = 0, 1
IPC_HANDLE_BYTES = 64
PEER_HEADER_BYTES = 4096


class DecoderConfig(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("layers", "hidden", "ffn", "vocab")] + [("rms_eps", C.c_float)] + \
               [(n, C.c_int) for n in ("full_attention_interval", "heads", "kv_heads", "head_dim", "rope_dim")] + \
               [("rope_theta", C.c_float)] + \
               [(n, C.c_int) for n in ("conv_kernel", "linear_key_heads", "linear_value_heads", "linear_head_dim",
                                       "max_positions", "use_graph", "experts", "experts_used", "expert_ffn")]


LAYER_MATRICES = ("attn_qkv", "attn_gate", "ssm_alpha", "ssm_beta", "ssm_out", "attn_q", "attn_k", "attn_v",
                  "attn_output", "ffn_gate", "ffn_up", "ffn_down", "ffn_gate_inp", "ffn_gate_inp_shexp",
                  "ffn_gate_exps", "ffn_up_exps", "ffn_down_exps")
LAYER_VECTORS = ("attn_norm", "post_attention_norm", "ssm_conv1d", "ssm_a", "ssm_dt_bias", "ssm_norm",
                 "attn_q_norm", "attn_k_norm")


class LayerWeights(C.Structure):
    _fields_ = [(n, C.c_int64) for n in LAYER_MATRICES] + [(n, _f32p) for n in LAYER_VECTORS]


class ExpertBank(C.Structure):
    _fields_ = [("gate_exps", C.c_int64), ("up_exps", C.c_int64), ("down_exps", C.c_int64),
                ("experts", C.c_int), ("expert_ffn", C.c_int), ("hidden", C.c_int)]


class DecoderWeights(C.Structure):
    _fields_ = [("token_embd", C.c_int64), ("output", C.c_int64), ("output_norm", _f32p),
                ("layers", C.POINTER(LayerWeights))]


# name -> (restype, argtypes); every symbol include/gufo_cuda.h declares.
SIGNATURES = {
    "gufo_cuda_ctx_create": (C.c_int, [C.c_int, C.c_void_p, C.POINTER(C.c_void_p)]),
    "gufo_cuda_ctx_destroy": (C.c_int, [C.c_void_p]),
    "gufo_cuda_ctx_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "gufo_cuda_ctx_synchronize": (C.c_int, [C.c_void_p]),
    "gufo_cuda_ctx_set_option": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "gufo_cuda_last_error": (C.c_char_p, [C.c_void_p]),
    "gufo_cuda_launch_count": (C.c_int64, [C.c_void_p]),
    "gufo_cuda_malloc": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "gufo_cuda_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "gufo_cuda_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "gufo_cuda_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "gufo_cuda_memset_zero": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "gufo_cuda_matrix_upload": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64,
                                          C.POINTER(C.c_int64)]),
    "gufo_cuda_matrix_from_device": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int64, C.c_int64,
                                               C.POINTER(C.c_int64)]),
    "gufo_cuda_matrix_free": (C.c_int, [C.c_void_p, C.c_int64]),
    "gufo_cuda_dequantize": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "gufo_cuda_dequantize_device": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "gufo_cuda_matmul": (C.c_int, [C.c_void_p, C.POINTER(Rows), C.c_int, C.c_void_p, C.c_int, C.c_void_p]),
    "gufo_cuda_matmul_device": (C.c_int, [C.c_void_p, C.POINTER(Rows), C.c_int, C.c_void_p, C.c_int,
                                          C.c_void_p]),
    "gufo_cuda_matmul_fused_device": (C.c_int, [C.c_void_p, C.POINTER(Rows), C.c_int, C.POINTER(FusedInput), C.c_int,
                                                C.c_void_p]),
    "gufo_cuda_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "gufo_cuda_peer_group_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p,
                                              C.POINTER(C.c_void_p)]),
    "gufo_cuda_peer_group_create_local": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_size_t,
                                                    C.POINTER(C.c_void_p)]),
    "gufo_cuda_peer_group_destroy": (C.c_int, [C.c_void_p]),
    "gufo_cuda_peer_group_set_limit": (C.c_int, [C.c_void_p, C.c_int64]),
    "gufo_cuda_peer_group_reset": (C.c_int, [C.c_void_p]),
    "gufo_cuda_peer_allgather_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t]),
    "gufo_cuda_peer_group_status": (C.c_int, [C.c_void_p]),
    "gufo_cuda_matmul_gather_device": (C.c_int, [C.c_void_p, C.POINTER(Rows), C.c_int, C.POINTER(FusedInput), C.c_size_t,
                                                 C.c_int, C.c_int]),
    "gufo_cuda_peer_wait_device": (C.c_int, [C.c_void_p, C.c_int]),
    "gufo_cuda_matmul_wait_device": (C.c_int, [C.c_void_p, C.POINTER(Rows), C.c_int, C.POINTER(FusedInput), C.c_int,
                                               C.c_void_p]),
    "gufo_cuda_matmul_q4k_static_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p,
                                                     C.c_int, C.c_void_p]),
    "gufo_cuda_delta_rule_device": (C.c_int, [C.c_void_p, C.POINTER(DeltaSeq), C.c_int, C.c_int, C.c_int,
                                              C.c_int]),
    "gufo_cuda_deltanet_layer_create": (C.c_int, [C.c_void_p, C.POINTER(DeltaNetParams),
                                                  C.POINTER(C.c_int64)]),
    "gufo_cuda_deltanet_layer_free": (C.c_int, [C.c_void_p, C.c_int64]),
    "gufo_cuda_deltanet_linear_device": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(LinearSeq), C.c_int]),
    "gufo_cuda_deltanet_step_device": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_float,
                                                 C.POINTER(DeltaNetStepSeq), C.c_int]),
    "gufo_cuda_embed_device": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p]),
    "gufo_cuda_add_rms_norm_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int,
                                                C.c_void_p, C.c_void_p]),
    "gufo_cuda_swiglu_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]),
    "gufo_cuda_attention_device": (C.c_int, [C.c_void_p, C.POINTER(AttentionArgs)]),
    "gufo_cuda_route_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                         C.c_void_p, C.c_void_p]),
    "gufo_cuda_expert_ffn_device": (C.c_int, [C.c_void_p, C.POINTER(ExpertBank), C.c_void_p, C.c_int, C.c_void_p,
                                              C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "gufo_cuda_moe_ffn_device": (C.c_int, [C.c_void_p, C.POINTER(ExpertBank), C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_int, C.c_int, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_void_p, C.c_void_p]),
    "gufo_cuda_moe_combine_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                               C.c_int, C.c_int, C.c_void_p]),
    "gufo_cuda_decoder_create": (C.c_int, [C.c_void_p, C.POINTER(DecoderConfig), C.POINTER(DecoderWeights),
                                           C.POINTER(C.c_void_p)]),
    "gufo_cuda_decoder_destroy": (C.c_int, [C.c_void_p]),
    "gufo_cuda_decoder_reset": (C.c_int, [C.c_void_p]),
    "gufo_cuda_decoder_step": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "gufo_cuda_decoder_status": (C.c_int, [C.c_void_p]),
    "gufo_cuda_decoder_step_profile": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int64),
                                                 C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "gufo_cuda_decoder_step_tokens": (C.c_int, [C.c_void_p, C.POINTER(C.c_int), C.c_int, C.c_int, C.c_void_p]),
    "gufo_cuda_decoder_resolve": (C.c_int, [C.c_void_p, C.c_int]),
    "gufo_cuda_decoder_hidden_device": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_void_p)]),
    "gufo_cuda_decoder_logits_device": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "gufo_cuda_decoder_position": (C.c_int, [C.c_void_p]),
    "gufo_cuda_decoder_timeline": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_int)]),
    "gufo_cuda_decoder_linear_state": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
}

_lib = None


def load(path: str = LIB_PATH) -> C.CDLL:
    """Loads the library and declares every entry point; raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(path):
        raise FileNotFoundError(
            f"{path} is not built: run `python -m gufo_npu_b200.build` (this backend has no CPU path)")
    lib = C.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(lib: C.CDLL, ctx, status: int) -> None:
    if status != OK:
        raise GufoCudaError(status, (lib.gufo_cuda_last_error(ctx) or b"").decode())
