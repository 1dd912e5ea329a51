"""ctypes bindings for the two oracle libraries: TEST INFRASTRUCTURE ONLY.

`Oracle`  - libgufo_oracle.so, the plain-C restatement (gufo_oracle.c).
`RefLib`  - _ref/libgufo_ref.so, the reference's own sources behind ref_shim.cpp
            (present when it was built where the reference tree is mounted).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libgufo_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libgufo_ref.so")

_f32p = C.POINTER(C.c_float)
_u8p = C.POINTER(C.c_uint8)
_i32p = C.POINTER(C.c_int)


def build(reference: str | None = None) -> None:
    """Runs oracle/Makefile (the restatement, and _ref when the reference tree exists).
    `reference` is the reference checkout; by default the environment's GUFO_REFERENCE,
    else a directory named "reference" beside this repository (neither: only the
    restatement is built)."""
    if reference is None:
        beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
        reference = os.environ.get("GUFO_REFERENCE") or (beside if os.path.isdir(beside) else "")
    subprocess.run(["make", "-C", HERE, f"REFERENCE={reference}"], check=True,
                   stdout=subprocess.DEVNULL)


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags.c_contiguous
    return a.ctypes.data_as(_f32p)


def _bp(a: np.ndarray):
    assert a.dtype == np.uint8 and a.flags.c_contiguous
    return a.ctypes.data_as(_u8p)


class OracleRows(C.Structure):
    _fields_ = [("data", _u8p), ("type", C.c_int), ("first", C.c_size_t), ("rows", C.c_size_t)]


class DeltaNetLayer(C.Structure):
    _fields_ = [("key_heads", C.c_int), ("value_heads", C.c_int), ("head_dim", C.c_int),
                ("conv_kernel", C.c_int), ("rms_eps", C.c_float), ("conv", _f32p),
                ("ssm_a", _f32p), ("dt_bias", _f32p), ("ssm_norm", _f32p)]


class Oracle:
    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        lib = C.CDLL(path)
        lib.gufo_oracle_half_to_float.restype = C.c_float
        lib.gufo_oracle_half_to_float.argtypes = [C.c_uint16]
        lib.gufo_oracle_dequantize.restype = C.c_int
        lib.gufo_oracle_dequantize.argtypes = [C.c_int, _u8p, _f32p, C.c_size_t]
        lib.gufo_oracle_dot.restype = C.c_float
        lib.gufo_oracle_dot.argtypes = [C.c_int, _u8p, _f32p, C.c_size_t]
        lib.gufo_oracle_dot_double.restype = C.c_float
        lib.gufo_oracle_dot_double.argtypes = [C.c_int, _u8p, _f32p, C.c_size_t]
        lib.gufo_oracle_row_bytes.restype = C.c_size_t
        lib.gufo_oracle_row_bytes.argtypes = [C.c_int, C.c_size_t]
        lib.gufo_oracle_matmul.restype = C.c_int
        lib.gufo_oracle_matmul.argtypes = [C.POINTER(OracleRows), C.c_int, C.c_size_t, _f32p,
                                           C.c_int, _f32p, C.c_int]
        lib.gufo_oracle_delta_rule.restype = None
        lib.gufo_oracle_delta_rule.argtypes = [_f32p, _f32p, C.c_int, _f32p, _f32p, _f32p,
                                               C.c_float, C.c_float, _f32p]
        lib.gufo_oracle_deltanet_linear.restype = None
        lib.gufo_oracle_deltanet_linear.argtypes = [C.POINTER(DeltaNetLayer), _f32p, _f32p, _f32p,
                                                    _f32p, _f32p]
        lib.gufo_oracle_route.restype = None
        lib.gufo_oracle_route.argtypes = [_f32p, C.c_int, C.c_int, _i32p, _f32p]
        lib.gufo_oracle_shared_expert_scale.restype = C.c_float
        lib.gufo_oracle_shared_expert_scale.argtypes = [C.c_float]
        lib.gufo_oracle_scale_min_k4.restype = None
        lib.gufo_oracle_scale_min_k4.argtypes = [C.c_size_t, _u8p, _u8p, _u8p]
        lib.gufo_oracle_rms_norm.restype = None
        lib.gufo_oracle_rms_norm.argtypes = [_f32p, _f32p, C.c_int, C.c_float, _f32p]
        self.lib = lib

    def half_to_float(self, bits: int) -> float:
        return float(self.lib.gufo_oracle_half_to_float(bits))

    def row_bytes(self, ggml_type: int, n: int) -> int:
        return int(self.lib.gufo_oracle_row_bytes(ggml_type, n))

    def dequantize(self, ggml_type: int, raw: np.ndarray, n: int) -> np.ndarray:
        raw = np.ascontiguousarray(raw.reshape(-1))
        out = np.empty(n, dtype=np.float32)
        if self.lib.gufo_oracle_dequantize(ggml_type, _bp(raw), _fp(out), n) != 0:
            raise ValueError("oracle dequantize: bad type or partial block")
        return out

    def dot(self, ggml_type: int, row: np.ndarray, x: np.ndarray, exact: bool = False) -> float:
        row = np.ascontiguousarray(row.reshape(-1))
        fn = self.lib.gufo_oracle_dot_double if exact else self.lib.gufo_oracle_dot
        return float(fn(ggml_type, _bp(row), _fp(x), x.size))

    def matmul(self, parts, cols: int, x: np.ndarray, exact: bool = False) -> np.ndarray:
        """parts: [(bytes uint8 2-D [rows_total, row_bytes], type, first, rows)]; x [tokens, cols]."""
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, cols)
        arr = (OracleRows * len(parts))()
        keep = []
        total = 0
        for i, (data, t, first, rows) in enumerate(parts):
            data = np.ascontiguousarray(data)
            keep.append(data)
            arr[i] = OracleRows(_bp(data.reshape(-1)), t, first, rows)
            total += rows
        y = np.empty((x.shape[0], total), dtype=np.float32)
        rc = self.lib.gufo_oracle_matmul(arr, len(parts), cols, _fp(x), x.shape[0], _fp(y), int(exact))
        if rc != 0:
            raise ValueError("oracle matmul failed")
        return y

    def delta_rule(self, s: np.ndarray, k, q, v, decay: float, beta: float):
        """One head: returns (S', y) for S [dk, dk]."""
        dk = s.shape[0]
        src = np.ascontiguousarray(s, dtype=np.float32)
        dst = np.empty_like(src)
        y = np.empty(dk, dtype=np.float32)
        self.lib.gufo_oracle_delta_rule(_fp(src), _fp(dst), dk, _fp(np.ascontiguousarray(k, dtype=np.float32)),
                                        _fp(np.ascontiguousarray(q, dtype=np.float32)),
                                        _fp(np.ascontiguousarray(v, dtype=np.float32)),
                                        float(decay), float(beta), _fp(y))
        return dst, y

    def deltanet_linear(self, cfg: dict, weights: dict, x_in: np.ndarray, conv: np.ndarray,
                        ssm: np.ndarray, speculative: bool = False):
        """Mixer::Linear; conv and ssm are updated in place (ssm kept when speculative).

        Returns (y, ssm_out or None)."""
        keep = {k: np.ascontiguousarray(weights[k], dtype=np.float32) for k in
                ("conv", "ssm_a", "dt_bias", "ssm_norm")}
        layer = DeltaNetLayer(cfg["key_heads"], cfg["value_heads"], cfg["head_dim"], cfg["conv_kernel"],
                              cfg["rms_eps"], _fp(keep["conv"]), _fp(keep["ssm_a"]),
                              _fp(keep["dt_bias"]), _fp(keep["ssm_norm"]))
        y = np.empty(cfg["value_heads"] * cfg["head_dim"], dtype=np.float32)
        out = np.empty_like(ssm) if speculative else None
        self.lib.gufo_oracle_deltanet_linear(C.byref(layer), _fp(x_in), _fp(conv), _fp(ssm), _fp(y),
                                             _fp(out) if speculative else None)
        return y, out

    def route(self, logits: np.ndarray, k: int):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        chosen = np.empty(k, dtype=np.int32)
        weights = np.empty(k, dtype=np.float32)
        self.lib.gufo_oracle_route(_fp(logits), logits.size, k, chosen.ctypes.data_as(_i32p), _fp(weights))
        return chosen, weights

    def shared_expert_scale(self, logit: float) -> float:
        return float(self.lib.gufo_oracle_shared_expert_scale(logit))

    def rms_norm(self, x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
        out = np.empty_like(x)
        self.lib.gufo_oracle_rms_norm(_fp(x), _fp(w), x.size, eps, _fp(out))
        return out


# Stage ids in the order of the reference's enum (src/models/qwen35/projections.hpp:14-39).
STAGES = {"linear_in": 0, "attention_in": 1, "mixer_out": 2, "ffn_in": 3, "ffn_down": 4,
          "lm_head": 5, "router": 6, "expert_in": 7, "expert_down": 8, "mtp_in": 9}


class RefLib:
    """The compiled reference. `available()` is False where it was never built."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self, path: str = REF_SO):
        lib = C.CDLL(path)
        lib.gufo_ref_last_error.restype = C.c_char_p
        lib.gufo_ref_usable_cpus.restype = C.c_int
        lib.gufo_ref_projection_threads.restype = C.c_int
        lib.gufo_ref_half_to_float.restype = C.c_float
        lib.gufo_ref_half_to_float.argtypes = [C.c_uint16]
        lib.gufo_ref_dequantize.restype = C.c_int
        lib.gufo_ref_dequantize.argtypes = [C.c_uint32, _u8p, _f32p, C.c_size_t]
        lib.gufo_ref_dot.restype = C.c_int
        lib.gufo_ref_dot.argtypes = [C.c_uint32, _u8p, _f32p, C.c_size_t, _f32p]
        lib.gufo_ref_route.restype = None
        lib.gufo_ref_route.argtypes = [_f32p, C.c_int, C.c_int, _i32p, _f32p]
        lib.gufo_ref_shared_expert_scale.restype = C.c_float
        lib.gufo_ref_shared_expert_scale.argtypes = [C.c_float]
        lib.gufo_ref_model_open.restype = C.c_void_p
        lib.gufo_ref_model_open.argtypes = [_u8p, C.c_size_t, C.c_int]
        lib.gufo_ref_model_close.restype = None
        lib.gufo_ref_model_close.argtypes = [C.c_void_p]
        for name in ("gufo_ref_stage_inputs", "gufo_ref_stage_outputs"):
            getattr(lib, name).restype = C.c_size_t
            getattr(lib, name).argtypes = [C.c_void_p, C.c_int, C.c_int]
        lib.gufo_ref_apply.restype = C.c_int
        lib.gufo_ref_apply.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, C.c_int, _f32p]
        lib.gufo_ref_apply_expert.restype = C.c_int
        lib.gufo_ref_apply_expert.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, _f32p, C.c_int, _f32p]
        lib.gufo_ref_linear.restype = C.c_int
        lib.gufo_ref_linear.argtypes = [C.c_void_p, C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p]
        lib.gufo_ref_deltanet_run.restype = C.c_int
        lib.gufo_ref_deltanet_run.argtypes = [C.c_void_p, C.c_int, C.c_int, _f32p, C.c_size_t, _f32p,
                                              C.c_size_t, _f32p, _f32p, _f32p, _f32p, _f32p, C.c_size_t]
        lib.gufo_ref_decoder_reset.restype = C.c_int
        lib.gufo_ref_decoder_reset.argtypes = [C.c_void_p]
        lib.gufo_ref_decoder_step.restype = C.c_int
        lib.gufo_ref_decoder_step.argtypes = [C.c_void_p, C.c_int, _f32p]
        lib.gufo_ref_decoder_linear_state.restype = C.c_int
        lib.gufo_ref_decoder_linear_state.argtypes = [C.c_void_p, C.c_int, _f32p, _f32p]
        lib.gufo_ref_decoder_position.restype = C.c_int
        lib.gufo_ref_decoder_position.argtypes = [C.c_void_p]
        self.lib = lib

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise RuntimeError("reference: " + self.lib.gufo_ref_last_error().decode())

    def usable_cpus(self) -> int:
        return int(self.lib.gufo_ref_usable_cpus())

    def projection_threads(self) -> int:
        return int(self.lib.gufo_ref_projection_threads())

    def half_to_float(self, bits: int) -> float:
        return float(self.lib.gufo_ref_half_to_float(bits))

    def dequantize(self, ggml_type: int, raw: np.ndarray, n: int) -> np.ndarray:
        raw = np.ascontiguousarray(raw.reshape(-1))
        out = np.empty(n, dtype=np.float32)
        self._check(self.lib.gufo_ref_dequantize(ggml_type, _bp(raw), _fp(out), n))
        return out

    def dot(self, ggml_type: int, row: np.ndarray, x: np.ndarray) -> float:
        row = np.ascontiguousarray(row.reshape(-1))
        out = C.c_float()
        self._check(self.lib.gufo_ref_dot(ggml_type, _bp(row), _fp(x), x.size, C.byref(out)))
        return float(out.value)

    def route(self, logits: np.ndarray, k: int):
        logits = np.ascontiguousarray(logits, dtype=np.float32)
        chosen = np.empty(k, dtype=np.int32)
        weights = np.empty(k, dtype=np.float32)
        self.lib.gufo_ref_route(_fp(logits), logits.size, k, chosen.ctypes.data_as(_i32p), _fp(weights))
        return chosen, weights

    def shared_expert_scale(self, logit: float) -> float:
        return float(self.lib.gufo_ref_shared_expert_scale(logit))

    def open_model(self, gguf_bytes: np.ndarray, precision_float: bool = True) -> "RefModel":
        gguf_bytes = np.ascontiguousarray(gguf_bytes, dtype=np.uint8)
        handle = self.lib.gufo_ref_model_open(_bp(gguf_bytes), gguf_bytes.size, int(precision_float))
        if not handle:
            raise RuntimeError("reference: " + self.lib.gufo_ref_last_error().decode())
        return RefModel(self, handle)


class RefModel:
    """GgufProjections + Mixer + Decoder of the reference over a GGUF image."""

    def __init__(self, ref: RefLib, handle):
        self.ref = ref
        self.handle = handle

    def close(self) -> None:
        if self.handle:
            self.ref.lib.gufo_ref_model_close(self.handle)
            self.handle = None

    def __del__(self):
        self.close()

    def stage_inputs(self, stage: str, layer: int) -> int:
        return int(self.ref.lib.gufo_ref_stage_inputs(self.handle, STAGES[stage], layer))

    def stage_outputs(self, stage: str, layer: int) -> int:
        return int(self.ref.lib.gufo_ref_stage_outputs(self.handle, STAGES[stage], layer))

    def apply(self, stage: str, layer: int, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        tokens = 1 if x.ndim == 1 else x.shape[0]
        y = np.empty((tokens, self.stage_outputs(stage, layer)), dtype=np.float32)
        self.ref._check(self.ref.lib.gufo_ref_apply(self.handle, STAGES[stage], layer, _fp(x), tokens, _fp(y)))
        return y

    def apply_expert(self, stage: str, layer: int, expert: int, x: np.ndarray) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        tokens = 1 if x.ndim == 1 else x.shape[0]
        y = np.empty((tokens, self.stage_outputs(stage, layer)), dtype=np.float32)
        self.ref._check(self.ref.lib.gufo_ref_apply_expert(self.handle, STAGES[stage], layer, expert,
                                                          _fp(x), tokens, _fp(y)))
        return y

    def linear(self, layer: int, x_in: np.ndarray, conv: np.ndarray, ssm: np.ndarray, value_dim: int,
               speculative: bool = False):
        y = np.empty(value_dim, dtype=np.float32)
        out = np.empty_like(ssm) if speculative else None
        self.ref._check(self.ref.lib.gufo_ref_linear(self.handle, layer, _fp(x_in), _fp(conv), _fp(ssm),
                                                    _fp(y), _fp(out) if speculative else None))
        return y, out

    def deltanet_run(self, layer: int, count: int, x_in: np.ndarray, h: np.ndarray, conv, ssm,
                     value_dim: int):
        """DeltaNetStep::Run on rows of x_in / h; returns (y [count, value_dim], ssm_spec, conv_saved)."""
        y = np.zeros((count, value_dim), dtype=np.float32)
        spec = np.zeros_like(ssm)
        saved = np.zeros_like(conv)
        self.ref._check(self.ref.lib.gufo_ref_deltanet_run(
            self.handle, layer, count, _fp(x_in), x_in.shape[1], _fp(h), h.shape[1], _fp(conv), _fp(ssm),
            _fp(spec), _fp(saved), _fp(y), value_dim))
        return y, spec, saved

    def decoder_reset(self) -> None:
        self.ref._check(self.ref.lib.gufo_ref_decoder_reset(self.handle))

    def decoder_step(self, token: int, vocab: int) -> np.ndarray:
        logits = np.empty(vocab, dtype=np.float32)
        self.ref._check(self.ref.lib.gufo_ref_decoder_step(self.handle, token, _fp(logits)))
        return logits

    def decoder_step_discard(self, token: int) -> None:
        self.ref._check(self.ref.lib.gufo_ref_decoder_step(self.handle, token, None))

    def decoder_linear_state(self, layer: int, conv_size: int, ssm_size: int):
        conv = np.empty(conv_size, dtype=np.float32)
        ssm = np.empty(ssm_size, dtype=np.float32)
        self.ref._check(self.ref.lib.gufo_ref_decoder_linear_state(self.handle, layer, _fp(conv), _fp(ssm)))
        return conv, ssm
