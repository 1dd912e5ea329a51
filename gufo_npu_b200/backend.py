"""Host side of the CUDA backend: the reference's operator interface over the C ABI.

`CudaProjections` mirrors `qwen35::Projections` / `GgufProjections`
(src/models/qwen35/projections.hpp:45-59, gguf_projections.hpp:19-58 in the
reference): the same stages, argument meaning and errors, with the matrix
products on the device. `CudaMixer.Linear` mirrors `Mixer::Linear`
(src/models/qwen35/decoder.hpp:78-84). Everything computes through
libgufo_cuda.so; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
import enum
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _capi
from .synth import ModelConfig, Tensor


class Stage(enum.IntEnum):
    """qwen35::Stage (src/models/qwen35/projections.hpp:14-39)."""
    kLinearIn = 0
    kAttentionIn = 1
    kMixerOut = 2
    kFfnIn = 3
    kFfnDown = 4
    kLmHead = 5
    kRouter = 6
    kExpertIn = 7
    kExpertDown = 8
    kMtpIn = 9


def stage_inputs(c: ModelConfig, stage: Stage, layer: int) -> int:
    """StageInputs (src/models/qwen35/reference.cpp:609-623)."""
    if stage == Stage.kMixerOut:
        return c.heads * c.head_dim if c.is_full_attention(layer) else c.value_dim
    if stage == Stage.kFfnDown:
        return c.ffn_width
    if stage == Stage.kExpertDown:
        return c.expert_ffn
    if stage == Stage.kMtpIn:
        return 2 * c.hidden
    return c.hidden


def stage_outputs(c: ModelConfig, stage: Stage, layer: int) -> int:
    """StageOutputs (src/models/qwen35/reference.cpp:625-648)."""
    if stage == Stage.kLinearIn:
        return c.conv_channels + c.value_dim + 2 * c.linear_value_heads
    if stage == Stage.kAttentionIn:
        return 2 * c.heads * c.head_dim + 2 * c.kv_heads * c.head_dim
    if stage in (Stage.kMixerOut, Stage.kFfnDown, Stage.kExpertDown, Stage.kMtpIn):
        return c.hidden
    if stage == Stage.kFfnIn:
        return 2 * c.ffn_width
    if stage == Stage.kLmHead:
        return c.vocab
    if stage == Stage.kRouter:
        return c.experts + 1
    if stage == Stage.kExpertIn:
        return 2 * c.expert_ffn
    raise ValueError(stage)


def _ptr(buf) -> int:
    """Device or host address of a torch tensor, numpy array or raw integer."""
    if buf is None:
        return 0
    if isinstance(buf, int):
        return buf
    if isinstance(buf, np.ndarray):
        return buf.ctypes.data
    return buf.data_ptr()


class Context:
    """One gufo_cuda_ctx: a device, a stream, its weights and scratch."""

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        self.lib = _capi.load()
        handle = C.c_void_p()
        status = self.lib.gufo_cuda_ctx_create(device, C.c_void_p(stream or 0), C.byref(handle))
        _capi.check(self.lib, None, status)
        self.handle = handle
        self.device = device
        self.stream = stream or None

    def require_torch_stream(self) -> None:
        """Raises unless this context enqueues on torch's current stream: callers that mix torch
        ops with this library's kernels on the same buffers need one stream for both."""
        import torch
        if self.stream is None or self.stream != torch.cuda.current_stream(self.device).cuda_stream:
            raise RuntimeError("gufo_cuda: create the Context on torch's current (non-default) stream, e.g. "
                               "s = torch.cuda.Stream(); Context(0, s.cuda_stream); with torch.cuda.stream(s): ...")

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.gufo_cuda_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int) -> None:
        _capi.check(self.lib, self.handle, status)

    def set_stream(self, stream: int) -> None:
        self._check(self.lib.gufo_cuda_ctx_set_stream(self.handle, C.c_void_p(stream)))
        self.stream = stream or None

    def set_option(self, name: str, value: int) -> None:
        self._check(self.lib.gufo_cuda_ctx_set_option(self.handle, name.encode(), value))

    def synchronize(self) -> None:
        self._check(self.lib.gufo_cuda_ctx_synchronize(self.handle))

    def launch_count(self) -> int:
        return int(self.lib.gufo_cuda_launch_count(self.handle))

    # -- device memory ----------------------------------------------------
    def malloc(self, nbytes: int) -> int:
        out = C.c_void_p()
        self._check(self.lib.gufo_cuda_malloc(self.handle, nbytes, C.byref(out)))
        return int(out.value)

    def free(self, ptr: int) -> None:
        self._check(self.lib.gufo_cuda_free(self.handle, C.c_void_p(ptr)))

    def upload(self, dst: int, src: np.ndarray) -> None:
        src = np.ascontiguousarray(src)
        self._check(self.lib.gufo_cuda_upload(self.handle, C.c_void_p(dst), C.c_void_p(src.ctypes.data), src.nbytes))

    def download(self, src: int, shape, dtype=np.float32) -> np.ndarray:
        out = np.empty(shape, dtype=dtype)
        self._check(self.lib.gufo_cuda_download(self.handle, C.c_void_p(out.ctypes.data), C.c_void_p(src), out.nbytes))
        return out

    def memset_zero(self, ptr: int, nbytes: int) -> None:
        self._check(self.lib.gufo_cuda_memset_zero(self.handle, C.c_void_p(ptr), nbytes))

    # -- weights ------------------------------------------------------------
    def matrix_upload(self, ggml_type: int, host_bytes: np.ndarray, rows: int, cols: int) -> int:
        host_bytes = np.ascontiguousarray(host_bytes)
        out = C.c_int64()
        self._check(self.lib.gufo_cuda_matrix_upload(self.handle, ggml_type, C.c_void_p(host_bytes.ctypes.data),
                                                     rows, cols, C.byref(out)))
        return int(out.value)

    def matrix_from_device(self, ggml_type: int, device_ptr: int, rows: int, cols: int) -> int:
        out = C.c_int64()
        self._check(self.lib.gufo_cuda_matrix_from_device(self.handle, ggml_type, C.c_void_p(device_ptr), rows,
                                                          cols, C.byref(out)))
        return int(out.value)

    def matrix_free(self, matrix: int) -> None:
        self._check(self.lib.gufo_cuda_matrix_free(self.handle, matrix))

    def dequantize(self, matrix: int, first: int, rows: int, cols: int) -> np.ndarray:
        out = np.empty((rows, cols), dtype=np.float32)
        self._check(self.lib.gufo_cuda_dequantize(self.handle, matrix, first, rows, C.c_void_p(out.ctypes.data)))
        return out

    def dequantize_device(self, matrix: int, first: int, rows: int, dst) -> None:
        self._check(self.lib.gufo_cuda_dequantize_device(self.handle, matrix, first, rows, C.c_void_p(_ptr(dst))))

    # -- products -----------------------------------------------------------
    @staticmethod
    def _parts(parts: Sequence) -> "C.Array":
        arr = (_capi.Rows * max(len(parts), 1))()
        for i, (w, first, rows) in enumerate(parts):
            arr[i] = _capi.Rows(w, first, rows)
        return arr

    def matmul(self, parts: Sequence, x: np.ndarray, tokens: int, out_width: int) -> np.ndarray:
        """Host pointers: copies x up, runs, copies y down. parts: [(matrix, first, rows)]."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty((tokens, out_width), dtype=np.float32)
        self._check(self.lib.gufo_cuda_matmul(self.handle, self._parts(parts), len(parts),
                                              C.c_void_p(x.ctypes.data), tokens, C.c_void_p(y.ctypes.data)))
        return y

    def matmul_host(self, parts_arr, nparts: int, x_ptr: int, tokens: int, y_ptr: int) -> None:
        """The same on caller-owned (for example pinned) host buffers, no allocation."""
        self._check(self.lib.gufo_cuda_matmul(self.handle, parts_arr, nparts, C.c_void_p(x_ptr), tokens,
                                              C.c_void_p(y_ptr)))

    def matmul_device(self, parts_arr, nparts: int, x, tokens: int, y) -> None:
        self._check(self.lib.gufo_cuda_matmul_device(self.handle, parts_arr, nparts, C.c_void_p(_ptr(x)), tokens,
                                                     C.c_void_p(_ptr(y))))

    def matmul_fused_device(self, parts_arr, nparts: int, tokens: int, y, *, x=None, residual=None, delta=None,
                            norm_weight=None, rms_eps: float = 0.0, residual_out=None, scratch=None,
                            advance=None, swiglu: bool = False, delta_parts: int = 0, delta_stride: int = 0,
                            activate: bool = False) -> None:
        """A product with its input step fused in (npu::Q4nxGemv's Prologue options,
        src/npu/gemv.hpp:58-68): plain `x`; `residual` (+ `delta`, or the sum of `delta_parts`
        vectors `delta_stride` floats apart) through RMSNorm; or SwiGLU of [gate | up] rows in
        `x`. `activate`: the parts are gate and up rows and y receives silu(gate) * up
        (Epilogue::kSwiGlu); raises GufoCudaError (unsupported type) where the kernel cannot."""
        kind = _capi.PROLOGUE_RES_NORM if residual is not None else (
            _capi.PROLOGUE_SWIGLU if swiglu else _capi.PROLOGUE_PLAIN)
        p = lambda t: C.c_void_p(_ptr(t)) if t is not None else None
        args = _capi.FusedInput(kind, p(x), p(residual), p(delta), p(norm_weight), rms_eps, p(residual_out),
                                p(scratch), p(advance), delta_parts, delta_stride,
                                _capi.EPILOGUE_SWIGLU if activate else _capi.EPILOGUE_NONE)
        self._check(self.lib.gufo_cuda_matmul_fused_device(self.handle, parts_arr, nparts, C.byref(args), tokens,
                                                           C.c_void_p(_ptr(y))))

    # -- routed experts -------------------------------------------------------
    def route_device(self, router, stride: int, tokens: int, experts: int, k: int, chosen, weights,
                     shared_scale=None) -> None:
        self._check(self.lib.gufo_cuda_route_device(self.handle, C.c_void_p(_ptr(router)), stride, tokens, experts, k,
                                                    C.c_void_p(_ptr(chosen)), C.c_void_p(_ptr(weights)),
                                                    C.c_void_p(_ptr(shared_scale))))

    def expert_ffn_device(self, bank: "_capi.ExpertBank", ids, pairs: int, x, x_stride: int, ffn, act, y,
                          pairs_per_input: int = 1) -> None:
        """Pair p multiplies input row p // pairs_per_input (rows x_stride floats apart)."""
        self._check(self.lib.gufo_cuda_expert_ffn_device(self.handle, C.byref(bank), C.c_void_p(_ptr(ids)), pairs,
                                                         C.c_void_p(_ptr(x)), x_stride, pairs_per_input,
                                                         C.c_void_p(_ptr(ffn)),
                                                         C.c_void_p(_ptr(act)), C.c_void_p(_ptr(y))))

    def moe_ffn_device(self, bank: "_capi.ExpertBank", ids, weights, scale, tokens: int, k: int, x, x_stride: int,
                       shared, ffn, act, expert_out, out) -> None:
        """out[t] = shared[t] * scale[t] + the weighted sum of token t's k experts' FFN (device tensors)."""
        self._check(self.lib.gufo_cuda_moe_ffn_device(
            self.handle, C.byref(bank), C.c_void_p(_ptr(ids)), C.c_void_p(_ptr(weights)), C.c_void_p(_ptr(scale)),
            tokens, k, C.c_void_p(_ptr(x)), x_stride, C.c_void_p(_ptr(shared)), C.c_void_p(_ptr(ffn)),
            C.c_void_p(_ptr(act)), C.c_void_p(_ptr(expert_out)), C.c_void_p(_ptr(out))))

    def moe_combine_device(self, shared, scale, weights, expert_out, tokens: int, k: int, hidden: int, out) -> None:
        self._check(self.lib.gufo_cuda_moe_combine_device(self.handle, C.c_void_p(_ptr(shared)),
                                                          C.c_void_p(_ptr(scale)), C.c_void_p(_ptr(weights)),
                                                          C.c_void_p(_ptr(expert_out)), tokens, k, hidden,
                                                          C.c_void_p(_ptr(out))))

    # -- DeltaNet -----------------------------------------------------------
    def delta_rule_device(self, seqs: List[dict], key_heads: int, value_heads: int, head_dim: int) -> None:
        arr = (_capi.DeltaSeq * max(len(seqs), 1))()
        for i, s in enumerate(seqs):
            arr[i] = _capi.DeltaSeq(_ptr(s["state"]), _ptr(s.get("state_out")), _ptr(s["q"]), _ptr(s["k"]),
                                    _ptr(s["v"]), _ptr(s["decay"]), _ptr(s["beta"]), _ptr(s["y"]))
        self._check(self.lib.gufo_cuda_delta_rule_device(self.handle, arr, len(seqs), key_heads, value_heads,
                                                         head_dim))

    def deltanet_layer_create(self, key_heads: int, value_heads: int, head_dim: int, conv_kernel: int,
                              rms_eps: float, conv, ssm_a, dt_bias, ssm_norm) -> int:
        keep = [np.ascontiguousarray(a, dtype=np.float32) for a in (conv, ssm_a, dt_bias, ssm_norm)]
        f32p = C.POINTER(C.c_float)
        params = _capi.DeltaNetParams(key_heads, value_heads, head_dim, conv_kernel, rms_eps,
                                      *(a.ctypes.data_as(f32p) for a in keep))
        out = C.c_int64()
        self._check(self.lib.gufo_cuda_deltanet_layer_create(self.handle, C.byref(params), C.byref(out)))
        return int(out.value)

    def deltanet_layer_free(self, layer: int) -> None:
        self._check(self.lib.gufo_cuda_deltanet_layer_free(self.handle, layer))

    def deltanet_linear_device(self, layer: int, seqs: List[dict]) -> None:
        arr = (_capi.LinearSeq * max(len(seqs), 1))()
        for i, s in enumerate(seqs):
            arr[i] = _capi.LinearSeq(_ptr(s["in"]), _ptr(s["conv_in"]), _ptr(s["conv_out"]), _ptr(s["ssm"]),
                                     _ptr(s.get("ssm_out")), _ptr(s["y"]))
        self._check(self.lib.gufo_cuda_deltanet_linear_device(self.handle, layer, arr, len(seqs)))


def _shape_error(name: str, shape, want) -> RuntimeError:
    return RuntimeError(f"qwen35: tensor {name} has shape {list(shape)}, expected {list(want)}")


class _DeviceArray:
    """A window of device memory for torch.as_tensor (the CUDA array interface)."""

    def __init__(self, ptr: int, floats: int):
        self.__cuda_array_interface__ = {"shape": (floats,), "typestr": "<f4", "data": (ptr, False), "version": 3,
                                         "strides": None}


class PeerGroup:
    """The ranks of a row-split step sharing their output vectors over NVLink peer memory
    (gufo_cuda_peer_group). Every rank constructs it with the same `arena_floats` and asks for
    the same buffers in the same order, so that a vector sits at one offset on every rank.
    `exchange(handle_bytes) -> [handle_bytes per rank]` is the host's all-gather of the IPC
    handles (torch.distributed.all_gather_object, for one)."""

    def __init__(self, ctx: Context, rank: int, world: int, arena_floats: int, exchange):
        import torch
        self.ctx, self.rank, self.world = ctx, rank, world
        self.bytes = _capi.PEER_HEADER_BYTES + 4 * arena_floats
        self.arena = ctx.malloc(self.bytes)
        handle = (C.c_ubyte * _capi.IPC_HANDLE_BYTES)()
        ctx._check(ctx.lib.gufo_cuda_ipc_export(ctx.handle, C.c_void_p(self.arena), handle))
        handles = exchange(bytes(handle))
        assert len(handles) == world and all(len(h) == _capi.IPC_HANDLE_BYTES for h in handles)
        packed = (C.c_ubyte * (world * _capi.IPC_HANDLE_BYTES)).from_buffer_copy(b"".join(handles))
        out = C.c_void_p()
        ctx._check(ctx.lib.gufo_cuda_peer_group_create(ctx.handle, rank, world, C.c_void_p(self.arena), self.bytes,
                                                       packed, C.byref(out)))
        self.handle = out
        self._next = _capi.PEER_HEADER_BYTES
        self._torch = torch

    def buffer(self, floats: int):
        """The next `floats` values of the arena as a torch tensor (256-byte aligned)."""
        offset = self._next
        self._next = (offset + 4 * floats + 255) // 256 * 256
        if self._next > self.bytes:
            raise ValueError("peer arena exhausted")
        # The arena was cleared when the group was created (before the ranks' barrier): clearing
        # a view here could wipe a slice a faster peer has already stored.
        return self._torch.as_tensor(_DeviceArray(self.arena + offset, floats),
                                     device=self._torch.device("cuda", self.ctx.device))

    def offset_of(self, tensor) -> int:
        return tensor.data_ptr() - self.arena

    def allgather(self, local, full, slice_floats: int) -> None:
        """Rank r's first `slice_floats` values of `local` to full[r * slice : (r + 1) * slice] on every rank."""
        self.ctx._check(self.ctx.lib.gufo_cuda_peer_allgather_device(self.handle, C.c_void_p(_ptr(local)),
                                                                     self.offset_of(full), slice_floats))

    def status(self) -> None:
        self.ctx._check(self.ctx.lib.gufo_cuda_peer_group_status(self.handle))

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.ctx.lib.gufo_cuda_peer_group_destroy(self.handle)
            self.handle = None


class CudaProjections:
    """The matrix products of a Qwen3.5 forward pass on the device.

    Construction uploads every projection tensor once and checks its shape as
    GgufProjections does (src/models/qwen35/gguf_projections.cpp:27-46,100-175):
    a wrong shape raises RuntimeError. Apply / ApplyExpert take and return host
    arrays like the reference's interface; apply_device is the same product on
    device-resident activations.
    """

    def __init__(self, ctx: Context, cfg: ModelConfig, tensors: Dict[str, Tensor]):
        self.ctx = ctx
        self.config = cfg
        self._matrices: Dict[str, int] = {}
        self._tensors = tensors
        c = cfg
        lm = "token_embd.weight" if c.tied_embeddings else "output.weight"
        self._check_shape(lm, (c.hidden, c.vocab))
        self.lm_head = [(self._matrix(lm), 0, c.vocab)]
        self.embed = self._matrix("token_embd.weight")
        attn_dim = c.heads * c.head_dim
        kv_dim = c.kv_heads * c.head_dim
        self.layers: List[dict] = []
        # The decoder layers, then the MTP layer (full attention) if the file has one
        # (gguf_projections.cpp:114-125).
        has_mtp = c.mtp_layers > 0 and f"blk.{c.layers}.nextn.eh_proj.weight" in tensors
        for il in range(c.layers + (1 if has_mtp else 0)):
            p = f"blk.{il}."
            layer: dict = {}
            if il >= c.layers:
                self._check_shape(p + "nextn.eh_proj.weight", (2 * c.hidden, c.hidden))
                layer[Stage.kMtpIn] = [self._all(p + "nextn.eh_proj.weight")]
            if c.is_moe:
                self._check_shape(p + "ffn_gate_inp.weight", (c.hidden, c.experts))
                self._check_shape(p + "ffn_gate_inp_shexp.weight", (c.hidden, 1))
                layer[Stage.kRouter] = [self._all(p + "ffn_gate_inp.weight"),
                                        self._all(p + "ffn_gate_inp_shexp.weight")]
                for name, cols, rows in (("ffn_gate_exps.weight", c.hidden, c.expert_ffn),
                                         ("ffn_up_exps.weight", c.hidden, c.expert_ffn),
                                         ("ffn_down_exps.weight", c.expert_ffn, c.hidden)):
                    self._check_shape(p + name, (cols, rows, c.experts))
                layer["gate_exps"] = self._matrix(p + "ffn_gate_exps.weight")
                layer["up_exps"] = self._matrix(p + "ffn_up_exps.weight")
                layer["down_exps"] = self._matrix(p + "ffn_down_exps.weight")
            suffix = "_shexp.weight" if c.is_moe else ".weight"
            self._check_shape(p + "ffn_gate" + suffix, (c.hidden, c.ffn_width))
            self._check_shape(p + "ffn_up" + suffix, (c.hidden, c.ffn_width))
            self._check_shape(p + "ffn_down" + suffix, (c.ffn_width, c.hidden))
            layer[Stage.kFfnIn] = [self._all(p + "ffn_gate" + suffix), self._all(p + "ffn_up" + suffix)]
            layer[Stage.kFfnDown] = [self._all(p + "ffn_down" + suffix)]
            if c.is_full_attention(il):
                self._check_shape(p + "attn_q.weight", (c.hidden, 2 * attn_dim))
                self._check_shape(p + "attn_k.weight", (c.hidden, kv_dim))
                self._check_shape(p + "attn_v.weight", (c.hidden, kv_dim))
                self._check_shape(p + "attn_output.weight", (attn_dim, c.hidden))
                layer[Stage.kAttentionIn] = [self._all(p + n) for n in
                                             ("attn_q.weight", "attn_k.weight", "attn_v.weight")]
                layer[Stage.kMixerOut] = [self._all(p + "attn_output.weight")]
            else:
                self._check_shape(p + "attn_qkv.weight", (c.hidden, c.conv_channels))
                self._check_shape(p + "attn_gate.weight", (c.hidden, c.value_dim))
                self._check_shape(p + "ssm_alpha.weight", (c.hidden, c.linear_value_heads))
                self._check_shape(p + "ssm_beta.weight", (c.hidden, c.linear_value_heads))
                self._check_shape(p + "ssm_out.weight", (c.value_dim, c.hidden))
                layer[Stage.kLinearIn] = [self._all(p + n) for n in
                                          ("attn_qkv.weight", "attn_gate.weight", "ssm_alpha.weight",
                                           "ssm_beta.weight")]
                layer[Stage.kMixerOut] = [self._all(p + "ssm_out.weight")]
            self.layers.append(layer)
        self._tensors = None  # host bytes are not referenced after upload

    # -- construction helpers ------------------------------------------------
    def _check_shape(self, name: str, want) -> None:
        if name not in self._tensors:
            raise RuntimeError(f"GGUF: missing tensor {name}")
        shape = tuple(self._tensors[name].shape)
        want = tuple(want)
        if len(want) == 2 and want[1] == 1 and len(shape) == 1:
            want = want[:1]
        if shape != want:
            raise _shape_error(name, shape, want)

    def _matrix(self, name: str) -> int:
        if name not in self._matrices:
            t = self._tensors[name]
            if t.data.is_cuda:
                # Weights generated on the device stay where they are; the tensor is kept alive here.
                self._keep = getattr(self, "_keep", [])
                self._keep.append(t.data)
                handle = self.ctx.matrix_from_device(t.ggml_type, t.data.data_ptr(), t.rows, t.cols)
            else:
                handle = self.ctx.matrix_upload(t.ggml_type, t.data.numpy(), t.rows, t.cols)
            self._matrices[name] = handle
        return self._matrices[name]

    def _all(self, name: str):
        return (self._matrix(name), 0, self._tensors[name].rows)

    # -- the reference's interface ---------------------------------------------
    def parts(self, stage: Stage, layer: int):
        if stage == Stage.kLmHead:
            return self.lm_head
        if layer < 0 or layer >= len(self.layers):
            raise IndexError("qwen35: no such layer")
        parts = self.layers[layer].get(stage)
        if not parts:
            raise LookupError("qwen35: no weights for this stage and layer")
        return parts

    def expert_parts(self, stage: Stage, layer: int, expert: int):
        c = self.config
        l = self.layers[layer]
        if "gate_exps" not in l or expert < 0 or expert >= c.experts:
            raise LookupError("qwen35: no such expert")
        if stage == Stage.kExpertIn:
            return [(l["gate_exps"], expert * c.expert_ffn, c.expert_ffn),
                    (l["up_exps"], expert * c.expert_ffn, c.expert_ffn)]
        if stage == Stage.kExpertDown:
            return [(l["down_exps"], expert * c.hidden, c.hidden)]
        raise LookupError("qwen35: ApplyExpert takes expert stages only")

    def Apply(self, stage: Stage, layer: int, x: np.ndarray, tokens: int) -> np.ndarray:
        """y[t] = W x[t]: `tokens` rows of StageInputs in, rows of StageOutputs out (host arrays)."""
        parts = self.parts(stage, layer)
        return self.ctx.matmul(parts, x, tokens, sum(p[2] for p in parts))

    def ApplyExpert(self, stage: Stage, layer: int, expert: int, x: np.ndarray, tokens: int) -> np.ndarray:
        parts = self.expert_parts(stage, layer, expert)
        return self.ctx.matmul(parts, x, tokens, sum(p[2] for p in parts))

    def apply_device(self, stage: Stage, layer: int, x, tokens: int, y) -> None:
        parts = self.parts(stage, layer)
        self.ctx.matmul_device(Context._parts(parts), len(parts), x, tokens, y)


class CudaMoe:
    """Decoder::MoeFfn (src/models/qwen35/decoder.cpp:535-557) for a few tokens with every
    step on the device: router product, Route, the chosen experts' FFN as grouped products,
    the weighted sum onto the scaled shared expert's output.

    `expert_range` = (first, count) keeps only those experts on this device (expert
    parallelism): pairs routed elsewhere are skipped and their rows of `expert_out` stay zero,
    so that a sum over the ranks restores every row before `combine`.
    """

    def __init__(self, projections: "CudaProjections", max_tokens: int = 4, expert_range=None):
        import torch
        c = projections.config
        if not c.is_moe:
            raise RuntimeError("qwen35: not a MoE model")
        self.projections = projections
        self.ctx = projections.ctx
        self.config = c
        self.max_tokens = max_tokens
        self.expert_range = expert_range
        dev = torch.device("cuda", self.ctx.device)
        k = c.experts_used
        f32 = dict(dtype=torch.float32, device=dev)
        self.router = torch.empty(max_tokens, c.experts + 1, **f32)
        self.chosen = torch.empty(max_tokens, k, dtype=torch.int32, device=dev)
        self.local = torch.empty(max_tokens, k, dtype=torch.int32, device=dev)
        self.weights = torch.empty(max_tokens, k, **f32)
        self.scale = torch.empty(max_tokens, **f32)
        self.ffn = torch.empty(max_tokens * k, 2 * c.expert_ffn, **f32)
        self.act = torch.empty(max_tokens * k, c.expert_ffn, **f32)
        self.expert_out = torch.zeros(max_tokens, k, c.hidden, **f32)
        self.banks = []
        for l in projections.layers:
            self.banks.append(_capi.ExpertBank(l["gate_exps"], l["up_exps"], l["down_exps"], c.experts,
                                               c.expert_ffn, c.hidden))

    def route(self, layer: int, normed, tokens: int) -> None:
        """Router product and top-k of `tokens` normed rows (device tensor)."""
        c = self.config
        self.projections.apply_device(Stage.kRouter, layer, normed, tokens, self.router)
        self.ctx.route_device(self.router, c.experts + 1, tokens, c.experts, c.experts_used, self.chosen,
                              self.weights, self.scale)

    def experts(self, layer: int, normed, tokens: int) -> None:
        """The chosen experts' FFN of every (token, slot) pair held here, into expert_out."""
        c = self.config
        k = c.experts_used
        ids = self.chosen
        if self.expert_range is not None:
            self.ctx.require_torch_stream()
            first, count = self.expert_range
            held = (self.chosen >= first) & (self.chosen < first + count)
            self.local.copy_(torch_where(held, self.chosen, -1))
            self.expert_out.zero_()
            ids = self.local
        # One pair of grouped launches for the whole batch: pair (t, slot) reads token t's row.
        self.ctx.expert_ffn_device(self.banks[layer], ids, tokens * k, normed, c.hidden, self.ffn, self.act,
                                   self.expert_out, pairs_per_input=k)

    def combine(self, shared, tokens: int, out) -> None:
        c = self.config
        self.ctx.moe_combine_device(shared, self.scale, self.weights, self.expert_out, tokens, c.experts_used,
                                    c.hidden, out)

    def MoeFfn(self, layer: int, normed, shared, tokens: int, out) -> None:
        """out[t] = shared[t] * scale + sum of the routed experts' outputs (device tensors)."""
        if tokens > self.max_tokens:
            raise ValueError("CudaMoe: more tokens than max_tokens")
        self.route(layer, normed, tokens)
        if self.expert_range is None:
            c = self.config
            self.ctx.moe_ffn_device(self.banks[layer], self.chosen, self.weights, self.scale, tokens, c.experts_used,
                                    normed, c.hidden, shared, self.ffn, self.act, self.expert_out, out)
            return
        self.experts(layer, normed, tokens)
        self.combine(shared, tokens, out)


def torch_where(cond, a, b):
    import torch
    return torch.where(cond, a, torch.full_like(a, b))


class CudaMixer:
    """Gated DeltaNet decode step with the state resident on the device (Mixer::Linear)."""

    def __init__(self, ctx: Context, cfg: ModelConfig, tensors: Dict[str, Tensor]):
        self.ctx = ctx
        self.config = cfg
        self.layers: Dict[int, int] = {}
        self.gates: Dict[int, tuple] = {}
        for il in range(cfg.layers):
            if cfg.is_full_attention(il):
                continue
            p = f"blk.{il}."

            def f32(name):
                return tensors[p + name].data.cpu().numpy().view(np.float32)
            self.layers[il] = ctx.deltanet_layer_create(
                cfg.linear_key_heads, cfg.linear_value_heads, cfg.linear_head_dim, cfg.conv_kernel, cfg.rms_eps,
                f32("ssm_conv1d.weight"), f32("ssm_a"), f32("ssm_dt.bias"), f32("ssm_norm.weight"))
            # For Run (the gates from the residual stream): the F32 alpha / beta rows and the norm.
            alpha, beta = tensors[p + "ssm_alpha.weight"], tensors[p + "ssm_beta.weight"]
            norm = ctx.malloc(cfg.hidden * 4)
            ctx.upload(norm, f32("attn_norm.weight"))
            self.gates[il] = (ctx.matrix_upload(alpha.ggml_type, alpha.data.cpu().numpy(), alpha.rows, alpha.cols),
                              ctx.matrix_upload(beta.ggml_type, beta.data.cpu().numpy(), beta.rows, beta.cols), norm)

    def conv_values(self) -> int:
        return (self.config.conv_kernel - 1) * self.config.conv_channels

    def ssm_values(self) -> int:
        c = self.config
        return c.linear_value_heads * c.linear_head_dim * c.linear_head_dim

    def Linear(self, layer: int, seqs: List[dict]) -> None:
        """One step for each sequence in `seqs` (device pointers: in, conv_in, conv_out, ssm, ssm_out?, y)."""
        if layer not in self.layers:
            raise ValueError(f"deltanet: layer {layer} is not a DeltaNet layer")
        self.ctx.deltanet_linear_device(self.layers[layer], seqs)


def _deltanet_run(self, layer: int, seqs: List[dict]) -> None:
    """DeltaNetStep::Run (src/models/qwen35_2b/deltanet.hpp:42-44) for each sequence in `seqs`:
    dicts with n_tokens, in [n, in_stride], h [n, h_stride], conv_in, conv_out, conv_saved, ssm,
    ssm_spec, y [n, y_stride] (device tensors; conv_saved / ssm_spec may be None for one token)."""
    if layer not in self.layers:
        raise ValueError(f"deltanet: layer {layer} is not a DeltaNet layer")
    arr = (_capi.DeltaNetStepSeq * max(len(seqs), 1))()
    for i, q in enumerate(seqs):
        arr[i] = _capi.DeltaNetStepSeq(q["n_tokens"], _ptr(q["in"]), q["in"].stride(0), _ptr(q["h"]),
                                       q["h"].stride(0), _ptr(q["conv_in"]), _ptr(q["conv_out"]),
                                       _ptr(q.get("conv_saved")), _ptr(q["ssm"]), _ptr(q.get("ssm_spec")),
                                       _ptr(q["y"]), q["y"].stride(0))
    alpha, beta, norm = self.gates[layer]
    self.ctx._check(self.ctx.lib.gufo_cuda_deltanet_step_device(self.ctx.handle, self.layers[layer], alpha, beta,
                                                                C.c_void_p(norm), self.config.rms_eps, arr,
                                                                len(seqs)))


CudaMixer.Run = _deltanet_run


class CudaDecoder:
    """qwen35::Decoder with every buffer on the device (dense and MoE models).

    `Step(token)` mirrors Decoder::Step (src/models/qwen35/decoder.cpp:478-528): it runs the
    token at the current position, advances the state and returns the vocab logits. The
    matrices are the ones `projections` uploaded; the small vectors are copied.
    """

    # GGUF tensor name of each field of gufo_cuda_layer_weights.
    _MATRIX_NAMES = {"attn_qkv": "attn_qkv.weight", "attn_gate": "attn_gate.weight",
                     "ssm_alpha": "ssm_alpha.weight", "ssm_beta": "ssm_beta.weight", "ssm_out": "ssm_out.weight",
                     "attn_q": "attn_q.weight", "attn_k": "attn_k.weight", "attn_v": "attn_v.weight",
                     "attn_output": "attn_output.weight", "ffn_gate": "ffn_gate.weight", "ffn_up": "ffn_up.weight",
                     "ffn_down": "ffn_down.weight"}
    # MoE layers: the shared expert stands where the dense FFN does.
    _MOE_MATRIX_NAMES = {"ffn_gate": "ffn_gate_shexp.weight", "ffn_up": "ffn_up_shexp.weight",
                         "ffn_down": "ffn_down_shexp.weight", "ffn_gate_inp": "ffn_gate_inp.weight",
                         "ffn_gate_inp_shexp": "ffn_gate_inp_shexp.weight", "ffn_gate_exps": "ffn_gate_exps.weight",
                         "ffn_up_exps": "ffn_up_exps.weight", "ffn_down_exps": "ffn_down_exps.weight"}
    _VECTOR_NAMES = {"attn_norm": "attn_norm.weight", "post_attention_norm": "post_attention_norm.weight",
                     "ssm_conv1d": "ssm_conv1d.weight", "ssm_a": "ssm_a", "ssm_dt_bias": "ssm_dt.bias",
                     "ssm_norm": "ssm_norm.weight", "attn_q_norm": "attn_q_norm.weight",
                     "attn_k_norm": "attn_k_norm.weight"}

    def __init__(self, projections: CudaProjections, tensors: Dict[str, Tensor], max_positions: int = 4096,
                 use_graph: bool = True):
        c = projections.config
        self.ctx = projections.ctx
        self.config = c
        self.projections = projections
        lib = self.ctx.lib
        f32p = C.POINTER(C.c_float)
        keep = []

        def vec(name):
            a = np.ascontiguousarray(tensors[name].data.cpu().numpy().view(np.float32))
            keep.append(a)
            return a.ctypes.data_as(f32p)
        layers = (_capi.LayerWeights * c.layers)()
        for il in range(c.layers):
            p = f"blk.{il}."
            names = dict(self._MATRIX_NAMES, **self._MOE_MATRIX_NAMES) if c.is_moe else self._MATRIX_NAMES
            for field, name in names.items():
                setattr(layers[il], field, projections._matrices.get(p + name, 0))
            for field, name in self._VECTOR_NAMES.items():
                if p + name in tensors:
                    setattr(layers[il], field, vec(p + name))
        weights = _capi.DecoderWeights(projections._matrices["token_embd.weight"],
                                       0 if c.tied_embeddings else projections._matrices["output.weight"],
                                       vec("output_norm.weight"), layers)
        config = _capi.DecoderConfig(c.layers, c.hidden, c.ffn_width, c.vocab, c.rms_eps, c.full_attention_interval,
                                     c.heads, c.kv_heads, c.head_dim, c.rope_dim, c.rope_theta, c.conv_kernel,
                                     c.linear_key_heads, c.linear_value_heads, c.linear_head_dim, max_positions,
                                     int(use_graph), c.experts, c.experts_used, c.expert_ffn)
        handle = C.c_void_p()
        _capi.check(lib, self.ctx.handle,
                    lib.gufo_cuda_decoder_create(self.ctx.handle, C.byref(config), C.byref(weights), C.byref(handle)))
        self.handle = handle

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.ctx.lib.gufo_cuda_decoder_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def Reset(self) -> None:
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_reset(self.handle))

    def Step(self, token: int, logits: Optional[np.ndarray] = None) -> np.ndarray:
        """Runs `token`; returns the logits (written into `logits` when given, e.g. pinned memory)."""
        if logits is None:
            logits = np.empty(self.config.vocab, dtype=np.float32)
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_step(self.handle, token, C.c_void_p(_ptr(logits))))
        return logits

    def StepTokens(self, tokens: Sequence[int], logits: bool = True) -> Optional[np.ndarray]:
        """NpuDecoder::Step(tokens, count, state, logits) (src/models/qwen35_2b/npu_decoder.hpp:57-65):
        one or two tokens from the current position in one pass; returns [count, vocab] logits, or
        None with `logits` off (prompt passes). After two tokens the second is a draft until
        `Resolve`."""
        count = len(tokens)
        ids = (C.c_int * max(count, 1))(*tokens)
        out = np.empty((count, self.config.vocab), dtype=np.float32) if logits else None
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_step_tokens(
            self.handle, ids, count, int(logits), C.c_void_p(_ptr(out)) if logits else None))
        return out

    def step_tokens_device(self, tokens: Sequence[int]) -> int:
        """`StepTokens` leaving the [count, vocab] logits on the device; returns their address."""
        ids = (C.c_int * len(tokens))(*tokens)
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_step_tokens(self.handle, ids, len(tokens), 1, None))
        out = C.c_void_p()
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_logits_device(self.handle, C.byref(out)))
        return int(out.value)

    def Resolve(self, keep_second: bool) -> None:
        """NpuDecoder::Resolve (src/models/qwen35_2b/npu_decoder.cpp:630-650): keeps the draft of
        the last two-token step, or rolls the decoder back to just after its first token."""
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_resolve(self.handle, int(keep_second)))

    def hidden(self, t: int = 0) -> np.ndarray:
        """NpuDecoder::hidden(t): the final residual (before output_norm) of token t of the last step."""
        out = C.c_void_p()
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_hidden_device(self.handle, t, C.byref(out)))
        return self.ctx.download(int(out.value), self.config.hidden)

    def step_device(self, token: int) -> int:
        """Runs `token` leaving the logits on the device; returns their device address."""
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_step(self.handle, token, None))
        out = C.c_void_p()
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_logits_device(self.handle, C.byref(out)))
        return int(out.value)

    def status(self) -> None:
        """Waits for the stream; raises GufoCudaError (timeout) if a wait inside the persistent
        step kernel ran out since the last check."""
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_status(self.handle))

    def step_profile(self) -> List[dict]:
        """Per operation of the last step run by the persistent kernel: stage name, bytes moved
        and device microseconds; empty when the model runs on the launch chain."""
        n = C.c_int()
        lib = self.ctx.lib
        self.ctx._check(lib.gufo_cuda_decoder_step_profile(self.handle, 0, None, None, None, C.byref(n)))
        if n.value == 0:
            return []
        stages = (C.c_int * n.value)()
        nbytes = (C.c_int64 * n.value)()
        us = (C.c_double * n.value)()
        self.ctx._check(lib.gufo_cuda_decoder_step_profile(self.handle, n.value, stages, nbytes, us, C.byref(n)))
        return [{"stage": self.TIMELINE_KINDS[stages[i]], "bytes": int(nbytes[i]), "us": float(us[i])}
                for i in range(n.value)]

    TIMELINE_KINDS = ("embed", "in", "deltanet", "attention", "out", "ffn_in", "ffn_down", "lm_head")

    def timeline(self, enable: bool) -> Dict[str, float]:
        """Per-stage device milliseconds per step collected since the last switch; then turns
        collection on or off (collection runs the step eagerly, without graph replay)."""
        ms = (C.c_double * len(self.TIMELINE_KINDS))()
        steps = C.c_int()
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_timeline(self.handle, int(enable), ms, C.byref(steps)))
        n = max(steps.value, 1)
        return {k: ms[i] / n for i, k in enumerate(self.TIMELINE_KINDS)}

    @property
    def position(self) -> int:
        return int(self.ctx.lib.gufo_cuda_decoder_position(self.handle))

    def linear_state(self, layer: int):
        c = self.config
        conv = np.empty((c.conv_kernel - 1) * c.conv_channels, dtype=np.float32)
        ssm = np.empty(c.linear_value_heads * c.linear_head_dim ** 2, dtype=np.float32)
        self.ctx._check(self.ctx.lib.gufo_cuda_decoder_linear_state(self.handle, layer, C.c_void_p(conv.ctypes.data),
                                                                    C.c_void_p(ssm.ctypes.data)))
        return conv, ssm
