"""Row-split tensor parallelism of the decode step over the GPUs of one box.

Every output row of a projection is an independent dot product
(src/models/qwen35/gguf_projections.cpp:241-243 in the reference), so a stage's stacked rows
are cut into `world` equal runs; rank r computes run r with this backend's GEMV kernels and an
all-gather over NVLink rebuilds the full vector on every rank: this library's own kernel over
peer memory (gufo_cuda_peer_allgather_device), or NCCL's. The mixers, norms and
activations between the products run replicated (they need the full vectors and are a few
percent of a step's bytes). The reference itself has no distributed execution; this module is
new work on top of its operator interface.

With collective="split" the ranks divide a layer the other way round: each rank owns a share
of the heads (its rows of the input projection, its slice of the mixer, the matching columns
of the output projection) and a share of the FFN width (its gate / up rows, the matching
columns of the down projection). The two column-split products leave partial sums of the whole
output vector; every rank stores its partial into all ranks' arenas and the next product adds
them to the residual in rank order. That is two exchanges per layer instead of four gathers,
and a rank never multiplies, convolves or updates another rank's heads.

One process per GPU (torch.distributed, backend "nccl", for the rendezvous and the comparison
path); the step is captured once per conv parity into a CUDA graph, gathers included.
"""
from __future__ import annotations

import ctypes as C
import json
import os
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

from . import _capi
from . import quantize as Q
from .synth import ModelConfig, Tensor


def shard_rows(parts: Sequence[Tuple[str, int]], rank: int, world: int) -> List[Tuple[str, int, int]]:
    """Cuts the stacked rows of `parts` [(name, rows)] into `world` equal runs and returns run
    `rank` as [(name, first, count)]. The total must divide by `world`."""
    total = sum(rows for _, rows in parts)
    if total % world:
        raise ValueError(f"{total} stacked rows do not divide over {world} ranks")
    per = total // world
    lo, hi = rank * per, (rank + 1) * per
    out, at = [], 0
    for name, rows in parts:
        first, last = max(lo, at), min(hi, at + rows)
        if first < last:
            out.append((name, first - at, last - first))
        at += rows
    return out


def split_plan(cfg: ModelConfig, rank: int, world: int) -> Dict[str, object]:
    """What rank `rank` of `world` owns when the ranks split heads and FFN width: counts and
    first indices. Raises ValueError when the model does not divide that way (column slices must
    be whole 256-value blocks; every rank needs whole heads)."""
    c = cfg
    if c.is_moe:
        raise ValueError("the head split covers dense models")
    if c.heads % world or c.linear_value_heads % world or c.linear_key_heads % world or c.ffn % world:
        raise ValueError("heads and FFN width must divide over the ranks")
    if c.linear_value_heads != c.linear_key_heads:
        raise ValueError("the head split takes DeltaNet layers with as many key heads as value heads")
    heads = c.heads // world
    # A KV head is owned by the ranks whose query heads share it: whole KV heads per rank while
    # there are enough of them, one (replicated over neighbouring ranks) afterwards.
    if c.kv_heads % world == 0:
        kv_heads, kv_first = c.kv_heads // world, rank * (c.kv_heads // world)
    elif world % c.kv_heads == 0:
        kv_heads, kv_first = 1, rank // (world // c.kv_heads)
    else:
        raise ValueError("KV heads and ranks must divide one another")
    linear = c.linear_value_heads // world
    plan = {"heads": heads, "head_first": rank * heads, "kv_heads": kv_heads, "kv_first": kv_first,
            "linear_heads": linear, "linear_first": rank * linear, "ffn": c.ffn // world, "ffn_first": rank * (c.ffn // world)}
    for cols in (heads * c.head_dim, linear * c.linear_head_dim, plan["ffn"]):
        if cols % 256:
            raise ValueError("a rank's columns of the output and down projections must be whole 256-value blocks")
    return plan


def stage_tensors(cfg: ModelConfig, il: int, gates_in_mixer: bool = False) -> Dict[str, List[str]]:
    """GGUF tensor names stacked per stage of layer `il`, in the reference's order
    (src/models/qwen35/gguf_projections.cpp:139-171). With `gates_in_mixer` the DeltaNet input
    stage stops after [qkv | z]: the F32 alpha / beta rows are multiplied inside the mixer's
    kernel (as the reference's fused step does, src/models/qwen35_2b/deltanet.cpp:358-392)."""
    p = f"blk.{il}."
    if cfg.is_full_attention(il):
        first = [p + "attn_q.weight", p + "attn_k.weight", p + "attn_v.weight"]
        out = [p + "attn_output.weight"]
    else:
        first = [p + "attn_qkv.weight", p + "attn_gate.weight"]
        if not gates_in_mixer:
            first += [p + "ssm_alpha.weight", p + "ssm_beta.weight"]
        out = [p + "ssm_out.weight"]
    return {"in": first, "out": out, "ffn_in": [p + "ffn_gate.weight", p + "ffn_up.weight"],
            "ffn_down": [p + "ffn_down.weight"]}


class TpDecoder:
    """One rank of the row-split decode step (dense models)."""

    def __init__(self, ctx, cfg: ModelConfig, tensors: Dict[str, Tensor], rank: int, world: int,
                 max_positions: int = 4096, collective: str = "peer"):
        """`collective`: "fused" lets every product store its rows into the peers' copies of
        the full vector itself (gufo_cuda_matmul_gather_device: product and gather in one
        kernel); "peer" gathers with a separate kernel over NVLink peer memory
        (gufo_cuda_peer_allgather_device); "nccl" with torch.distributed's all-gather."""
        self.ctx, self.cfg, self.rank, self.world = ctx, cfg, rank, world
        self.collective = collective if world > 1 or collective == "split" else "none"
        self.fused = self.collective == "fused"
        self.split = self.collective == "split"
        self.lib = ctx.lib
        dev = torch.device("cuda", ctx.device)
        self.dev = dev
        self._keep = []
        c = cfg
        self.position_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self.token_dev = torch.zeros(1, dtype=torch.int32, device=dev)
        self.position = 0
        self.graphs = {}
        self.kernels_per_step = 0
        self.replayed_kernels = 0      # this backend's kernels launched through graph replays
        self.max_positions = max_positions
        self.inv_freq = torch.tensor([1.0 / (float(c.rope_theta) ** (2.0 * i / c.rope_dim))
                                      for i in range(c.rope_dim // 2)], dtype=torch.float64).float().to(dev)
        if self.split:
            self._init_split(tensors)
            return

        def f32(name):
            t = tensors[name].data.to(dev).view(torch.float32).contiguous()
            self._keep.append(t)
            return t

        def product(names):
            """(parts array, nparts, local rows, total rows) of this rank's run of a stage."""
            runs = shard_rows([(n, tensors[n].rows) for n in names], rank, world)
            arr = (_capi.Rows * len(runs))()
            for i, (name, first, count) in enumerate(runs):
                t = tensors[name]
                rb = Q.row_bytes(t.ggml_type, t.cols)
                # A rank keeps its own rows only: a copy of the run, so that the whole tensor can
                # be released once every stage has been cut.
                view = t.data[first * rb:(first + count) * rb].to(dev)
                if world > 1 and view.data_ptr() == t.data.data_ptr() + first * rb:
                    view = view.clone()
                self._keep.append(view)
                arr[i] = _capi.Rows(ctx.matrix_from_device(t.ggml_type, view.data_ptr(), count, t.cols), 0, count)
            local = sum(count for _, _, count in runs)
            return arr, len(runs), local, local * world

        self.layers = []
        for il in range(c.layers):
            names = stage_tensors(c, il, gates_in_mixer=self.fused)
            layer = {k: product(v) for k, v in names.items()}
            p = f"blk.{il}."
            layer["attn_norm"] = f32(p + "attn_norm.weight")
            layer["post_norm"] = f32(p + "post_attention_norm.weight")
            if c.is_full_attention(il):
                layer["q_norm"] = f32(p + "attn_q_norm.weight")
                layer["k_norm"] = f32(p + "attn_k_norm.weight")
                kv = c.kv_heads * c.head_dim
                layer["keys"] = torch.zeros(max_positions, kv, dtype=torch.float16, device=dev)
                layer["values"] = torch.zeros(max_positions, kv, dtype=torch.float16, device=dev)
            else:
                layer["linear"] = ctx.deltanet_layer_create(
                    c.linear_key_heads, c.linear_value_heads, c.linear_head_dim, c.conv_kernel, c.rms_eps,
                    *(tensors[p + n].data.cpu().numpy().view(np.float32) for n in
                      ("ssm_conv1d.weight", "ssm_a", "ssm_dt.bias", "ssm_norm.weight")))
                if self.fused:
                    # The whole F32 alpha / beta rows on every rank: the mixer multiplies them.
                    layer["gates"] = tuple(
                        ctx.matrix_upload(tensors[p + n].ggml_type, tensors[p + n].data.cpu().numpy(), tensors[p + n].rows,
                                          tensors[p + n].cols) for n in ("ssm_alpha.weight", "ssm_beta.weight"))
                layer["conv"] = [torch.zeros((c.conv_kernel - 1) * c.conv_channels, device=dev) for _ in range(2)]
                layer["ssm"] = torch.zeros(c.linear_value_heads * c.linear_head_dim ** 2, device=dev)
            self.layers.append(layer)
        head = "token_embd.weight" if c.tied_embeddings else "output.weight"
        self.lm_head = product([head])
        embed = tensors["token_embd.weight"]
        self._embed_data = embed.data.to(dev)
        self.embed = ctx.matrix_from_device(embed.ggml_type, self._embed_data.data_ptr(), embed.rows, embed.cols)
        self.output_norm = f32("output_norm.weight")
        width = max(l["in"][3] for l in self.layers)
        z = lambda n: torch.zeros(n, device=dev)
        self.h, self.normed = z(c.hidden), z(c.hidden)
        self.h_next = z(c.hidden)
        self._residual = (self.h, self.h_next)
        self.mixed = z(max(c.value_dim, c.heads * c.head_dim))
        self.act = z(c.ffn)
        # The vectors every rank needs whole: in the peer arena when this library gathers them.
        full_sizes = (width, c.hidden, 2 * c.ffn, c.vocab)
        self.peers = None
        if self.collective in ("peer", "fused"):
            from .backend import PeerGroup

            def exchange(handle):
                handles = [None] * world
                dist.all_gather_object(handles, handle)
                return handles
            try:
                self.peers = PeerGroup(ctx, rank, world, sum(n + 64 for n in full_sizes), exchange)
            except Exception as e:   # noqa: BLE001 - e.g. a box whose GPUs cannot open each other's memory
                import sys
                print(f"rank {rank}: no peer-memory group ({e}); gathering with NCCL", file=sys.stderr, flush=True)
            # Every rank or none: the ranks agree before anyone gathers (the reduction is also the
            # barrier after which all flags are zero).
            ok = torch.tensor([1 if self.peers is not None else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                if self.peers is not None:
                    self.peers.close()
                self.peers = None
                if self.fused:
                    raise RuntimeError("the fused gather needs the peers' arenas; use collective=\"nccl\"")
                self.collective = "nccl"
        full = self.peers.buffer if self.peers is not None else z
        self.full_in, self.out, self.ffn, self.logits = (full(n) for n in full_sizes)
        self.local = z(max(max(max(l[k][2] for k in ("in", "out", "ffn_in", "ffn_down")) for l in self.layers),
                           self.lm_head[2]))
        self.queries = z(c.heads * c.head_dim)
        self.partials = z(c.kv_heads * 32 * (c.heads // c.kv_heads) * (c.head_dim + 2))
        self.gathers_per_step = 4 * c.layers + 1

    def _init_split(self, tensors: Dict[str, Tensor]) -> None:
        """The rank's share of every layer for collective="split" (see the module text)."""
        ctx, c, rank, world, dev = self.ctx, self.cfg, self.rank, self.world, self.dev
        plan = split_plan(c, rank, world)
        self.plan = plan

        def f32(name):
            t = tensors[name].data.to(dev).view(torch.float32).contiguous()
            self._keep.append(t)
            return t

        def rows_of(name, first, count):
            """Rows [first, first + count) of a tensor as a matrix of their own."""
            t = tensors[name]
            rb = Q.row_bytes(t.ggml_type, t.cols)
            view = t.data[first * rb:(first + count) * rb].to(dev).clone()
            self._keep.append(view)
            return _capi.Rows(ctx.matrix_from_device(t.ggml_type, view.data_ptr(), count, t.cols), 0, count)

        def cols_of(name, first, count):
            """Columns [first, first + count) (whole 256-value blocks) of every row."""
            t = tensors[name]
            bb = Q.row_bytes(t.ggml_type, 256)
            blocks = t.cols // 256
            view = t.data.to(dev).view(t.rows, blocks, bb)[:, first // 256:(first + count) // 256, :].contiguous().view(-1)
            self._keep.append(view)
            return _capi.Rows(ctx.matrix_from_device(t.ggml_type, view.data_ptr(), t.rows, count), 0, t.rows)

        def stack(*rows):
            arr = (_capi.Rows * len(rows))(*rows)
            local = sum(int(r.rows) for r in rows)
            return arr, len(rows), local, local * world

        hd, dk = c.head_dim, c.linear_head_dim
        nh, h0 = plan["heads"], plan["head_first"]
        nkv, kv0 = plan["kv_heads"], plan["kv_first"]
        nl, l0 = plan["linear_heads"], plan["linear_first"]
        nf, f0 = plan["ffn"], plan["ffn_first"]
        key_dim = c.linear_key_heads * dk
        self.layers = []
        for il in range(c.layers):
            p = f"blk.{il}."
            layer = {"attn_norm": f32(p + "attn_norm.weight"), "post_norm": f32(p + "post_attention_norm.weight")}
            if c.is_full_attention(il):
                layer["in"] = stack(rows_of(p + "attn_q.weight", h0 * 2 * hd, nh * 2 * hd),
                                    rows_of(p + "attn_k.weight", kv0 * hd, nkv * hd),
                                    rows_of(p + "attn_v.weight", kv0 * hd, nkv * hd))
                layer["out"] = stack(cols_of(p + "attn_output.weight", h0 * hd, nh * hd))
                layer["q_norm"] = f32(p + "attn_q_norm.weight")
                layer["k_norm"] = f32(p + "attn_k_norm.weight")
                layer["keys"] = torch.zeros(self.max_positions, nkv * hd, dtype=torch.float16, device=dev)
                layer["values"] = torch.zeros(self.max_positions, nkv * hd, dtype=torch.float16, device=dev)
            else:
                # [q | k | v | z] of the rank's heads, as a smaller layer of its own.
                layer["in"] = stack(rows_of(p + "attn_qkv.weight", l0 * dk, nl * dk),
                                    rows_of(p + "attn_qkv.weight", key_dim + l0 * dk, nl * dk),
                                    rows_of(p + "attn_qkv.weight", 2 * key_dim + l0 * dk, nl * dk),
                                    rows_of(p + "attn_gate.weight", l0 * dk, nl * dk))
                layer["out"] = stack(cols_of(p + "ssm_out.weight", l0 * dk, nl * dk))
                conv = tensors[p + "ssm_conv1d.weight"].data.cpu().numpy().view(np.float32).reshape(-1, c.conv_kernel)
                mine = np.concatenate([conv[l0 * dk:(l0 + nl) * dk], conv[key_dim + l0 * dk:key_dim + (l0 + nl) * dk],
                                       conv[2 * key_dim + l0 * dk:2 * key_dim + (l0 + nl) * dk]])
                small = lambda n: tensors[p + n].data.cpu().numpy().view(np.float32)
                layer["linear"] = ctx.deltanet_layer_create(
                    nl, nl, dk, c.conv_kernel, c.rms_eps, np.ascontiguousarray(mine).reshape(-1),
                    np.ascontiguousarray(small("ssm_a")[l0:l0 + nl]), np.ascontiguousarray(small("ssm_dt.bias")[l0:l0 + nl]),
                    small("ssm_norm.weight"))
                layer["gates"] = tuple(
                    ctx.matrix_upload(Q.GGML_F32, np.ascontiguousarray(
                        small(n).reshape(c.linear_value_heads, c.hidden)[l0:l0 + nl]).view(np.uint8).reshape(-1), nl, c.hidden)
                    for n in ("ssm_alpha.weight", "ssm_beta.weight"))
                layer["conv"] = [torch.zeros((c.conv_kernel - 1) * 3 * nl * dk, device=dev) for _ in range(2)]
                layer["ssm"] = torch.zeros(nl * dk * dk, device=dev)
            layer["ffn_in"] = stack(rows_of(p + "ffn_gate.weight", f0, nf), rows_of(p + "ffn_up.weight", f0, nf))
            layer["ffn_down"] = stack(cols_of(p + "ffn_down.weight", f0, nf))
            self.layers.append(layer)
        head = "token_embd.weight" if c.tied_embeddings else "output.weight"
        if c.vocab % world:
            raise ValueError("the LM head's rows must divide over the ranks")
        self.lm_head = stack(rows_of(head, rank * (c.vocab // world), c.vocab // world))
        embed = tensors["token_embd.weight"]
        self._embed_data = embed.data.to(dev)
        self.embed = ctx.matrix_from_device(embed.ggml_type, self._embed_data.data_ptr(), embed.rows, embed.cols)
        self.output_norm = f32("output_norm.weight")
        z = lambda n: torch.zeros(n, device=dev)
        self.h, self.h_next, self.normed = z(c.hidden), z(c.hidden), z(c.hidden)
        self._residual = (self.h, self.h_next)
        self.local_in = z(max(l["in"][2] for l in self.layers))
        self.mixed = z(max(nh * hd, nl * dk))
        self.ffn_rows = z(2 * nf)
        self.act = z(nf)
        self.local = z(self.lm_head[2])
        self.queries = z(nh * hd)
        self.partials = z(nkv * 32 * (nh // nkv) * (hd + 2))
        from .backend import PeerGroup

        def exchange(handle):
            handles = [None] * world
            if world > 1:
                dist.all_gather_object(handles, handle)
            else:
                handles[0] = handle
            return handles
        sizes = (world * c.hidden, world * c.hidden, c.vocab)
        self.peers = PeerGroup(ctx, rank, world, sum(n + 64 for n in sizes), exchange)
        if world > 1:
            ok = torch.tensor([1], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)   # every arena is open and zeroed before anyone stores
        # The partial sums of the output and of the down projection, [world][hidden] each, and the logits.
        self.part_out, self.part_down, self.logits = (self.peers.buffer(n) for n in sizes)
        self.gathers_per_step = 2 * c.layers + 1

    def _split_product(self, prod, *, x=None, swiglu=False, residual=None, delta=None, norm_weight=None,
                       wait_slot: int = -1, store=None, slot: int = -1, local=None, advance: bool = False) -> None:
        """One product of the head-split step. `store` (an arena vector) and `slot`: the rows go
        to every rank's copy, this rank's at rank * rows; else they stay in `local`, and the
        input's `wait_slot` is awaited. `delta`: the [world][hidden] partial sums to add."""
        arr, n, *_ = prod
        kind = _capi.PROLOGUE_RES_NORM if residual is not None else (
            _capi.PROLOGUE_SWIGLU if swiglu else _capi.PROLOGUE_PLAIN)
        p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
        dst = self.h_next if residual is not None else None
        args = _capi.FusedInput(kind, p(x), p(residual), p(delta), p(norm_weight), self.cfg.rms_eps, p(dst),
                                p(self.normed if residual is not None else self.act),
                                p(self.position_dev) if advance else None,
                                self.world if delta is not None else 0, self.cfg.hidden)
        if store is not None:
            self._check(self.lib.gufo_cuda_matmul_gather_device(self.peers.handle, arr, n, C.byref(args),
                                                                self.peers.offset_of(store), slot, wait_slot))
        elif wait_slot >= 0:
            self._check(self.lib.gufo_cuda_matmul_wait_device(self.peers.handle, arr, n, C.byref(args), wait_slot,
                                                              C.c_void_p(local.data_ptr())))
        else:
            self._check(self.lib.gufo_cuda_matmul_fused_device(self.ctx.handle, arr, n, C.byref(args), 1,
                                                               C.c_void_p(local.data_ptr())))
        if residual is not None:
            self.h, self.h_next = self.h_next, self.h

    def enqueue_split(self, parity: int) -> None:
        """The head-split step. Slot 1: the output projections' partial sums, slot 2: the down
        projections', slot 3: the logits."""
        c, plan = self.cfg, self.plan
        lib, h = self.lib, self.ctx.handle
        self.h, self.h_next = self._residual
        self._check(lib.gufo_cuda_embed_device(h, self.embed, self.token_dev.data_ptr(), self.h.data_ptr()))
        pending, pending_slot = None, -1
        for il, l in enumerate(self.layers):
            self._split_product(l["in"], residual=self.h, delta=pending, norm_weight=l["attn_norm"],
                                wait_slot=pending_slot, local=self.local_in)
            if c.is_full_attention(il):
                args = _capi.AttentionArgs(plan["heads"], plan["kv_heads"], c.head_dim, c.rope_dim, self.max_positions,
                                           c.rms_eps, self.position_dev.data_ptr(), self.local_in.data_ptr(),
                                           l["q_norm"].data_ptr(), l["k_norm"].data_ptr(), self.inv_freq.data_ptr(),
                                           l["keys"].data_ptr(), l["values"].data_ptr(), self.queries.data_ptr(),
                                           self.partials.data_ptr(), self.mixed.data_ptr())
                self._check(lib.gufo_cuda_attention_device(h, C.byref(args)))
            else:
                # The gates from the residual stream (the product's norm wrote it to self.h).
                seq = _capi.DeltaNetStepSeq(1, self.local_in.data_ptr(), 0, self.h.data_ptr(), 0,
                                            l["conv"][parity].data_ptr(), l["conv"][parity ^ 1].data_ptr(), None,
                                            l["ssm"].data_ptr(), None, self.mixed.data_ptr(), 0)
                alpha, beta = l["gates"]
                self._check(lib.gufo_cuda_deltanet_step_device(h, l["linear"], alpha, beta,
                                                               C.c_void_p(l["attn_norm"].data_ptr()), c.rms_eps,
                                                               C.byref(seq), 1))
            self._split_product(l["out"], x=self.mixed, store=self.part_out, slot=1)
            self._split_product(l["ffn_in"], residual=self.h, delta=self.part_out, norm_weight=l["post_norm"],
                                wait_slot=1, local=self.ffn_rows)
            self._split_product(l["ffn_down"], x=self.ffn_rows, swiglu=True, store=self.part_down, slot=2)
            pending, pending_slot = self.part_down, 2
        self._split_product(self.lm_head, residual=self.h, delta=pending, norm_weight=self.output_norm,
                            wait_slot=pending_slot, store=self.logits, slot=3, advance=True)
        self._check(lib.gufo_cuda_peer_wait_device(self.peers.handle, 3))

    def _check(self, status):
        _capi.check(self.lib, self.ctx.handle, status)

    def _gather(self, prod, y_full):
        _, _, local, total = prod
        if self.world == 1:
            y_full[:total].copy_(self.local[:local])
        elif self.peers is not None:
            self.peers.allgather(self.local, y_full, local)
        else:
            dist.all_gather_into_tensor(y_full[:total], self.local[:local])

    def _product(self, prod, x, y_full, swiglu=False):
        """Local rows of a stage into self.local (x plain, or [gate | up] rows through SwiGLU
        inside the product), then all-gather into y_full."""
        arr, n, _, _ = prod
        if swiglu:
            self.ctx.matmul_fused_device(arr, n, 1, self.local, x=x, swiglu=True, scratch=self.act)
        else:
            self.ctx.matmul_device(arr, n, x, 1, self.local)
        self._gather(prod, y_full)

    def _norm_product(self, prod, delta, weight, y_full, advance=False):
        """The residual add + RMSNorm inside the product's kernels (the residual stream
        alternates between two buffers), then the all-gather."""
        arr, n, _, _ = prod
        src, dst = self.h, self.h_next
        self.ctx.matmul_fused_device(arr, n, 1, self.local, residual=src, delta=delta, norm_weight=weight,
                                     rms_eps=self.cfg.rms_eps, residual_out=dst, scratch=self.normed,
                                     advance=self.position_dev if advance else None)
        self.h, self.h_next = dst, src
        self._gather(prod, y_full)

    def enqueue(self, parity: int) -> None:
        c = self.cfg
        lib, h = self.lib, self.ctx.handle
        self.h, self.h_next = self._residual   # every step starts in the same buffer (graphs keep addresses)
        self._check(lib.gufo_cuda_embed_device(h, self.embed, self.token_dev.data_ptr(), self.h.data_ptr()))
        pending = None
        for il, l in enumerate(self.layers):
            self._norm_product(l["in"], pending, l["attn_norm"], self.full_in)
            if c.is_full_attention(il):
                args = _capi.AttentionArgs(c.heads, c.kv_heads, c.head_dim, c.rope_dim, self.max_positions, c.rms_eps,
                                           self.position_dev.data_ptr(), self.full_in.data_ptr(),
                                           l["q_norm"].data_ptr(), l["k_norm"].data_ptr(), self.inv_freq.data_ptr(),
                                           l["keys"].data_ptr(), l["values"].data_ptr(), self.queries.data_ptr(),
                                           self.partials.data_ptr(), self.mixed.data_ptr())
                self._check(lib.gufo_cuda_attention_device(h, C.byref(args)))
            else:
                self.ctx.deltanet_linear_device(l["linear"], [{
                    "in": self.full_in, "conv_in": l["conv"][parity], "conv_out": l["conv"][parity ^ 1],
                    "ssm": l["ssm"], "y": self.mixed}])
            self._product(l["out"], self.mixed, self.out)
            self._norm_product(l["ffn_in"], self.out, l["post_norm"], self.ffn)
            self._product(l["ffn_down"], self.ffn, self.out, swiglu=True)
            pending = self.out
        self._norm_product(self.lm_head, pending, self.output_norm, self.logits, advance=True)

    def _gather_product(self, prod, full, slot: int, wait_slot: int, *, x=None, residual=None, delta=None,
                        norm_weight=None, swiglu: bool = False, advance: bool = False) -> None:
        """A stage's local rows by the kernel that also stores them into every rank's `full`
        vector and raises the slot's flag; `wait_slot` >= 0: its input is the vector of that slot."""
        arr, n, _, _ = prod
        kind = _capi.PROLOGUE_RES_NORM if residual is not None else (
            _capi.PROLOGUE_SWIGLU if swiglu else _capi.PROLOGUE_PLAIN)
        p = lambda t: C.c_void_p(t.data_ptr()) if t is not None else None
        dst = None
        if residual is not None:
            dst = self.h_next
        args = _capi.FusedInput(kind, p(x), p(residual), p(delta), p(norm_weight), self.cfg.rms_eps, p(dst),
                                p(self.normed if residual is not None else self.act),
                                p(self.position_dev) if advance else None)
        self._check(self.lib.gufo_cuda_matmul_gather_device(self.peers.handle, arr, n, C.byref(args),
                                                            self.peers.offset_of(full), slot, wait_slot))
        if residual is not None:
            self.h, self.h_next = self.h_next, self.h

    def enqueue_fused(self, parity: int) -> None:
        """The step with every product gathering by itself. Vector slots: 0 the mixers' input,
        1 the projections' output (twice per layer), 2 the FFN rows, 3 the logits."""
        c = self.cfg
        lib, h = self.lib, self.ctx.handle
        self.h, self.h_next = self._residual
        self._check(lib.gufo_cuda_embed_device(h, self.embed, self.token_dev.data_ptr(), self.h.data_ptr()))
        pending, pending_slot = None, -1
        for il, l in enumerate(self.layers):
            self._gather_product(l["in"], self.full_in, 0, pending_slot, residual=self.h, delta=pending,
                                 norm_weight=l["attn_norm"])
            self._check(lib.gufo_cuda_peer_wait_device(self.peers.handle, 0))
            if c.is_full_attention(il):
                args = _capi.AttentionArgs(c.heads, c.kv_heads, c.head_dim, c.rope_dim, self.max_positions, c.rms_eps,
                                           self.position_dev.data_ptr(), self.full_in.data_ptr(),
                                           l["q_norm"].data_ptr(), l["k_norm"].data_ptr(), self.inv_freq.data_ptr(),
                                           l["keys"].data_ptr(), l["values"].data_ptr(), self.queries.data_ptr(),
                                           self.partials.data_ptr(), self.mixed.data_ptr())
                self._check(lib.gufo_cuda_attention_device(h, C.byref(args)))
            else:
                # The gates from the residual stream (the product's norm wrote it to self.h).
                seq = _capi.DeltaNetStepSeq(1, self.full_in.data_ptr(), 0, self.h.data_ptr(), 0,
                                            l["conv"][parity].data_ptr(), l["conv"][parity ^ 1].data_ptr(), None,
                                            l["ssm"].data_ptr(), None, self.mixed.data_ptr(), 0)
                alpha, beta = l["gates"]
                self._check(lib.gufo_cuda_deltanet_step_device(h, l["linear"], alpha, beta,
                                                               C.c_void_p(l["attn_norm"].data_ptr()), c.rms_eps,
                                                               C.byref(seq), 1))
            self._gather_product(l["out"], self.out, 1, -1, x=self.mixed)
            self._gather_product(l["ffn_in"], self.ffn, 2, 1, residual=self.h, delta=self.out,
                                 norm_weight=l["post_norm"])
            self._gather_product(l["ffn_down"], self.out, 1, 2, x=self.ffn, swiglu=True)
            pending, pending_slot = self.out, 1
        self._gather_product(self.lm_head, self.logits, 3, pending_slot, residual=self.h, delta=pending,
                             norm_weight=self.output_norm, advance=True)
        self._check(lib.gufo_cuda_peer_wait_device(self.peers.handle, 3))

    def step(self, token: int, stream, use_graph: bool = True) -> torch.Tensor:
        """Runs `token` at the current position on every rank; returns the full logits (device)."""
        if self.position >= self.max_positions:
            raise RuntimeError("the attention cache is full")
        self.token_dev.fill_(token)
        parity = self.position & 1
        enqueue = self.enqueue_split if self.split else (self.enqueue_fused if self.fused else self.enqueue)
        if not use_graph or self.position < 2:
            enqueue(parity)
        else:
            if parity not in self.graphs:
                g = torch.cuda.CUDAGraph()
                torch.cuda.synchronize()
                before = self.ctx.launch_count()
                with torch.cuda.graph(g, stream=stream):
                    enqueue(parity)
                self.kernels_per_step = self.ctx.launch_count() - before
                self.graphs[parity] = g
            self.graphs[parity].replay()
            self.replayed_kernels += self.kernels_per_step
        self.position += 1
        return self.logits


PARITY_TOKENS = (11, 4242, 98765, 7)   # the first steps of every decoder in run_bench


def first_logits(step, vocab: int) -> np.ndarray:
    """Logits [len(PARITY_TOKENS), vocab] of a fresh decoder's first steps (`step(token)` returns
    a host array or a device tensor)."""
    rows = []
    for tok in PARITY_TOKENS:
        out = step(tok % vocab)
        rows.append(out.detach().cpu().numpy().copy() if isinstance(out, torch.Tensor) else np.array(out, copy=True))
    return np.stack(rows)


def rel_l2(got: np.ndarray, want: np.ndarray) -> float:
    got, want = got.astype(np.float64), want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def run_bench(args, cfg: ModelConfig, metric: str, unit: str, workload: str) -> None:
    """bench.py's N > 1 arm: launched by torchrun, one rank per GPU."""
    from . import synth
    from .backend import Context
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    # The line this arm prints is the only thing on stdout: whatever the libraries write there
    # (NCCL's version banner, for one) goes to stderr, the line itself to the saved descriptor.
    import sys
    sys.stdout.flush()
    line_out = os.dup(1)
    os.dup2(2, 1)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    stream = torch.cuda.Stream()
    torch.cuda.set_stream(stream)
    tensors = synth.build_model(cfg, seed=1, device=f"cuda:{local}")
    ctx = Context(local, stream.cuda_stream)
    steps, warmup = args.steps, max(args.warmup, 3)
    rng = np.random.default_rng(7)
    tokens = iter(rng.integers(0, cfg.vocab, size=40 * (steps + warmup) + 64).tolist())
    host = torch.empty(cfg.vocab, dtype=torch.float32).pin_memory()
    positions = 8 * (steps + warmup) + 64

    def timed(fn):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / steps], device=f"cuda:{local}")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # The ways to run the step over the ranks: heads and FFN width split (partial sums exchanged
    # twice per layer), or rows split with the full vectors rebuilt by every product storing its
    # rows into the peers' arenas itself, by a separate gather kernel, by NCCL. Each decoder
    # starts with the same few tokens (their logits are compared below), warms up, and is timed;
    # the line's value is the fastest, `parallelism` names it and gives the others' times.
    how = {"split": "heads and FFN width split over the ranks: a rank multiplies its heads' input rows, runs its "
                    "slice of the mixer, and the column-split output and down products store partial sums into "
                    "every rank's arena (NVLink peer stores, flags) that the next product adds to the residual: "
                    "two exchanges per layer",
           "fused": "every product stores its rows into the peers' copies itself (one kernel per stage, "
                    "NVLink peer stores, flags)",
           "peer": "a gather kernel of this library over NVLink peer memory after every product",
           "nccl": "NCCL's all-gather after every product"}
    parity_logits, measured, decoders = {}, {}, {}
    for name in ("split", "fused", "peer", "nccl"):
        ok = 1
        d = None
        try:
            d = TpDecoder(ctx, cfg, tensors, rank, world, max_positions=positions, collective=name)
            if d.collective != name:
                ok = 0   # the peers' arenas could not be opened: this decoder fell back to NCCL
        except Exception as e:   # noqa: BLE001
            import sys
            print(f"rank {rank}: no {name} decoder ({e})", file=sys.stderr, flush=True)
            ok = 0
        agreed = torch.tensor([ok], device=f"cuda:{local}")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            del d
            continue
        parity_logits[name] = first_logits(lambda t, d=d: d.step(t, stream), cfg.vocab)
        for _ in range(warmup):
            d.step(next(tokens), stream)
        torch.cuda.synchronize()
        healthy = 1
        if d.peers is not None:
            try:
                d.peers.status()
            except Exception as e:   # noqa: BLE001 - a wait for a peer's flag ran out
                import sys
                print(f"rank {rank}: {name}: {e}", file=sys.stderr, flush=True)
                healthy = 0
        agreed = torch.tensor([healthy], device=f"cuda:{local}")
        dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
        if int(agreed.item()) == 0:
            d.graphs.clear()
            continue
        before = ctx.launch_count() + d.replayed_kernels
        ms = timed(lambda d=d: d.step(next(tokens), stream))
        measured[name] = (ms, ctx.launch_count() + d.replayed_kernels - before)
        decoders[name] = d
        if d.peers is not None:
            d.peers.status()
    del tensors
    best = min(measured, key=lambda k: measured[k][0])
    dec = decoders[best]
    ms_resident, launches = measured[best]
    gathered_by = how[best]
    other = "; ".join(f"{how[k]}: {measured[k][0]:.3f} ms per step" for k in measured if k != best)
    other = f"; measured beside it: {other}" if other else ""

    def e2e_step():
        logits = dec.step(next(tokens), stream)
        host.copy_(logits, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    ms_e2e = timed(e2e_step)
    # For context beside the row-split number: the same GPUs as independent replicas, every rank
    # decoding its own sequence with the single-GPU resident decoder at the same time (no
    # collective on the data path). Timed the same way: barrier, device events, max over ranks.
    from .backend import CudaDecoder, CudaProjections
    full = synth.build_model(cfg, seed=1, device=f"cuda:{local}")
    replica = CudaDecoder(CudaProjections(ctx, cfg, full), full, max_positions=2 * (steps + warmup) + 64,
                          use_graph=True)
    del full
    parity_logits["one_gpu"] = first_logits(lambda t: replica.Step(t), cfg.vocab)
    for _ in range(warmup):
        replica.step_device(next(tokens))
    torch.cuda.synchronize()
    ms_replica = timed(lambda: replica.step_device(next(tokens)))
    # The row-split decoders against the one-GPU decoder on the same tokens (every rank checks
    # its own copy of the gathered logits; the worst over the ranks is reported), and the two
    # gathers against each other, which must agree bit for bit.
    one = parity_logits.pop("one_gpu")
    worst = max(rel_l2(rows[i], one[i]) for rows in parity_logits.values() for i in range(len(PARITY_TOKENS)))
    same_argmax = all(int(np.argmax(rows[i])) == int(np.argmax(one[i]))
                      for rows in parity_logits.values() for i in range(len(PARITY_TOKENS)))
    gathers_equal = 1
    if "peer" in parity_logits and "nccl" in parity_logits:
        gathers_equal = int(np.array_equal(parity_logits["peer"].view(np.uint32), parity_logits["nccl"].view(np.uint32)))
    check = torch.tensor([worst, 0.0 if same_argmax else 1.0, 0.0 if gathers_equal else 1.0], device=f"cuda:{local}")
    dist.all_reduce(check, op=dist.ReduceOp.MAX)
    worst, argmax_differs, gathers_differ = (float(v) for v in check.tolist())
    parity = {"row_split_vs_one_gpu_logits_rel_l2": worst, "same_argmax": argmax_differs == 0.0,
              "decoders_compared": sorted(parity_logits),
              "peer_and_nccl_gathers_bit_equal": (gathers_differ == 0.0) if "peer" in parity_logits and "nccl" in parity_logits else None,
              "tokens": len(PARITY_TOKENS), "tolerance": 2e-3}
    if worst > 2e-3 or argmax_differs or gathers_differ:
        raise SystemExit(f"row-split parity failed: {parity}")
    # The HBM roofline of the step's largest kernel on a rank: its run of the LM head's rows.
    from .bench_support import measured_hbm_peak
    peak, peak_kind = measured_hbm_peak()
    head_arr, head_n, head_rows, _ = dec.lm_head
    xh = torch.randn(1, cfg.hidden, device=f"cuda:{local}")
    for _ in range(3):
        ctx.matmul_device(head_arr, head_n, xh, 1, dec.local)
    ms_head = timed(lambda: ctx.matmul_device(head_arr, head_n, xh, 1, dec.local))
    head_bytes = head_rows * Q.row_bytes(Q.GGML_Q6_K, cfg.hidden) + 4 * cfg.hidden + 4 * head_rows
    roofline = {"bound": "hbm", "achieved": head_bytes / ms_head / 1e6, "peak": peak, "unit": "GB/s",
                "frac": head_bytes / ms_head / 1e6 / peak, "traffic": None, "peak_kind": peak_kind,
                "kernel": "GemvMma<Q6_K, 1 token>", "shape": f"{head_rows}x{cfg.hidden} Q6_K: one rank's rows of the LM head",
                "bytes_per_launch": head_bytes, "us_per_launch": ms_head * 1e3}
    # The two other sharded paths: the row-split verify batch and the expert-parallel MoE layer.
    for d in decoders.values():
        d.graphs.clear()
    del replica
    torch.cuda.empty_cache()
    from . import mgpu_bench
    sections = {}
    for name, fn in (("verify_batch_row_split", mgpu_bench.verify_batch_tp), ("moe_layer_expert_parallel", mgpu_bench.moe_layer_ep)):
        sections[name] = fn(ctx, rank, world, torch.device("cuda", local), max(steps // 2, 8), peak)
    if rank == 0:
        os.write(line_out, (json.dumps({
            "metric": metric, "value": 1e3 / ms_resident, "unit": unit, "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms_resident, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32 (int8 tensor-core code dots, 24-bit fixed-point activations)",
            "data": "synthetic",
            "config": {"workload": workload, "seed": 1},
            "notes": {"parallelism": (f"tp{world}: {gathered_by} ({dec.gathers_per_step} exchanges per step){other}"
                                      if best == "split" else
                                      f"tp{world}: projections row-split, {dec.gathers_per_step} gathers per step: "
                                      f"{gathered_by}; mixers replicated{other}"),
                      "l2": "weights exceed L2; no flush needed"},
            "e2e": {"value": 1e3 / ms_e2e, "unit": unit, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": cfg.vocab * 4,
                    "ms_per_step": ms_e2e},
            "gpu_launches": int(launches),
            "replicas": {"value": world * 1e3 / ms_replica, "unit": unit, "ms_per_step": ms_replica,
                         "note": "the same GPUs as independent sequences, one resident decoder per GPU, no "
                                 "collective; not the metric's row-split configuration"},
            "parity": parity,
            "roofline": roofline, "cpu_baseline": None,
            "verify_batch_row_split": sections["verify_batch_row_split"],
            "moe_layer_expert_parallel": sections["moe_layer_expert_parallel"],
        }) + "\n").encode())
    dist.barrier()
    torch.cuda.synchronize()
    # Captured graphs hold NCCL kernels: release them before the communicator goes away, and
    # leave without the collective teardown (it blocked here while graphs were alive).
    for d in decoders.values():
        d.graphs.clear()
    import sys
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)
