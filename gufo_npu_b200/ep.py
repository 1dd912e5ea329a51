"""Expert parallelism of the routed-expert FFN over the GPUs of one box.

Experts are independent (GgufProjections::ApplyExpert, src/models/qwen35/gguf_projections.cpp:
218-237 in the reference, picks a row slice per expert), so rank r holds experts
[r * E / G, (r + 1) * E / G) of every layer and the shared expert and router are replicated. Two
exchanges are provided, both without a host round trip (the chosen experts never leave the
device):

* `moe_ffn_replicated`: every rank holds the same tokens (the row-split decode step after its
  all-gather). Each rank runs the pairs whose expert it holds into a zeroed [tokens][k][hidden]
  buffer; one all-reduce (sum) fills in the other ranks' rows. Exactly one rank writes a row, so
  the sum only adds zeros and the result is bit-identical to one GPU.
* `moe_ffn_sharded`: every rank brings its own tokens. An all-to-all carries each rank's token
  rows and per-destination expert ids (-1 where the destination does not hold the expert) to
  every rank, the ranks run the grouped expert FFN on what they received, and a second
  all-to-all returns the rows; the home rank adds them up per slot and combines in slot order as
  Decoder::MoeFfn does (src/models/qwen35/decoder.cpp:541-556). Buffers have a fixed capacity
  (tokens * k pairs per rank pair), so no counts are exchanged.

The reference has no distributed execution; this module is new work on its operator interface.
The plan functions are plain torch ops and run on CPU tensors too (the gloo tests use them with
a host stand-in for the expert FFN).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

import torch
import torch.distributed as dist

from . import _capi
from .backend import Context, CudaProjections, Stage
from .synth import ModelConfig, Tensor


def expert_range(experts: int, rank: int, world: int) -> Tuple[int, int]:
    """(first, count) of the experts rank `rank` holds. `experts` must divide by `world`."""
    if experts % world:
        raise ValueError(f"{experts} experts do not divide over {world} ranks")
    per = experts // world
    return rank * per, per


def local_ids(chosen: torch.Tensor, first: int, count: int) -> torch.Tensor:
    """Global expert ids -> ids within [first, first + count), -1 for experts held elsewhere."""
    held = (chosen >= first) & (chosen < first + count)
    return torch.where(held, chosen - first, torch.full_like(chosen, -1))


def dispatch_ids(chosen: torch.Tensor, experts: int, world: int) -> torch.Tensor:
    """[world][tokens * k] int32: for each destination rank, the local id of every (token, slot)
    pair there, or -1 when that rank does not hold the pair's expert."""
    per = experts // world
    flat = chosen.reshape(1, -1)
    owner = torch.div(flat, per, rounding_mode="floor")
    ranks = torch.arange(world, device=chosen.device, dtype=chosen.dtype).reshape(world, 1)
    return torch.where(owner == ranks, flat - ranks * per, torch.full_like(flat, -1)).contiguous()


def exchange(send: torch.Tensor, group=None) -> torch.Tensor:
    """all_to_all of equal slices along dim 0 (slice r goes to rank r)."""
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv


def sharded_expert_rows(x: torch.Tensor, chosen: torch.Tensor, experts: int, world: int,
                        run_pairs: Callable[[torch.Tensor, torch.Tensor], torch.Tensor],
                        group=None) -> torch.Tensor:
    """The exchange of `moe_ffn_sharded`: x [tokens][hidden] and chosen [tokens][k] of this rank
    -> expert_out [tokens][k][hidden]. `run_pairs(x_pairs [P][hidden], ids [P]) -> y [P][hidden]`
    runs this rank's experts on received pairs, leaving zero rows where ids < 0."""
    tokens, k = chosen.shape
    hidden = x.shape[1]
    ids = exchange(dispatch_ids(chosen, experts, world), group)            # [src][tokens * k]
    rows = exchange(x.unsqueeze(0).expand(world, tokens, hidden).contiguous(), group)  # [src][tokens][hidden]
    pairs = rows.repeat_interleave(k, dim=1).reshape(world * tokens * k, hidden)
    y = run_pairs(pairs, ids.reshape(-1))
    back = exchange(y.reshape(world, tokens * k, hidden), group)           # [owner][tokens * k][hidden]
    # Exactly one owner holds a non-zero row per pair: the sum adds zeros only.
    return back.sum(dim=0).reshape(tokens, k, hidden)


class EpMoe:
    """One rank's share of the routed experts of a MoE model, with the exchanges above.

    `tensors` are the full model's tensors; only this rank's slice of the stacked expert tensors
    is uploaded. Router and shared expert come from `projections` (replicated). The context
    must enqueue on torch's current stream (torch ops and collectives sit between its kernels).
    """

    def __init__(self, ctx: Context, cfg: ModelConfig, tensors: Dict[str, Tensor], projections: CudaProjections,
                 rank: int, world: int, max_tokens: int = 4, group=None):
        if not cfg.is_moe:
            raise RuntimeError("qwen35: not a MoE model")
        self.ctx, self.cfg, self.rank, self.world, self.group = ctx, cfg, rank, world, group
        self.projections = projections
        self.max_tokens = max_tokens
        self.first, self.count = expert_range(cfg.experts, rank, world)
        dev = torch.device("cuda", ctx.device)
        self.dev = dev
        c = cfg
        self.banks = []
        self._keep = []
        for il in range(c.layers):
            handles = []
            for name, rows in (("ffn_gate_exps.weight", c.expert_ffn), ("ffn_up_exps.weight", c.expert_ffn),
                               ("ffn_down_exps.weight", c.hidden)):
                t = tensors[f"blk.{il}.{name}"]
                data = t.data.reshape(t.rows, -1)[self.first * rows:(self.first + self.count) * rows].contiguous()
                if data.is_cuda:
                    self._keep.append(data)
                    handles.append(ctx.matrix_from_device(t.ggml_type, data.data_ptr(), self.count * rows, t.cols))
                else:
                    handles.append(ctx.matrix_upload(t.ggml_type, data.numpy(), self.count * rows, t.cols))
            self.banks.append(_capi.ExpertBank(*handles, self.count, c.expert_ffn, c.hidden))
        k = c.experts_used
        f32 = dict(dtype=torch.float32, device=dev)
        pairs = world * max_tokens * k
        self.router = torch.empty(max_tokens, c.experts + 1, **f32)
        self.chosen = torch.empty(max_tokens, k, dtype=torch.int32, device=dev)
        self.weights = torch.empty(max_tokens, k, **f32)
        self.scale = torch.empty(max_tokens, **f32)
        self.ffn = torch.empty(pairs, 2 * c.expert_ffn, **f32)
        self.act = torch.empty(pairs, c.expert_ffn, **f32)
        self.expert_out = torch.zeros(max_tokens, k, c.hidden, **f32)

    def route(self, layer: int, normed: torch.Tensor, tokens: int) -> None:
        c = self.cfg
        self.projections.apply_device(Stage.kRouter, layer, normed, tokens, self.router)
        self.ctx.route_device(self.router, c.experts + 1, tokens, c.experts, c.experts_used, self.chosen,
                              self.weights, self.scale)

    def _run_pairs(self, layer: int, x_pairs: torch.Tensor, ids: torch.Tensor, x_stride: Optional[int] = None):
        pairs = ids.numel()
        y = torch.zeros(pairs, self.cfg.hidden, dtype=torch.float32, device=self.dev)
        self.ctx.expert_ffn_device(self.banks[layer], ids.contiguous(), pairs, x_pairs,
                                   self.cfg.hidden if x_stride is None else x_stride, self.ffn, self.act, y)
        return y

    def moe_ffn_replicated(self, layer: int, normed: torch.Tensor, shared: torch.Tensor, tokens: int,
                           out: torch.Tensor) -> None:
        """Every rank holds the same `tokens` rows; one all-reduce of the experts' rows."""
        c = self.cfg
        k = c.experts_used
        self.ctx.require_torch_stream()
        self.route(layer, normed, tokens)
        ids = local_ids(self.chosen[:tokens], self.first, self.count)
        pairs = tokens * k
        y = torch.zeros(pairs, c.hidden, dtype=torch.float32, device=self.dev)
        self.ctx.expert_ffn_device(self.banks[layer], ids.reshape(-1).contiguous(), pairs, normed, c.hidden, self.ffn,
                                   self.act, y, pairs_per_input=k)
        if self.world > 1:
            dist.all_reduce(y, group=self.group)
        self.expert_out[:tokens] = y.reshape(tokens, k, c.hidden)
        self.ctx.moe_combine_device(shared, self.scale, self.weights, self.expert_out, tokens, k, c.hidden, out)

    def moe_ffn_sharded(self, layer: int, normed: torch.Tensor, shared: torch.Tensor, tokens: int,
                        out: torch.Tensor) -> None:
        """This rank's own `tokens` rows (the same count on every rank); two all-to-alls."""
        c = self.cfg
        k = c.experts_used
        self.ctx.require_torch_stream()
        self.route(layer, normed, tokens)
        rows = sharded_expert_rows(normed[:tokens], self.chosen[:tokens], c.experts, self.world,
                                   lambda x, ids: self._run_pairs(layer, x, ids), self.group)
        self.expert_out[:tokens] = rows
        self.ctx.moe_combine_device(shared, self.scale, self.weights, self.expert_out, tokens, k, c.hidden, out)
