"""Expert parallelism, host logic on the CPU: the dispatch plan and the two all-to-alls of the
token-sharded exchange with two `gloo` ranks. The expert FFN itself comes from the CPU oracle
here; on a GPU each rank runs this backend's grouped kernels in its place."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gufo_npu_b200 import synth
from gufo_npu_b200.ep import dispatch_ids, expert_range, local_ids, sharded_expert_rows
from tests.golden import make_golden as G


def test_expert_range_and_local_ids():
    assert [expert_range(256, r, 4) for r in range(4)] == [(0, 64), (64, 64), (128, 64), (192, 64)]
    with pytest.raises(ValueError):
        expert_range(10, 0, 4)
    chosen = torch.tensor([[0, 63, 64, 255], [128, 5, 200, 70]], dtype=torch.int32)
    assert local_ids(chosen, 64, 64).tolist() == [[-1, -1, 0, -1], [-1, -1, -1, 6]]


def test_dispatch_ids_sends_each_pair_to_exactly_one_rank():
    rng = np.random.default_rng(3)
    for world in (1, 2, 4, 8):
        chosen = torch.from_numpy(np.stack([rng.permutation(256)[:8] for _ in range(4)]).astype(np.int32))
        plan = dispatch_ids(chosen, 256, world)
        assert plan.shape == (world, 32) and plan.dtype == torch.int32
        held = plan >= 0
        assert torch.equal(held.sum(dim=0), torch.ones(32, dtype=torch.int64))
        per = 256 // world
        owner = held.to(torch.int32).argmax(dim=0)
        rebuilt = plan.max(dim=0).values + owner.to(torch.int32) * per
        assert torch.equal(rebuilt, chosen.reshape(-1))


def _expert_rows(oracle, cfg, tensors, il, x_pairs, ids, first):
    """Host stand-in for the grouped expert FFN: zero rows where ids < 0."""
    ef, hidden = cfg.expert_ffn, cfg.hidden
    p = f"blk.{il}."
    raw = {n: tensors[p + f"ffn_{n}_exps.weight"] for n in ("gate", "up", "down")}
    data = {n: t.data.numpy().reshape(t.rows, -1) for n, t in raw.items()}
    y = np.zeros((len(ids), hidden), dtype=np.float32)
    for i, local in enumerate(ids):
        if local < 0:
            continue
        e = int(local) + first
        mid = oracle.matmul([(data["gate"], raw["gate"].ggml_type, e * ef, ef),
                             (data["up"], raw["up"].ggml_type, e * ef, ef)], hidden, x_pairs[i])[0]
        gate, up = mid[:ef], mid[ef:]
        act = (gate / (1.0 + np.exp(-gate.astype(np.float64)))).astype(np.float32) * up
        y[i] = oracle.matmul([(data["down"], raw["down"].ggml_type, e * hidden, hidden)], ef, act)[0]
    return y


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import binding
    oracle = binding.Oracle()
    cfg = synth.ModelConfig(**G.MOE)
    tensors = synth.build_model(cfg, G.MOE_SEED)
    tokens, k = 3, cfg.experts_used
    first, count = expert_range(cfg.experts, rank, world)
    # Every rank brings its own tokens and its own routing.
    x = G.normal(400 + rank, tokens, cfg.hidden)
    chosen = np.stack([oracle.route(G.normal(500 + 10 * rank + t, cfg.experts), k)[0] for t in range(tokens)])

    def run_pairs(x_pairs, ids):
        return torch.from_numpy(_expert_rows(oracle, cfg, tensors, 0, x_pairs.numpy(), ids.numpy(), first))

    got = sharded_expert_rows(torch.from_numpy(x), torch.from_numpy(chosen.astype(np.int32)), cfg.experts, world,
                              run_pairs)
    # The same pairs with every expert at hand.
    want = _expert_rows(oracle, cfg, tensors, 0, np.repeat(x, k, axis=0), chosen.reshape(-1), 0)
    ok = np.array_equal(got.numpy().reshape(tokens * k, cfg.hidden), want) and float(np.abs(want).sum()) > 0
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


def test_token_sharded_exchange_matches_all_experts_local():
    """Two gloo ranks, each holding half of the experts and bringing its own three tokens: rows
    travel to the owning rank and back; the result equals running every pair locally, bit for bit."""
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=10) == 1
