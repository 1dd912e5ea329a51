"""Row-split tensor parallelism, host logic on the CPU: the partition of a stage's stacked rows
and the all-gather that rebuilds the full vector, with two `gloo` ranks. The row products
themselves come from the CPU oracle here; on a GPU each rank runs this backend's kernels."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from gufo_npu_b200 import synth
from gufo_npu_b200.tp import shard_rows, stage_tensors
from tests.golden import make_golden as G


def test_shard_rows_partitions_exactly():
    parts = [("qkv", 6144), ("z", 2048), ("alpha", 16), ("beta", 16)]
    for world in (1, 2, 4, 8):
        seen = []
        for rank in range(world):
            run = shard_rows(parts, rank, world)
            assert sum(c for _, _, c in run) == 8224 // world
            seen += run
        # Every row of every part exactly once, in order.
        rebuilt = {}
        for name, first, count in seen:
            assert rebuilt.get(name, 0) == first
            rebuilt[name] = first + count
        assert rebuilt == dict(parts)
    with pytest.raises(ValueError):
        shard_rows([("a", 10)], 0, 3)
    # A run that straddles three parts.
    assert shard_rows([("a", 3), ("b", 2), ("c", 7)], 0, 2) == [("a", 0, 3), ("b", 0, 2), ("c", 0, 1)]
    assert shard_rows([("a", 3), ("b", 2), ("c", 7)], 1, 2) == [("c", 1, 6)]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import binding
    oracle = binding.Oracle()
    cfg = synth.ModelConfig(**G.DENSE)
    tensors = synth.build_model(cfg, G.DENSE_SEED)
    ok = True
    for il in (0, 3):
        for stage, names in stage_tensors(cfg, il).items():
            cols = tensors[names[0]].cols
            x = G.normal(90 + il, cols)
            runs = shard_rows([(n, tensors[n].rows) for n in names], rank, world)
            parts = [(tensors[n].data.numpy().reshape(tensors[n].rows, -1), tensors[n].ggml_type, first, count)
                     for n, first, count in runs]
            local = torch.from_numpy(oracle.matmul(parts, cols, x)[0].copy())
            full = torch.empty(local.numel() * world)
            dist.all_gather_into_tensor(full, local)
            whole = [(tensors[n].data.numpy().reshape(tensors[n].rows, -1), tensors[n].ggml_type, 0, tensors[n].rows)
                     for n in names]
            want = oracle.matmul(whole, cols, x)[0]
            ok = ok and np.array_equal(full.numpy(), want)
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


def test_row_split_products_gather_to_the_full_vector():
    """Two gloo ranks: each computes its run of every stage of a DeltaNet and an attention layer;
    the gathered vector equals the unsplit product bit for bit."""
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=5) == 1


def test_split_plan_partitions_heads_and_widths():
    """collective="split": every head, KV head and FFN column belongs to some rank, slices are
    whole 256-value blocks, and models that do not divide are refused."""
    from gufo_npu_b200.tp import split_plan
    cfg = synth.ModelConfig(layers=4, hidden=2048, ffn=6144, vocab=1024, heads=8, kv_heads=2, head_dim=256,
                            rope_dim=64, linear_key_heads=16, linear_value_heads=16, linear_head_dim=128)
    for world in (1, 2, 4, 8):
        heads, kv, linear, ffn = [], set(), [], []
        for rank in range(world):
            p = split_plan(cfg, rank, world)
            heads += list(range(p["head_first"], p["head_first"] + p["heads"]))
            linear += list(range(p["linear_first"], p["linear_first"] + p["linear_heads"]))
            ffn.append((p["ffn_first"], p["ffn"]))
            mine = set(range(p["kv_first"], p["kv_first"] + p["kv_heads"]))
            kv |= mine
            # The rank's query heads all use one of its KV heads.
            group = cfg.heads // cfg.kv_heads
            assert {h // group for h in range(p["head_first"], p["head_first"] + p["heads"])} <= mine
            assert (p["heads"] * cfg.head_dim) % 256 == 0 and (p["linear_heads"] * cfg.linear_head_dim) % 256 == 0
            assert p["ffn"] % 256 == 0
        assert heads == list(range(cfg.heads)) and linear == list(range(cfg.linear_value_heads))
        assert kv == set(range(cfg.kv_heads))
        assert [f for f, _ in ffn] == [r * (cfg.ffn // world) for r in range(world)]
    with pytest.raises(ValueError):
        split_plan(cfg, 0, 3)
    with pytest.raises(ValueError):   # 16 ranks: one 128-wide DeltaNet head each is half a block
        split_plan(cfg, 0, 16)
    with pytest.raises(ValueError):
        split_plan(synth.ModelConfig(**G.MOE), 0, 2)


def _split_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import binding
    oracle = binding.Oracle()
    # A down projection split over its columns: the ranks' partial sums, added in rank order,
    # are the unsplit product to fp32 summation order.
    rows, cols = 96, 1024
    from gufo_npu_b200 import quantize as Q
    ok = True
    for t in (Q.GGML_Q4_K, Q.GGML_Q6_K):
        raw = Q.quantize(t, torch.from_numpy(G.normal(70, rows, cols) * 0.02)).numpy().reshape(rows, -1)
        x = G.normal(71, cols)
        bb = Q.row_bytes(t, 256)
        per = cols // world
        mine = np.ascontiguousarray(raw.reshape(rows, cols // 256, bb)[:, rank * per // 256:(rank + 1) * per // 256]
                                    .reshape(rows, -1))
        partial = torch.from_numpy(oracle.matmul([(mine, t, 0, rows)], per, x[rank * per:(rank + 1) * per])[0].copy())
        parts = [torch.empty_like(partial) for _ in range(world)]
        dist.all_gather(parts, partial)
        total = np.zeros(rows, dtype=np.float32)
        for p in parts:
            total += p.numpy()
        want = oracle.matmul([(raw, t, 0, rows)], cols, x)[0]
        err = float(np.linalg.norm(total - want) / np.linalg.norm(want))
        ok = ok and err < 1e-6
    flag = torch.tensor([1 if ok else 0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put(int(flag.item()))
    dist.destroy_process_group()


def test_column_split_partial_sums_add_up():
    """Two gloo ranks: block-column slices of Q4_K and Q6_K rows, partial products summed in rank
    order, against the unsplit product."""
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    procs = [ctx.Process(target=_split_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=5) == 1
