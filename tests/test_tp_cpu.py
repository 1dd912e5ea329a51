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
