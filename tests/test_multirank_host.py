"""Host logic of the one-process-per-GPU launch, run as two gloo ranks on the CPU: every rank derives its share
of the conversion from the plan alone, the shares tile the model exactly, and timings reduce to the slowest rank."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from libgguf_b200 import row_size
from libgguf_b200.convert import assign_shards, llama3_8b_plan, max_over_ranks, plan_shards, rank_batch


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, result_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        plan = llama3_8b_plan(n_layers=2)
        tensors = [(t.qtype, t.rows, t.cols) for t in plan]
        shards = plan_shards(tensors, chunk_bytes=64 << 20)
        mine = assign_shards(shards, [t.cols for t in plan], world)[rank]
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        if rank == 0:
            everything = sorted(s for part in gathered for s in part)
            assert everything == sorted(shards)
            loads = [sum(r * plan[t].cols for t, _, r in part) for part in gathered]
            assert max(loads) - min(loads) <= max(r * plan[t].cols for t, _, r in shards)
        slowest = max_over_ranks(1.0 + rank)
        assert slowest == float(world)
        # the views rank_batch hands to the pipeline: same rows of source and destination
        qtype, rows, n = 12, 40, 256
        src = np.arange(rows * n, dtype=np.float32).reshape(rows, n)
        dst = np.zeros(rows * row_size(qtype, n), dtype=np.uint8)
        batch = rank_batch([(qtype, src, None, dst)], world, rank, chunk_bytes=8 * n * 4)
        covered = np.zeros(rows, dtype=np.int64)
        for q, s, im, d in batch:
            assert q == qtype and im is None and np.shares_memory(s, src)
            row0 = int(s[0, 0]) // n
            assert d.ctypes.data - dst.ctypes.data == row0 * row_size(qtype, n)
            assert d.size == s.shape[0] * row_size(qtype, n)
            covered[row0:row0 + s.shape[0]] += 1
        t = torch.from_numpy(covered)
        dist.all_reduce(t)
        assert bool((t == 1).all())
        open(os.path.join(result_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_ranks_split_the_conversion_without_talking(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_assignment_is_deterministic_and_balanced():
    plan = llama3_8b_plan()
    shards = plan_shards([(t.qtype, t.rows, t.cols) for t in plan])
    widths = [t.cols for t in plan]
    for world in (1, 2, 4, 8):
        parts = assign_shards(shards, widths, world)
        assert parts == assign_shards(shards, widths, world)
        loads = [sum(r * widths[t] for t, _, r in part) for part in parts]
        assert sum(loads) == 8_029_995_008
        assert max(loads) / (sum(loads) / world) < 1.02
    assert max_over_ranks(3.5) == 3.5


def test_assignment_weighted_by_link_rates():
    """Half of the GPUs behind links of half the rate (as measured on an 8-GPU host): the shares follow the rates, so
    every process finishes at the same time, and every shard is still assigned exactly once."""
    import pytest
    plan = llama3_8b_plan()
    shards = plan_shards([(t.qtype, t.rows, t.cols) for t in plan])
    widths = [t.cols for t in plan]
    rates = [27.0, 27.0, 27.5, 27.5, 55.0, 55.0, 54.0, 55.0]
    parts = assign_shards(shards, widths, 8, rates)
    assert parts == assign_shards(shards, widths, 8, list(rates))
    assert sorted(s for part in parts for s in part) == sorted(shards)
    loads = [sum(r * widths[t] for t, _, r in part) for part in parts]
    finish = [l / r for l, r in zip(loads, rates)]
    assert max(finish) / (sum(loads) / sum(rates)) < 1.03
    assert loads[4] > 1.8 * loads[0]
    # equal rates give the unweighted answer
    assert assign_shards(shards, widths, 4, [3.0] * 4) == assign_shards(shards, widths, 4)
    with pytest.raises(ValueError):
        assign_shards(shards, widths, 2, [1.0])
    with pytest.raises(ValueError):
        assign_shards(shards, widths, 2, [1.0, 0.0])
