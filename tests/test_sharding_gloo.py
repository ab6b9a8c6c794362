"""Host-side multi-rank logic on CPU: world_size-2 gloo processes."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from axono_b200 import sharding


def test_shard_sequences_balances_bytes():
    rng = np.random.default_rng(3000)
    lens = rng.integers(16384, 32769, 64).tolist()
    for world in (1, 2, 4, 8):
        plan = sharding.shard_sequences(lens, world)
        assert sorted(i for o in plan for i in o) == list(range(64))
        loads = [sum(lens[i] for i in o) for o in plan]
        assert max(loads) - min(loads) <= max(lens)
        assert max(loads) / (sum(lens) / world) < 1.02  # within 2 % of perfect balance
    assert sharding.shard_sequences([], 2) == [[], []]
    assert sharding.shard_sequences([5], 2) == [[0], []]


def test_shard_kv_heads():
    kv, qh = sharding.shard_kv_heads(16, 8, 8, 3)
    assert list(kv) == [3] and list(qh) == [6, 7]
    kv, qh = sharding.shard_kv_heads(16, 8, 2, 1)
    assert list(kv) == [4, 5, 6, 7] and list(qh) == list(range(8, 16))
    with pytest.raises(ValueError):
        sharding.shard_kv_heads(16, 8, 3, 0)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # reductions: slowest rank's time, total work
        assert sharding.max_over_ranks(1.0 + rank) == float(world)
        assert sharding.sum_over_ranks(10.0) == 10.0 * world
        assert sharding.throughput(100.0, 1.0 + rank) == 100.0 * world / world
        # sequence sharding: every rank derives the same plan and owns a disjoint part
        lens = np.random.default_rng(1).integers(100, 1000, 17).tolist()
        plan = sharding.shard_sequences(lens, world)
        mine = torch.zeros(17, dtype=torch.int64)
        mine[plan[rank]] = 1
        dist.all_reduce(mine)
        assert torch.equal(mine, torch.ones(17, dtype=torch.int64))
        # head sharding + all-gather: rank r fills its heads with their global index
        hq, hkv, d, batch = 16, 8, 4, 3
        _, qh = sharding.shard_kv_heads(hq, hkv, world, rank)
        local = torch.stack([torch.full((batch, d), float(h)) for h in qh], dim=1)
        full = sharding.all_gather_heads(local)
        assert full.shape == (batch, hq, d)
        assert torch.equal(full[0, :, 0], torch.arange(hq, dtype=torch.float32))
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
