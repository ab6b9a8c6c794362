"""Multi-GPU partitioning of the decode path (one process per GPU).

The attention path shards two ways with no collective inside it: by sequence (each rank owns whole
sequences and their pages) and by KV head (each rank owns hkv/world KV heads and the matching query
heads of every sequence; the per-head outputs are all-gathered before the output projection).
This module holds the host-side logic: who owns what, and the cross-rank reductions the benchmark
needs (max of times, sum of work).  It runs on any `torch.distributed` backend, so it is testable
with gloo on CPU.
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_sequences(lens: Sequence[int], world: int) -> List[List[int]]:
    """Assigns sequences to ranks so that KV bytes (proportional to length), not sequence counts,
    are balanced: longest first onto the least-loaded rank.  Returns, per rank, the sorted indices
    it owns.  Deterministic; every rank computes the same plan."""
    if world <= 0:
        raise ValueError("world must be positive")
    order = sorted(range(len(lens)), key=lambda i: (-int(lens[i]), i))
    loads = [0] * world
    owned: List[List[int]] = [[] for _ in range(world)]
    for i in order:
        r = min(range(world), key=lambda j: (loads[j], j))
        owned[r].append(i)
        loads[r] += int(lens[i])
    return [sorted(o) for o in owned]


def shard_kv_heads(hq: int, hkv: int, world: int, rank: int) -> Tuple[range, range]:
    """KV heads and query heads owned by `rank` when heads are sharded: hkv must divide evenly.
    Query head h reads KV head h // (hq // hkv), so a rank's query heads are contiguous."""
    if hkv % world != 0 or hq % hkv != 0:
        raise ValueError(f"cannot shard {hkv} KV heads over {world} ranks")
    per = hkv // world
    group = hq // hkv
    kv = range(rank * per, (rank + 1) * per)
    return kv, range(kv.start * group, kv.stop * group)


def _device_for_backend() -> torch.device:
    if dist.is_initialized() and dist.get_backend() == "nccl":
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def max_over_ranks(x: float) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return float(x)
    t = torch.tensor([x], dtype=torch.float64, device=_device_for_backend())
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float) -> float:
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return float(x)
    t = torch.tensor([x], dtype=torch.float64, device=_device_for_backend())
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def all_gather_heads(local: torch.Tensor) -> torch.Tensor:
    """All-gather of per-head attention outputs when KV heads are sharded: local (batch, hq/world, d)
    -> (batch, hq, d), ranks in head order.  The only collective of the decode path."""
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous())
    return torch.cat(parts, dim=1)


def throughput(total_work: float, seconds_local: float) -> float:
    """Whole-job rate: work summed over ranks / the slowest rank's time."""
    return sum_over_ranks(total_work) / max_over_ranks(seconds_local)
