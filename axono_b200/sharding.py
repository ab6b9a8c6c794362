"""Multi-GPU partitioning of the decode path (one process per GPU).

The attention path shards two ways with no collective inside it: by sequence (each rank owns whole
sequences and their pages) and by KV head (each rank owns hkv/world KV heads and the matching query
heads of every sequence; the per-head outputs are all-gathered before the output projection).
This module holds the host-side logic: who owns what, and the cross-rank reductions the benchmark
needs (max of times, sum of work).  It runs on any `torch.distributed` backend, so it is testable
with gloo on CPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


from .partition import shard_kv_heads, shard_sequences  # noqa: E402,F401 - the plans themselves need no framework


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
