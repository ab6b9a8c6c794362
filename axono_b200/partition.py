"""Who owns what when the decode path is spread over the GPUs of one node - pure host logic, no
device and no framework involved, so every rank computes the same plan on its own.

The attention path shards two ways with no collective inside it: by sequence (each rank owns whole
sequences and their pages) and by KV head (each rank owns hkv/world KV heads and the matching query
heads of every sequence; the per-head outputs are gathered before the output projection)."""
from __future__ import annotations

from typing import List, Sequence, Tuple


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


def shard_tokens_by_page(length: int, page_tokens: int, world: int, rank: int) -> List[int]:
    """Context-parallel split of one sequence: its pages are dealt round-robin to the ranks; returns
    the token indices rank `rank` caches, in order."""
    out: List[int] = []
    for page, start in enumerate(range(0, length, page_tokens)):
        if page % world == rank:
            out.extend(range(start, min(length, start + page_tokens)))
    return out
