"""Partitioning of one attention call over the GPUs of a node.

Attention is independent across (batch, KV-head group) units: a unit needs q/o/dO/dq of the G
query heads of the group, k/v/dk/dv of its one KV head and the G sink logits, and produces all
of its outputs -- including dSinks of its heads when every batch element of a group stays on one
rank -- without talking to any other unit.  So the path shards with no collective: ranks take
whole KV-head groups (all batches) while there are at least as many groups as ranks, and split
the batch as well only beyond that.  Results are bitwise those of the single-GPU run.

The reference has no such code (its launcher replicates the whole model per process,
``configs/zero3.yaml:18-19``); this module is the host-side logic the multi-GPU benchmark and
tests use.
"""
from __future__ import annotations

from typing import List, Tuple


def partition_units(B: int, Hkv: int, world: int) -> List[List[Tuple[int, int]]]:
    """(batch, kv_group) units of each rank.  Groups first, batch second; sizes differ by <= 1 group."""
    if world <= 0:
        raise ValueError("world must be positive")
    ranks: List[List[Tuple[int, int]]] = [[] for _ in range(world)]
    if world <= Hkv:
        base, extra = divmod(Hkv, world)
        g0 = 0
        for r in range(world):
            n = base + (1 if r < extra else 0)
            ranks[r] = [(b, g) for g in range(g0, g0 + n) for b in range(B)]
            g0 += n
    else:  # more ranks than groups: deal (group, batch) pairs round-robin, group-major
        units = [(b, g) for g in range(Hkv) for b in range(B)]
        for idx, u in enumerate(units):
            ranks[idx % world].append(u)
    return ranks


def group_range(Hkv: int, rank: int, world: int) -> Tuple[int, int]:
    """[g0, g1) of the KV-head groups a rank owns when world <= Hkv."""
    if world > Hkv:
        raise ValueError("group_range needs world <= Hkv")
    base, extra = divmod(Hkv, world)
    g0 = rank * base + min(rank, extra)
    return g0, g0 + base + (1 if rank < extra else 0)


def shard_by_group(q, k, v, do, sinks, rank: int, world: int):
    """Views of one rank's share: q (B,Hq,S,d), k/v (B,Hkv,S,d), do (B,S,Hq,d), sinks (Hq,)."""
    Hkv = k.shape[1]
    G = q.shape[1] // Hkv
    g0, g1 = group_range(Hkv, rank, world)
    return (q[:, g0 * G:g1 * G], k[:, g0:g1], v[:, g0:g1], do[:, :, g0 * G:g1 * G], sinks[g0 * G:g1 * G]), (g0, g1)
