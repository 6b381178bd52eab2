"""Gradient bucket layout over the flat gradient buffer.

A bucket is a contiguous run of whole parameters of the flat buffer (a parameter never
straddles buckets; it may straddle the rank shards inside a bucket). Buckets are closed
greedily once they hold at least ``target`` elements, and each bucket's size is a multiple of
``world * shard_align`` so that every rank's shard is an aligned, equal slice. Behavioural
spec: the reference's ``compute_grad_buckets``
(exports/train_engine_0.5B/src/training_engine_tensor/nccl.py:584-651).
"""
from __future__ import annotations

from dataclasses import dataclass, field


@dataclass
class Bucket:
    index: int
    start: int                      # offset in the flat buffer
    size: int                       # elements, multiple of world
    params: list[str] = field(default_factory=list)
    param_offsets: dict[str, int] = field(default_factory=dict)   # relative to ``start``
    param_sizes: dict[str, int] = field(default_factory=dict)     # padded sizes

    def shard_size(self, world: int) -> int:
        return self.size // world

    def shard_range(self, rank: int, world: int) -> tuple[int, int]:
        n = self.size // world
        return self.start + rank * n, self.start + (rank + 1) * n


def compute_grad_buckets(entries: list[tuple[str, int, int]], world: int, target: int) -> list[Bucket]:
    """``entries``: (name, offset, padded numel) in flat-buffer order, contiguous."""
    if world <= 0:
        raise ValueError(f"world must be positive, got {world}")
    if target <= 0:
        raise ValueError(f"bucket target must be positive, got {target}")
    if not entries:
        raise ValueError("no parameters to bucket")
    buckets: list[Bucket] = []
    cur: Bucket | None = None
    expect = entries[0][1]
    for name, off, n in entries:
        if off != expect:
            raise ValueError(f"flat buffer is not contiguous at {name}: {off} != {expect}")
        if n <= 0:
            raise ValueError(f"parameter {name} has no elements")
        expect = off + n
        if cur is None:
            cur = Bucket(index=len(buckets), start=off, size=0)
        cur.params.append(name)
        cur.param_offsets[name] = off - cur.start
        cur.param_sizes[name] = n
        cur.size += n
        if cur.size >= target:
            buckets.append(cur)
            cur = None
    if cur is not None:
        buckets.append(cur)
    for b in buckets:
        if b.size % world:
            raise ValueError(f"bucket {b.index} size {b.size} is not a multiple of world {world}; "
                             f"pad parameters to a multiple of the world size")
    return buckets
