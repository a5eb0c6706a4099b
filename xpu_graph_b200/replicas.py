"""Batch sharding for independent replicas (one process per GPU, no data-path collective).

The hot path has no cross-sample reduction, so multi-GPU inference is N replicas that each own a
contiguous slice of the global batch. These helpers are pure host logic (tested with gloo ranks on CPU).
"""
from __future__ import annotations

from typing import List, Tuple


def shard_batch(global_batch: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Half-open sample range [lo, hi) owned by `rank`; earlier ranks take the remainder samples."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    if global_batch < 0:
        raise ValueError("negative batch")
    base, rem = divmod(global_batch, world_size)
    lo = rank * base + min(rank, rem)
    hi = lo + base + (1 if rank < rem else 0)
    return lo, hi


def all_shards(global_batch: int, world_size: int) -> List[Tuple[int, int]]:
    return [shard_batch(global_batch, world_size, r) for r in range(world_size)]


def aggregate_throughput(samples_per_rank: List[int], seconds_per_rank: List[float]) -> float:
    """Whole-job samples/s: all samples divided by the slowest rank's time (ranks run concurrently)."""
    if not samples_per_rank or len(samples_per_rank) != len(seconds_per_rank):
        raise ValueError("mismatched inputs")
    slowest = max(seconds_per_rank)
    if slowest <= 0:
        raise ValueError("non-positive time")
    return sum(samples_per_rank) / slowest
