"""Batch sharding for independent replicas (one process per GPU, no data-path collective).

The hot path has no cross-sample reduction, so multi-GPU inference is N replicas that each own a
contiguous slice of the global batch. These helpers are pure host logic (tested with gloo ranks on CPU).
"""
from __future__ import annotations

import os
from typing import List, Optional, Set, Tuple


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


# ---- host placement of a replica ---------------------------------------------------------------------------------
def _parse_cpulist(text: str) -> Set[int]:
    cpus: Set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        if "-" in part:
            a, b = part.split("-")
            cpus.update(range(int(a), int(b) + 1))
        else:
            cpus.add(int(part))
    return cpus


def numa_cpus_of_pci_device(pci_bus_id: str, sysfs: str = "/sys") -> Optional[Set[int]]:
    """CPUs of the NUMA node that the PCI device (domain:bus:device.function) hangs off, or None when the
    platform does not say (single node, virtualised, files missing)."""
    bdf = pci_bus_id.lower()
    if bdf.count(":") == 1:
        bdf = "0000:" + bdf
    try:
        with open(os.path.join(sysfs, "bus/pci/devices", bdf, "numa_node")) as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(os.path.join(sysfs, "devices/system/node", f"node{node}", "cpulist")) as f:
            return _parse_cpulist(f.read()) or None
    except (OSError, ValueError):
        return None


def bind_to_device_numa_node(pci_bus_id: str, sysfs: str = "/sys") -> Optional[Set[int]]:
    """Restrict this process to the CPUs next to its GPU, so that the pinned host buffers of the replica (first touch)
    and its copy threads sit on the memory controller the GPU's PCIe root is attached to. With eight replicas on a
    two-socket host this keeps half of the host <-> device traffic off the inter-socket link. Returns the previous
    affinity (to restore it), or None when nothing was changed."""
    if not hasattr(os, "sched_setaffinity"):
        return None
    want = numa_cpus_of_pci_device(pci_bus_id, sysfs)
    if not want:
        return None
    before = set(os.sched_getaffinity(0))
    allowed = want & before
    if not allowed or allowed == before:
        return None
    os.sched_setaffinity(0, allowed)
    return before
