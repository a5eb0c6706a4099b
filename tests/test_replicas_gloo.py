"""Replica sharding: pure host logic, plus a world_size-2 gloo run on CPU that mirrors how bench.py
combines ranks (barrier, max over ranks of the timed region, whole-job throughput)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from xpu_graph_b200.replicas import aggregate_throughput, all_shards, shard_batch


def test_shard_batch_covers_everything():
    for batch in (0, 1, 7, 8, 64, 65):
        for world in (1, 2, 3, 4, 8):
            shards = all_shards(batch, world)
            assert shards[0][0] == 0 and shards[-1][1] == batch
            for (a, b), (c, d) in zip(shards, shards[1:]):
                assert b == c and a <= b and c <= d
            sizes = [b - a for a, b in shards]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_batch(8, 2, 2)
    with pytest.raises(ValueError):
        shard_batch(-1, 2, 0)


def test_aggregate_throughput():
    assert aggregate_throughput([8, 8], [0.5, 1.0]) == 16.0
    with pytest.raises(ValueError):
        aggregate_throughput([8], [0.0])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = shard_batch(16, world, rank)
    x = torch.arange(16, dtype=torch.float32)[lo:hi]  # this replica's samples
    local = x.sum()  # stands in for "ran the graph on my shard"; no data-path collective
    dist.barrier()
    t = torch.tensor([0.010 * (rank + 1)], dtype=torch.float64)  # pretend per-rank time
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    gathered = [torch.zeros(()) for _ in range(world)]
    dist.all_gather(gathered, local)
    if rank == 0:
        q.put((float(t.item()), [float(g) for g in gathered], hi - lo))
    dist.destroy_process_group()


def test_two_rank_gloo_replicas():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    slowest, sums, per_rank = q.get(timeout=10)
    assert slowest == pytest.approx(0.020)
    assert sums == [sum(range(0, 8)), sum(range(8, 16))]
    assert aggregate_throughput([per_rank] * world, [0.010, 0.020]) == pytest.approx(16 / 0.020)


def test_numa_placement_reads_sysfs(tmp_path):
    """bind_to_device_numa_node against a fake sysfs tree: the GPU's node and that node's CPU list decide the
    affinity; unknown devices and node -1 change nothing."""
    import os

    from xpu_graph_b200 import replicas

    dev = tmp_path / "bus/pci/devices/0000:1b:00.0"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices/system/node/node1"
    node.mkdir(parents=True)
    have = sorted(os.sched_getaffinity(0))
    (node / "cpulist").write_text(f"{have[0]}-{have[0]},4096-4100\n")
    assert replicas.numa_cpus_of_pci_device("0000:1B:00.0", str(tmp_path)) == {have[0], 4096, 4097, 4098, 4099, 4100}
    assert replicas.numa_cpus_of_pci_device("0000:99:00.0", str(tmp_path)) is None
    before = replicas.bind_to_device_numa_node("1b:00.0", str(tmp_path))
    try:
        if len(have) > 1:
            assert before == set(have) and os.sched_getaffinity(0) == {have[0]}
        else:
            assert before is None
    finally:
        os.sched_setaffinity(0, set(have))
    (dev / "numa_node").write_text("-1\n")
    assert replicas.bind_to_device_numa_node("0000:1b:00.0", str(tmp_path)) is None
