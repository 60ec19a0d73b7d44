"""The N>1 host path on CPU: world_size-2 gloo process group, image sharding, max-over-ranks timing
and the gather of per-rank results in image order."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from msnhnet_b200 import sharding


def test_shard_range_partitions_exactly():
    for n in (0, 1, 7, 8, 64, 257):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def test_weak_job_ids_are_disjoint():
    spans = [sharding.weak_job(8, r, 4) for r in range(4)]
    assert spans == [(0, 8), (8, 16), (16, 24), (24, 32)]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = sharding.shard_range(5, rank, world)
    local = [f"img{i}" for i in range(lo, hi)]
    everything = sharding.gather_in_image_order(local, lo, dist)
    slowest = sharding.reduce_max(10.0 + rank, dist)
    total = sharding.reduce_sum(float(hi - lo), dist)
    q.put((rank, everything, slowest, total))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_over_gloo():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, everything, slowest, total in got:
        assert everything == [f"img{i}" for i in range(5)]
        assert slowest == 11.0 and total == 5.0
