"""CPU, two gloo ranks: scene sharding and the max-over-ranks timing reduction used by bench.py."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from spira_b200 import sharding


def test_assignment_partitions_the_scenes():
    for n, g in [(16, 1), (16, 2), (16, 4), (16, 8), (5, 4), (0, 2), (3, 8)]:
        parts = [sharding.assign_scenes(n, g, r) for r in range(g)]
        assert sorted(i for p in parts for i in p) == list(range(n))
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
    with pytest.raises(ValueError):
        sharding.assign_scenes(4, 2, 2)


def test_single_process_needs_no_group():
    assert sharding.max_over_ranks(3.5) == 3.5
    assert sharding.all_ranks(3.5) == [3.5]
    assert sharding.job_throughput(500.0, [4]) == pytest.approx(8.0)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.distributed.init_process_group("gloo", rank=rank, world_size=world)
    try:
        mine = sharding.assign_scenes(7, world, rank)
        local_ms = 100.0 * (rank + 1)                      # rank 1 is the slow one
        counts = [len(sharding.assign_scenes(7, world, r)) for r in range(world)]
        out[rank] = (mine, sharding.max_over_ranks(local_ms), sharding.job_throughput(local_ms, counts), sharding.all_ranks(local_ms))
    finally:
        torch.distributed.destroy_process_group()


def test_two_ranks_gloo():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    out = manager.dict()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    assert out[0][0] == [0, 2, 4, 6] and out[1][0] == [1, 3, 5]
    for r in (0, 1):
        assert out[r][1] == 200.0                           # the slowest rank's time, on every rank
        assert out[r][2] == pytest.approx(7 / 0.2)
        assert out[r][3] == [100.0, 200.0]                  # every rank's value, in rank order
