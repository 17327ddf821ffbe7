"""Multi-rank host logic on CPU: two gloo ranks shard a batch, run the (CPU oracle) forward on their
slices, gather, and agree with the single-rank result; timing and counter reductions behave."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from nncase_b200 import sharding


def test_shard_range_partitions_exactly():
    for total in (0, 1, 7, 512, 513):
        for world in (1, 2, 3, 8):
            seen = []
            for r in range(world):
                s, c = sharding.shard_range(total, world, r)
                seen += list(range(s, s + c))
            assert seen == list(range(total))
    with pytest.raises(ValueError):
        sharding.shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        start, count = sharding.shard_range(total, world, rank)
        x = torch.arange(total, dtype=torch.float32).reshape(total, 1).repeat(1, 3)
        local = x[start:start + count] * 2.0  # stand-in for "run the program on my images"
        counts = [sharding.shard_range(total, world, r)[1] for r in range(world)]
        full = sharding.gather_outputs(local, counts)
        t_max = sharding.max_over_ranks([1.0 + rank, 5.0 - rank])
        n_sum = sharding.sum_over_ranks([10 + rank])
        dist.barrier()
        if rank == 0:
            q.put((full.numpy(), t_max, n_sum))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_gather_and_reduce():
    world, total = 2, 7
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, total, q)) for r in range(world)]
    for p in procs:
        p.start()
    full, t_max, n_sum = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    want = (np.arange(total, dtype=np.float32).reshape(total, 1).repeat(3, 1)) * 2.0
    assert np.array_equal(full, want)
    assert t_max == [2.0, 5.0] and n_sum == [21]


def test_single_process_helpers_are_identity():
    assert sharding.max_over_ranks([3.0]) == [3.0]
    assert sharding.sum_over_ranks([4]) == [4]
