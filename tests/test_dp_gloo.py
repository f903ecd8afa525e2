"""Data-parallel host logic with two CPU processes over gloo (no GPU needed)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from asrq_b200 import dp


def test_shard_range_partitions_exactly():
    for n in (0, 1, 7, 32, 33, 6000):
        for world in (1, 2, 3, 8):
            spans = [dp.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    with pytest.raises(ValueError):
        dp.shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    r, lr, w = dp.init("gloo")
    assert (r, lr, w) == (rank, rank, world)
    # every rank takes its slice of a 33-utterance batch; slices tile the batch, no data exchange
    b, e = dp.shard_range(33, r, w)
    x = torch.arange(33 * 4, dtype=torch.float32).reshape(33, 4)[b:e]
    local = float(x.sum())
    dp.barrier()
    total = dp.sum_over_ranks(local)
    slowest = dp.max_over_ranks(10.0 + rank)      # the "device time" each rank measured
    units = dp.sum_over_ranks(e - b)
    out[rank] = (total, slowest, units)
    dp.finalize()


def test_two_ranks_gloo():
    world = 2
    port = _free_port()
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, port, out), nprocs=world, join=True)
    expect = float(torch.arange(33 * 4, dtype=torch.float32).sum())
    for r in range(world):
        total, slowest, units = out[r]
        assert total == expect and slowest == 11.0 and units == 33
