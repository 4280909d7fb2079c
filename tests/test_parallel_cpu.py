"""CPU tests of the multi-GPU host logic: shard bounds and the all-gather that
assembles a replicated C, on two gloo ranks."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sspmm_b200 import parallel


def test_shard_bounds_cover_and_align():
    for N in (8, 64, 200, 3136, 25088, 25096):
        for world in (1, 2, 3, 4, 8):
            b = parallel.shard_bounds(N, world)
            assert b[0][0] == 0 and b[-1][1] == N
            for (s0, e0), (s1, e1) in zip(b, b[1:]):
                assert e0 == s1 and s1 % parallel.COLUMN_QUANTUM == 0
            widths = [e - s for s, e in b]
            assert max(widths) - min(widths) <= parallel.COLUMN_QUANTUM
    assert parallel.shard_bounds(25088, 8) == [(i * 3136, (i + 1) * 3136) for i in range(8)]


def test_sweep_distribution():
    ids = list(range(20))
    parts = [parallel.shard_matrices(ids, r, 8) for r in range(8)]
    assert sorted(sum(parts, [])) == ids
    assert parts[3] == [3, 11, 19]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, N, rows):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(rows * N, dtype=torch.float32).reshape(rows, N).to(torch.float16)
        s, e = parallel.shard_bounds(N, world)[rank]
        got = parallel.gather_columns(full[:, s:e].contiguous(), N)
        assert torch.equal(got, full)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("N", [64, 200])
def test_gather_columns_two_ranks(N):
    mp.spawn(_worker, args=(2, _free_port(), N, 5), nprocs=2, join=True)
