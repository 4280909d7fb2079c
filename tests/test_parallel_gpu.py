"""Multi-GPU path on real GPUs: B and C sharded by columns over the ranks, optional NCCL all-gather
that assembles a replicated C.  Skipped with fewer than two GPUs."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from oracle import spmm_oracle, svc_oracle
        from sspmm_b200 import parallel, synthetic
        a, rhs = synthetic.config1()
        V, N = 16, rhs.shape[1]
        r = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), V)
        vals = svc_oracle.pack_values(a.M, V, a.row_ptr, a.col_idx, a.values, r)
        dev = torch.device("cuda", rank)
        ptr = torch.tensor(r.vec_row_ptr, dtype=torch.int32, device=dev)
        col = torch.tensor(r.vec_colInd_list, dtype=torch.int32, device=dev)
        val = torch.from_numpy(vals).to(dev)
        n0, n1 = parallel.shard_bounds(N, world)[rank]
        b_local = torch.from_numpy(np.ascontiguousarray(rhs[:, n0:n1])).to(dev)
        c = parallel.sharded_sspmm(ptr, col, val, b_local, V, N, replicate=True, out_dtype=torch.float16)
        torch.cuda.synchronize()
        ref = spmm_oracle.sspmm_host(V, r.vec_row_ptr, r.vec_colInd_list, vals, rhs, threads=4)
        got = c.float().cpu().numpy()
        assert got.shape == ref.shape
        rms = np.sqrt(np.mean((got - ref) ** 2)) / np.sqrt(np.mean(ref ** 2))
        assert rms < 2e-3, rms
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_sharded_spmm_with_allgather_two_gpus(lib):
    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)
