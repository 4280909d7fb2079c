"""Randomised GPU parity: seeded CSR matrices of mixed shapes (empty rows, ragged
tails, unsorted and duplicated column ids, a few very long rows, K up to the
largest supported) go through compression and then through every SpMM kernel;
each result is compared with the CPU oracle.  Integer outputs bit-exact, products
within 1e-4 relative RMS of the fp32 oracle (the kernels accumulate in fp32 in a
different order)."""
import numpy as np
import pytest
import torch

from oracle import spmm_oracle, svc_oracle
from sspmm_b200 import ops, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def random_csr(rng):
    M = int(rng.integers(1, 300))
    K = int(rng.choice([7, 64, 500, 2048, 5000, 70000, 260000]))
    style = int(rng.integers(0, 4))
    rows = []
    for _ in range(M):
        if style == 0:
            n = int(rng.integers(0, min(K, 60)))
        elif style == 1:
            n = int(min(K, rng.zipf(1.5)))
        elif style == 2:
            n = int(rng.integers(0, min(K, 2000))) if rng.random() < 0.05 else int(rng.integers(0, min(K, 12)))
        else:
            n = int(rng.integers(0, min(K, 400)))
        if rng.random() < 0.3:
            c = rng.integers(0, K, n)                       # may repeat a column inside the row
        elif K < 5000:
            c = rng.permutation(K)[:n]
        else:
            c = np.unique(rng.integers(0, K, n))
        if rng.random() < 0.5:
            c = np.sort(c)
        rows.append(c.astype(np.int32))
    ptr = np.zeros(M + 1, dtype=np.int32)
    np.cumsum([len(r) for r in rows], out=ptr[1:])
    col = np.concatenate(rows + [np.zeros(0, dtype=np.int32)]).astype(np.int32)
    val = rng.uniform(-1, 1, col.size).astype(np.float16)
    return synthetic.CSR(M, K, ptr, col, val)


@pytest.mark.parametrize("seed", range(24))
def test_random_matrix_through_svc_and_every_spmm_kernel(lib, seed):
    rng = np.random.default_rng(1000 + seed)
    a = random_csr(rng)
    V = int(rng.choice([8, 16]))
    o = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), V)
    vp, vc, vv, _ = ops.svc(torch.from_numpy(a.row_ptr).to(DEV), torch.from_numpy(a.col_idx).to(DEV),
                            torch.from_numpy(a.values).to(DEV), a.M, a.K, V)
    assert vp.cpu().tolist() == o.vec_row_ptr
    assert vc.cpu().tolist() == o.vec_colInd_list
    if a.K > 70000:
        return
    N = int(rng.choice([8, 24, 64, 136, 256, 520]))
    rhs = rng.normal(0, 1, (a.K, N)).astype(np.float16)
    ref = spmm_oracle.sspmm_host(V, o.vec_row_ptr, o.vec_colInd_list, vv.cpu().numpy(), rhs, threads=8)
    scale = np.sqrt(np.mean(ref ** 2)) + 1e-30
    try:
        for kern in (ops.KERNEL_AUTO, ops.KERNEL_GATHER, ops.KERNEL_BLOCK, ops.KERNEL_GATHER_LSU):
            if kern == ops.KERNEL_BLOCK and o.num_vec_row * V * a.K * 2 > (1 << 28):
                continue
            ops.set_kernel(kern)
            got = ops.sspmm(vp, vc, vv, torch.from_numpy(rhs).to(DEV), V, out_dtype=torch.float32).cpu().numpy()
            assert np.isfinite(got).all()
            assert np.sqrt(np.mean((got - ref) ** 2)) / scale <= 1e-4, f"kernel {kern}"
    finally:
        ops.set_kernel(ops.KERNEL_AUTO)
    assert ops.device_status() == 0
