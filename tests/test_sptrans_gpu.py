"""PyTorch operator boundary (`sptrans.spmm.spmm` / `bspmm`): same checks as the reference's own
verification scripts end2end/sspmm_e2e/verify/spmm.py:36-41 and bspmm.py:37-44 -- a random CSR mask
of vectors, rows scheduled by length, result compared with torch.matmul / torch.bmm on the densified
operand -- plus the CPU oracle."""
import numpy as np
import pytest
import scipy.sparse
import torch

from oracle import spmm_oracle, svc_oracle
from sspmm_b200.sptrans.spmm import bspmm, spmm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def static_random_mask(m, n, sparsity, seed):
    """verify/static_mask.py:7-26: scipy random CSR mask, row_indices = argsort(row length)."""
    csr = scipy.sparse.random(m, n, density=1.0 - sparsity, format="csr", random_state=np.random.RandomState(seed))
    col = csr.indices.astype(np.int32)
    ptr = csr.indptr.astype(np.int32)
    order = np.argsort(np.diff(ptr), kind="stable").astype(np.int32)
    return col, ptr, order


@pytest.mark.parametrize("V", [8, 16])
@pytest.mark.parametrize("seq_len,feature,sparsity", [(512, 128, 0.9), (1024, 64, 0.95), (256, 256, 0.5)])
def test_spmm_matches_dense_matmul(lib, V, seq_len, feature, sparsity):
    m = seq_len // V
    col, ptr, order = static_random_mask(m, seq_len, sparsity, seed=V + seq_len)
    rng = np.random.default_rng(1)
    vals = rng.normal(0, 1, col.size * V).astype(np.float16)
    rhs = rng.normal(0, 1, (seq_len, feature)).astype(np.float16)
    out = spmm(torch.from_numpy(order).to(DEV), torch.from_numpy(ptr).to(DEV), torch.from_numpy(col).to(DEV),
               torch.from_numpy(vals).to(DEV), torch.from_numpy(rhs).to(DEV), V)
    assert out.shape == (m * V, feature) and out.dtype == torch.float16
    dense = svc_oracle.densify(m, V, seq_len, ptr.tolist(), col.tolist(), vals)
    ref = torch.matmul(torch.from_numpy(dense).to(DEV).float(), torch.from_numpy(rhs).to(DEV).float())
    assert (out.float() - ref).abs().max().item() < 0.05 * max(1.0, ref.abs().max().item() / 8)
    host = spmm_oracle.sspmm_host(V, ptr, col, vals, rhs, threads=4)
    rms = np.sqrt(np.mean((out.float().cpu().numpy() - host) ** 2)) / np.sqrt(np.mean(host ** 2))
    assert rms < 2e-3


@pytest.mark.parametrize("V", [8, 16])
@pytest.mark.parametrize("batch", [1, 3])
def test_bspmm_matches_bmm(lib, V, batch):
    seq_len, feature = 512, 128
    m = seq_len // V
    col, ptr, order = static_random_mask(m, seq_len, 0.9, seed=7 * V + batch)
    rng = np.random.default_rng(2)
    nnz = col.size * V
    vals = rng.normal(0, 1, (batch, nnz)).astype(np.float16)
    rhs = rng.normal(0, 1, (batch, seq_len, feature)).astype(np.float16)
    out = bspmm(torch.from_numpy(order).to(DEV), torch.from_numpy(ptr).to(DEV), torch.from_numpy(col).to(DEV),
                torch.from_numpy(vals).to(DEV), torch.from_numpy(rhs).to(DEV), V)
    assert out.shape == (batch, m * V, feature)
    for b in range(batch):
        host = spmm_oracle.sspmm_host(V, ptr, col, vals[b], rhs[b], threads=4)
        got = out[b].float().cpu().numpy()
        rms = np.sqrt(np.mean((got - host) ** 2)) / np.sqrt(np.mean(host ** 2))
        assert rms < 2e-3, (b, rms)


def test_bspmm_shared_weights_uses_any_kernel(lib):
    """One value array for the whole batch (pruned-weight linear layer applied to a batch)."""
    V, seq_len, feature, batch = 16, 256, 64, 4
    m = 8
    col, ptr, order = static_random_mask(m, seq_len, 0.3, seed=3)
    rng = np.random.default_rng(4)
    vals = rng.normal(0, 1, col.size * V).astype(np.float16)
    rhs = rng.normal(0, 1, (batch, seq_len, feature)).astype(np.float16)
    out = bspmm(torch.from_numpy(order).to(DEV), torch.from_numpy(ptr).to(DEV), torch.from_numpy(col).to(DEV),
                torch.from_numpy(vals).to(DEV), torch.from_numpy(rhs).to(DEV), V)
    for b in range(batch):
        host = spmm_oracle.sspmm_host(V, ptr, col, vals, rhs[b])
        got = out[b].float().cpu().numpy()
        assert np.sqrt(np.mean((got - host) ** 2)) / np.sqrt(np.mean(host ** 2)) < 2e-3
