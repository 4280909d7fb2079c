"""Row-reordering extension.  Parity with the reference is unpinned (its reorder sources are not in
the reference checkout); the CUDA kernel is pinned to the CPU restatement of OUR algorithm and checked
through invariants: valid permutation, fewer vectors on inputs with shared row patterns, and an SpMM
result that equals the un-reordered one up to the permutation."""
import numpy as np
import pytest
import torch

from oracle import reorder_oracle, svc_oracle
from sspmm_b200 import ops, reorder, synthetic

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def templated_matrix(M, K, templates, per_row, noise, seed):
    """Rows are noisy copies of a few column patterns, in shuffled order."""
    rng = np.random.default_rng(seed)
    pats = [rng.permutation(K)[:per_row] for _ in range(templates)]
    rows = []
    for r in range(M):
        base = pats[rng.integers(templates)]
        keep = base[rng.random(per_row) > noise]
        extra = rng.integers(0, K, rng.integers(0, 3))
        rows.append(np.unique(np.concatenate([keep, extra])))
    ptr = np.zeros(M + 1, dtype=np.int32)
    np.cumsum([len(r) for r in rows], out=ptr[1:])
    col = np.concatenate(rows).astype(np.int32)
    vals = rng.uniform(-1, 1, col.size).astype(np.float16)
    return synthetic.CSR(M, K, ptr, col, vals)


def gpu_perm(a, V):
    p = reorder.row_permutation(torch.from_numpy(a.row_ptr).to(DEV), torch.from_numpy(a.col_idx).to(DEV), a.M, a.K, V)
    torch.cuda.synchronize()
    return p


@pytest.mark.parametrize("V", [8, 16])
@pytest.mark.parametrize("case", ["random_small_k", "random_hashed_k", "templated", "ragged"])
def test_permutation_matches_cpu_restatement(lib, V, case):
    if case == "random_small_k":
        a, _ = synthetic.config1()
    elif case == "random_hashed_k":
        a = synthetic.power_law(4096, np.random.default_rng(31))
        a = synthetic.CSR(700, a.K, (a.row_ptr[:701] - a.row_ptr[0]).astype(np.int32), a.col_idx[: a.row_ptr[700]], a.values[: a.row_ptr[700]])
    elif case == "templated":
        a = templated_matrix(600, 1024, 12, 40, 0.1, 5)
    else:
        a = templated_matrix(37, 300, 3, 20, 0.2, 6)
    perm = gpu_perm(a, V).cpu().numpy()
    assert sorted(perm.tolist()) == list(range(a.M))
    assert np.array_equal(perm, reorder_oracle.row_permutation(a.M, a.K, V, a.row_ptr, a.col_idx))
    # windows of 256 rows stay windows
    for w0 in range(0, a.M, 256):
        blk = perm[w0: w0 + 256]
        assert blk.min() >= w0 and blk.max() < min(a.M, w0 + 256)


def test_reordering_reduces_vectors_and_keeps_the_product(lib):
    from oracle import spmm_oracle
    V = 8
    a = templated_matrix(1024, 2048, 24, 48, 0.05, 11)
    d_ptr, d_col, d_val = (torch.from_numpy(x).to(DEV) for x in (a.row_ptr, a.col_idx, a.values))
    vp0, vc0, vv0, _ = ops.svc(d_ptr, d_col, d_val, a.M, a.K, V)
    perm = reorder.row_permutation(d_ptr, d_col, a.M, a.K, V)
    p2, c2, v2 = reorder.permute_rows(d_ptr, d_col, d_val, perm)
    # device-side permutation equals the CPU one
    e_ptr, e_col, e_val = reorder_oracle.permute_rows(a.M, a.row_ptr, a.col_idx, a.values, perm.cpu().numpy())
    assert np.array_equal(p2.cpu().numpy(), e_ptr) and np.array_equal(c2.cpu().numpy(), e_col)
    vp1, vc1, vv1, _ = ops.svc(p2, c2, v2, a.M, a.K, V)
    nvec0, nvec1 = vc0.numel(), vc1.numel()
    assert nvec1 < 0.6 * nvec0, (nvec0, nvec1)          # shared patterns are found
    # and bit-exact SVC of the permuted matrix against the oracle
    pa = synthetic.CSR(a.M, a.K, e_ptr, e_col.astype(np.int32), e_val)
    r = svc_oracle.cvse(pa.M, pa.K, pa.nnz, pa.row_lists(), V)
    assert vc1.cpu().tolist() == r.vec_colInd_list
    rhs = torch.randn(a.K, 128, device=DEV, dtype=torch.float16)
    c_orig = ops.sspmm(vp0, vc0, vv0, rhs, V, out_dtype=torch.float32)
    c_perm = ops.sspmm(vp1, vc1, vv1, rhs, V, out_dtype=torch.float32)
    torch.cuda.synchronize()
    diff = (c_perm[: a.M] - c_orig[: a.M][perm.long()]).abs().max().item()
    assert diff <= 1e-3 * c_orig.abs().max().item()


def test_unstructured_pruned_weights_gain_a_little(lib):
    """On magnitude-pruned random weights there is little structure to find; the count must not grow much."""
    a, _ = synthetic.ffn(0, 3)
    V = 16
    d_ptr, d_col, d_val = (torch.from_numpy(x).to(DEV) for x in (a.row_ptr, a.col_idx, a.values))
    _, vc0, _, _ = ops.svc(d_ptr, d_col, d_val, a.M, a.K, V)
    perm = reorder.row_permutation(d_ptr, d_col, a.M, a.K, V)
    p2, c2, v2 = reorder.permute_rows(d_ptr, d_col, d_val, perm)
    _, vc1, _, _ = ops.svc(p2, c2, v2, a.M, a.K, V)
    assert vc1.numel() <= 1.01 * vc0.numel()
