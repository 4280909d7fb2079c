"""SuiteSparse side of the preprocessing stage (mirror of RowMerge/suit_sparse_matrix.py) against files written
by the unmodified reference driver on the seeded fixture tests/golden/tiny_suite.mtx (tests/golden/make_golden.py)."""
import os
import shutil

import numpy as np
import pytest

from tests.golden_cases import load_golden

GOLD = load_golden()
FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "tiny_suite.mtx")


def test_matrix_market_reader_and_csr_file_match_the_reference(lib, tmp_path):
    from sspmm_b200 import suit_sparse_matrix as ssm
    src = str(tmp_path / "tiny_suite.mtx")
    shutil.copy(FIXTURE, src)
    m = ssm.suite_matrix(src)
    assert (m.M, m.K, m.nnz) == (70, 90, 420)
    row_ptr, col = m.coo2csr(1)
    assert open(str(tmp_path / "tiny_suite_csr.mtx"), "rb").read() == bytes(GOLD["suite_tiny/csr"])
    rows = m.colInd_list_array()
    assert len(rows) == 70 and rows[0] == col[row_ptr[0]:row_ptr[1]].tolist()
    assert abs(m.sparsity() - (1.0 - 420 / 70 / 90)) < 1e-12


@pytest.mark.parametrize("V", [8, 16])
def test_oracle_reproduces_the_reference_files(tmp_path, V):
    """The CPU restatement on the same fixture: scipy's COO -> CSR, oracle compression, oracle writer."""
    from scipy.io import mmread
    from scipy.sparse import coo_matrix
    from oracle import svc_oracle
    coo = coo_matrix(mmread(FIXTURE))
    csr = coo.tocsr()
    rows = svc_oracle.col_lists(coo.shape[0], csr.indptr.tolist(), csr.indices.tolist())
    r = svc_oracle.cvse(coo.shape[0], coo.shape[1], coo.nnz, rows, V)
    out = str(tmp_path / "o.smtx")
    svc_oracle.write_smtx(out, r.num_vec_row, r.K, r.nnz, r.vec_row_ptr, r.vec_colInd_list)
    assert open(out, "rb").read() == bytes(GOLD[f"suite_tiny/cvse_v{V}"])


@pytest.mark.gpu
@pytest.mark.parametrize("V", [8, 16])
def test_batch_driver_writes_the_reference_files(lib, tmp_path, V):
    from sspmm_b200 import suit_sparse_matrix as ssm
    os.makedirs(tmp_path / "src")
    os.makedirs(tmp_path / "dst")
    shutil.copy(FIXTURE, str(tmp_path / "src" / "tiny_suite.mtx"))
    listing = str(tmp_path / "files.txt")
    with open(listing, "w") as f:
        f.write("tiny_suite.mtx\n")
    ssm.generate_suitesparse_CVSE_file(str(tmp_path / "src") + "/", str(tmp_path / "dst") + "/", listing, V)
    assert open(str(tmp_path / "dst" / "tiny_suite.smtx"), "rb").read() == bytes(GOLD[f"suite_tiny/cvse_v{V}"])
    assert open(str(tmp_path / "src" / "tiny_suite_csr.mtx"), "rb").read() == bytes(GOLD["suite_tiny/csr"])
