"""CPU tests of the .smtx reader / writer in the library (host-only C++ code, no GPU)."""
import hashlib
import os

import numpy as np
import pytest

from oracle import svc_oracle
from sspmm_b200 import synthetic
from tests.golden_cases import golden_cases, load_golden

CASES = golden_cases()
GOLD = load_golden()


def test_writer_is_byte_identical_to_the_reference_writer(lib, tmp_path):
    from sspmm_b200 import sparse_matrix_format as smf
    for name in ("config1_v8", "ragged_unsorted_v16"):
        a, V = CASES[name]
        ptr, col = GOLD[name + "/vec_row_ptr"], GOLD[name + "/vec_colInd_list"]
        p = str(tmp_path / (name + ".smtx"))
        smf.write_smtx(p, ptr.size - 1, a.K, a.nnz, ptr, col)
        # sha256 of what the reference's CVSE_out wrote for the same arrays
        assert hashlib.sha256(open(p, "rb").read()).digest() == bytes(GOLD[name + "/cvse_out_sha256"])
        rows, cols, nnz, rp, ci = smf.read_smtx(p)
        assert (rows, cols, nnz) == (ptr.size - 1, a.K, a.nnz)
        assert np.array_equal(rp, ptr) and np.array_equal(ci, col)
        # and the oracle's reader agrees
        m, k, z, rp2, ci2 = svc_oracle.read_smtx(p)
        assert (m, k, z) == (rows, cols, nnz) and rp2 == rp.tolist() and ci2 == ci.tolist()


def test_reader_handles_dlmc_style_files(lib, tmp_path):
    from sspmm_b200 import sparse_matrix_format as smf
    a, _ = synthetic.ffn(1, 5)
    p = str(tmp_path / "a.smtx")
    with open(p, "w") as f:                       # DLMC files end the third line with a newline
        f.write(f"{a.M}, {a.K}, {a.nnz}\n" + " ".join(map(str, a.row_ptr.tolist())) + "\n" + " ".join(map(str, a.col_idx.tolist())) + "\n")
    m = smf.sparse_matrix(p)
    assert (m.M, m.N, m.nnz) == (a.M, a.K, a.nnz)
    assert m.rowPtr == a.row_ptr.tolist() and m.colInd == a.col_idx.tolist()
    assert m.colInd_list_array() == a.row_lists()
    assert len(m.rowInd) == a.nnz and m.rowInd[0] == 0 and m.rowInd[-1] == a.M - 1


def test_row_sequence_of_the_reader_behaves_like_the_reference_lists(lib, tmp_path):
    """colInd_list_array() returns a sequence over the CSR arrays: indexing, negative indices, slices,
    iteration and comparison give what the reference's list of lists gives."""
    from sspmm_b200 import sparse_matrix_format as smf
    a, _ = synthetic.config1()
    p = str(tmp_path / "c.smtx")
    smf.write_smtx(p, a.M, a.K, a.nnz, a.row_ptr, a.col_idx)
    rows = smf.sparse_matrix(p).colInd_list_array()
    ref = a.row_lists()
    assert len(rows) == a.M and rows[0] == ref[0] and rows[-1] == ref[-1] and rows[3:7] == ref[3:7]
    assert [r for r in rows] == ref and rows == ref
    assert isinstance(rows[5], list)
    with pytest.raises(IndexError):
        rows[a.M]


def test_empty_matrix_and_errors(lib, tmp_path):
    from sspmm_b200 import capi
    from sspmm_b200 import sparse_matrix_format as smf
    p = str(tmp_path / "e.smtx")
    smf.write_smtx(p, 3, 10, 0, [0, 0, 0, 0], [])
    assert open(p).read() == "3, 10, 0\n0 0 0 0\n"
    rows, cols, nnz, rp, ci = smf.read_smtx(p)
    assert (rows, cols, nnz) == (3, 10, 0) and rp.tolist() == [0, 0, 0, 0] and ci.size == 0
    with pytest.raises(capi.SspmmError):
        smf.read_smtx(str(tmp_path / "missing.smtx"))
    bad = tmp_path / "bad.smtx"
    bad.write_text("3, x, 0\n0 0\n")
    with pytest.raises(capi.SspmmError):
        smf.read_smtx(str(bad))
