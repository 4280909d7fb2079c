"""Regenerates tests/golden/svc_golden.npz (and the fixture tests/golden/tiny_suite.mtx) by running the
UNMODIFIED reference modules RowMerge/sparse_matrix_format.py and RowMerge/suit_sparse_matrix.py (imported
from a reference checkout, with a stub standing in for their unused matplotlib import) on seeded synthetic
inputs.  The reference checkout is only needed to regenerate; the tests read the
committed .npz.

    python tests/golden/make_golden.py /path/to/reference
"""
import hashlib
import os
import sys
import tempfile
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from sspmm_b200 import synthetic  # noqa: E402


def golden_cases():
    """name -> (CSR, V).  Shared with the tests, which rebuild the same inputs."""
    cases = {}
    a, _ = synthetic.config1()
    cases["config1_v8"] = (a, 8)
    a, _ = synthetic.ffn(1, 5)          # 512x2048 @ 0.98
    cases["ffn_512x2048_s98_v8"] = (a, 8)
    cases["ffn_512x2048_s98_v16"] = (a, 16)
    a, _ = synthetic.ffn(0, 3)          # 2048x512 @ 0.9
    cases["ffn_2048x512_s90_v16"] = (a, 16)
    pl = synthetic.power_law(4096, np.random.default_rng(77))
    cases["powerlaw_4096_v8"] = (pl, 8)
    cases["powerlaw_4096_v16"] = (pl, 16)
    # ragged: M not a multiple of V, empty rows, unsorted rows
    rng = np.random.default_rng(9)
    M, K = 37, 3000
    lens = rng.integers(0, 40, M)
    lens[[3, 4, 5, 6, 7, 8, 9, 10]] = 0          # one vector row fully empty at V=8 (rows 8..15 partly)
    lens[16:32] = 0                              # an empty vector row at V=16
    ptr = np.zeros(M + 1, dtype=np.int32)
    np.cumsum(lens, out=ptr[1:])
    cols = np.concatenate([rng.permutation(K)[:l] for l in lens] + [np.zeros(0, dtype=np.int64)]).astype(np.int32)
    vals = rng.uniform(-1, 1, cols.size).astype(np.float16)
    rag = synthetic.CSR(M, K, ptr, cols, vals)
    cases["ragged_unsorted_v8"] = (rag, 8)
    cases["ragged_unsorted_v16"] = (rag, 16)
    return cases


def input_digest(a) -> str:
    h = hashlib.sha256()
    h.update(np.ascontiguousarray(a.row_ptr).tobytes())
    h.update(np.ascontiguousarray(a.col_idx).tobytes())
    return h.hexdigest()


def main(ref_root: str) -> None:
    for name in ("matplotlib", "matplotlib.pyplot"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.path.insert(0, os.path.join(ref_root, "RowMerge"))
    import sparse_matrix_format as ref  # the reference module, unmodified

    out = {}
    for name, (a, V) in golden_cases().items():
        rows = a.row_lists()
        c = ref.CVSE(a.M, a.K, a.nnz, rows, V)
        out[name + "/vec_row_ptr"] = np.asarray(c.vec_row_ptr, dtype=np.int32)
        out[name + "/vec_colInd_list"] = np.asarray(c.vec_colInd_list, dtype=np.int32)
        out[name + "/tile_num"] = np.asarray(c.tile_num, dtype=np.int32)
        out[name + "/storage"] = np.asarray(
            [c.return_CSR_storage(), c.return_CVSE_storage(), c.return_TCF_storage(), c.return_SRBCSR_storage()],
            dtype=np.int64)
        out[name + "/digest"] = np.frombuffer(bytes.fromhex(input_digest(a)), dtype=np.uint8)
        if a.M * a.K <= 1 << 21:
            # the reference's dense path: origin_matrix + return_all_zero_vec (needs a .smtx on disk)
            with tempfile.TemporaryDirectory() as d:
                p = os.path.join(d, "m.smtx")
                with open(p, "w") as f:
                    f.write(f"{a.M}, {a.K}, {a.nnz}\n")
                    f.write(" ".join(map(str, a.row_ptr.tolist())) + "\n")
                    f.write(" ".join(map(str, a.col_idx.tolist())))
                sm = ref.sparse_matrix(p)
                assert sm.colInd_list_array() == rows
                zero = ref.return_all_zero_vec(V, sm.M, sm.N, sm.origin_matrix())
                out[name + "/all_zero_vec_cnt"] = np.asarray([zero], dtype=np.int64)
                q = os.path.join(d, "o.smtx")
                c.CVSE_out(q)
                out[name + "/cvse_out_sha256"] = np.frombuffer(
                    hashlib.sha256(open(q, "rb").read()).digest(), dtype=np.uint8)
    # SuiteSparse side: the reference's Matrix Market driver, unmodified, on a small seeded .mtx written
    # here by scipy (coordinate format with repeated entries, so that the COO -> CSR step sums duplicates)
    import scipy.io
    import scipy.sparse
    import suit_sparse_matrix as ref_suite
    rng = np.random.default_rng(31)
    M, K, n = 70, 90, 420
    coo = scipy.sparse.coo_matrix((rng.uniform(0.5, 1.5, n), (rng.integers(0, M, n), rng.integers(0, K, n))), shape=(M, K))
    mtx = os.path.join(HERE, "tiny_suite.mtx")
    scipy.io.mmwrite(mtx, coo, comment="seeded synthetic matrix, see make_golden.py", precision=6)
    with tempfile.TemporaryDirectory() as d:
        import shutil
        os.makedirs(os.path.join(d, "src"))
        os.makedirs(os.path.join(d, "dst"))
        shutil.copy(mtx, os.path.join(d, "src", "tiny_suite.mtx"))
        listing = os.path.join(d, "files.txt")
        with open(listing, "w") as f:
            f.write("tiny_suite.mtx\n")
        for V in (8, 16):
            ref_suite.generate_suitesparse_CVSE_file(os.path.join(d, "src") + "/", os.path.join(d, "dst") + "/", listing, V)
            out[f"suite_tiny/cvse_v{V}"] = np.frombuffer(open(os.path.join(d, "dst", "tiny_suite.smtx"), "rb").read(), dtype=np.uint8)
        out["suite_tiny/csr"] = np.frombuffer(open(os.path.join(d, "src", "tiny_suite_csr.mtx"), "rb").read(), dtype=np.uint8)
    np.savez_compressed(os.path.join(HERE, "svc_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    main(sys.argv[1])
