"""CPU tests: the oracle against the golden vectors produced by the unmodified
reference module, and the oracle's internal consistency."""
import hashlib
import os
import random
import tempfile

import numpy as np
import pytest

from oracle import spmm_oracle, svc_oracle
from sspmm_b200 import synthetic
from tests.golden_cases import golden_cases, input_digest, load_golden

CASES = golden_cases()
GOLD = load_golden()


@pytest.mark.parametrize("name", sorted(CASES))
def test_inputs_match_fixture_digest(name):
    a, _ = CASES[name]
    assert bytes(GOLD[name + "/digest"]).hex() == input_digest(a)


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("fn", [svc_oracle.cvse, svc_oracle.cvse_emulated])
def test_svc_oracle_matches_reference_output(name, fn):
    a, V = CASES[name]
    r = fn(a.M, a.K, a.nnz, a.row_lists(), V)
    assert np.array_equal(np.asarray(r.vec_row_ptr, dtype=np.int32), GOLD[name + "/vec_row_ptr"])
    assert np.array_equal(np.asarray(r.vec_colInd_list, dtype=np.int32), GOLD[name + "/vec_colInd_list"])
    assert np.array_equal(np.asarray(r.tile_num, dtype=np.int32), GOLD[name + "/tile_num"])
    storage = [r.return_CSR_storage(), r.return_CVSE_storage(), r.return_TCF_storage(), r.return_SRBCSR_storage()]
    assert storage == GOLD[name + "/storage"].tolist()
    key = name + "/all_zero_vec_cnt"
    if key in GOLD:
        zero = svc_oracle.all_zero_vec_count(V, a.M, a.K, a.row_lists())
        assert zero == int(GOLD[key][0])
        assert zero == r.num_vec_row * a.K - r.num_vec
        with tempfile.TemporaryDirectory() as d:
            p = os.path.join(d, "o.smtx")
            svc_oracle.write_smtx(p, r.num_vec_row, a.K, a.nnz, r.vec_row_ptr, r.vec_colInd_list)
            assert hashlib.sha256(open(p, "rb").read()).digest() == bytes(GOLD[name + "/cvse_out_sha256"])
            m, k, nnz, ptr, col = svc_oracle.read_smtx(p)
            assert (m, k, nnz) == (r.num_vec_row, a.K, a.nnz) and ptr == r.vec_row_ptr and col == r.vec_colInd_list


def test_hash_order_cases_are_not_trivially_sorted():
    # the fixtures must exercise the hash-order path, not only ascending lists
    a, V = CASES["powerlaw_4096_v8"]
    r = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), V)
    unsorted = sum(1 for l in r.vec_colInd_list_array if l != sorted(l))
    assert unsorted > len(r.vec_colInd_list_array) // 2


def test_set_model_matches_cpython_set():
    rnd = random.Random(3)
    for _ in range(1500):
        n = rnd.choice([0, 1, 4, 5, 18, 19, 76, 77, 306, 307, 1228, 1229, 3000])
        k = rnd.choice([8, 64, 512, 2048, 65536, 10 ** 6])
        seq = [rnd.randrange(k) for _ in range(n)]
        assert svc_oracle.set_order(seq) == list(set(seq))
        assert svc_oracle.final_table_len(len(set(seq))) >= 8


def test_set_model_chained_rebuilds():
    rnd = random.Random(4)
    for _ in range(200):
        k = rnd.choice([512, 4096, 65536])
        a, b = [], []
        for _ in range(16):
            row = rnd.sample(range(k), rnd.choice([0, 3, 16, 40, 200]))
            rnd.shuffle(row)
            a = list(set(a + row))
            b = svc_oracle.set_order(b + row)
        assert a == b


def test_pack_values_round_trip():
    a, _ = synthetic.config1()
    for V in (8, 16):
        r = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), V)
        vals = svc_oracle.pack_values(a.M, V, a.row_ptr, a.col_idx, a.values, r)
        dense = svc_oracle.densify(r.num_vec_row, V, a.K, r.vec_row_ptr, r.vec_colInd_list, vals)
        assert np.array_equal(dense[: a.M], a.dense())


def test_spmm_oracle_against_float64():
    a, rhs = synthetic.config1()
    V = 8
    r = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), V)
    vals = svc_oracle.pack_values(a.M, V, a.row_ptr, a.col_idx, a.values, r)
    out = spmm_oracle.sspmm_host(V, r.vec_row_ptr, r.vec_colInd_list, vals, rhs)
    ref64 = svc_oracle.spmm_numpy(r.num_vec_row, V, rhs.shape[1], r.vec_row_ptr, r.vec_colInd_list, vals, rhs)
    assert out.shape == ref64.shape
    assert np.max(np.abs(out - ref64)) < 1e-4
    # equals the dense product too (the packed format is lossless)
    dense = a.dense().astype(np.float64) @ rhs.astype(np.float64)
    assert np.max(np.abs(ref64[: a.M] - dense)) < 1e-9
    # threaded and row-subset variants are bit-identical to the scalar loop
    out_mt = spmm_oracle.sspmm_host(V, r.vec_row_ptr, r.vec_colInd_list, vals, rhs, threads=4)
    assert np.array_equal(out, out_mt)
    part = spmm_oracle.sspmm_host(V, r.vec_row_ptr, r.vec_colInd_list, vals, rhs, rows=(5, 9))
    assert np.array_equal(part, out[5 * V: 9 * V])


def test_sorted_row_swizzle_oracle():
    ptr = [0, 3, 3, 10, 12, 19]
    assert svc_oracle.sorted_row_swizzle(ptr).tolist() == [2, 4, 0, 3, 1]
