"""GPU parity tests of sparse vector compression: the CUDA path, called through
the C ABI, against the golden vectors of the unmodified reference module and
against the CPU oracle on seeded inputs.  Integer outputs must be bit-exact."""
import numpy as np
import pytest
import torch

from oracle import svc_oracle
from sspmm_b200 import ops, synthetic
from tests.golden_cases import golden_cases, load_golden

pytestmark = pytest.mark.gpu

CASES = golden_cases()
GOLD = load_golden()


def run_gpu(a, V, with_values=True):
    dev = torch.device("cuda:0")
    ptr = torch.from_numpy(a.row_ptr).to(dev)
    col = torch.from_numpy(a.col_idx).to(dev)
    val = torch.from_numpy(a.values).to(dev) if with_values else None
    vec_ptr, vec_col, vec_val, replayed = ops.svc(ptr, col, val, a.M, a.K, V)
    torch.cuda.synchronize()
    return (vec_ptr.cpu().numpy(), vec_col.cpu().numpy(), None if vec_val is None else vec_val.cpu().numpy(), replayed)


def check_against_oracle(a, V):
    r = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), V)
    ptr, col, val, _ = run_gpu(a, V)
    assert np.array_equal(ptr, np.asarray(r.vec_row_ptr, dtype=np.int32))
    assert np.array_equal(col, np.asarray(r.vec_colInd_list, dtype=np.int32))
    exp = svc_oracle.pack_values(a.M, V, a.row_ptr, a.col_idx, a.values, r)
    assert np.array_equal(val.view(np.uint16), exp.view(np.uint16))
    return r


@pytest.mark.parametrize("name", sorted(CASES))
def test_svc_matches_reference_golden(lib, name):
    a, V = CASES[name]
    ptr, col, val, replayed = run_gpu(a, V)
    assert np.array_equal(ptr, GOLD[name + "/vec_row_ptr"])
    assert np.array_equal(col, GOLD[name + "/vec_colInd_list"])
    # value vectors: densifying the compressed form gives back A
    dense = svc_oracle.densify(ptr.size - 1, V, a.K, ptr.tolist(), col.tolist(), val)
    assert np.array_equal(dense[: a.M].view(np.uint16), a.dense().view(np.uint16))
    assert not dense[a.M:].any()
    if name.startswith("powerlaw"):
        assert replayed > 0          # the hash-order replay really ran


@pytest.mark.parametrize("name", sorted(CASES))
def test_python_entry_point_matches_reference_golden(lib, name):
    from sspmm_b200 import sparse_matrix_format as smf
    a, V = CASES[name]
    c = smf.CVSE(a.M, a.K, a.nnz, a.row_lists(), V)
    assert c.vec_row_ptr == GOLD[name + "/vec_row_ptr"].tolist()
    assert c.vec_colInd_list == GOLD[name + "/vec_colInd_list"].tolist()
    assert c.tile_num == GOLD[name + "/tile_num"].tolist()
    assert [c.return_CSR_storage(), c.return_CVSE_storage(), c.return_TCF_storage(),
            c.return_SRBCSR_storage()] == GOLD[name + "/storage"].tolist()
    assert c.num_vec == len(c.vec_colInd_list) and len(c.vec_colInd_list_array) == c.num_vec_row


@pytest.mark.parametrize("V", [8, 16])
@pytest.mark.parametrize("shape_id,sparsity_id", [(0, 0), (0, 5), (1, 2), (1, 4)])
def test_svc_ffn_configs(lib, V, shape_id, sparsity_id):
    a, _ = synthetic.ffn(shape_id, sparsity_id)
    check_against_oracle(a, V)


def test_svc_power_law_with_giant_rows(lib):
    a = synthetic.power_law(16384, np.random.default_rng(123))
    r = check_against_oracle(a, 8)
    assert max(len(l) for l in r.vec_colInd_list_array) > 1229     # a table of 8192 slots or more was replayed


@pytest.mark.parametrize("V", [8, 16])
def test_svc_edge_cases(lib, V):
    rng = np.random.default_rng(V)
    cases = []
    # empty matrix rows everywhere
    cases.append(synthetic.CSR(40, 100, np.zeros(41, dtype=np.int32), np.zeros(0, dtype=np.int32), np.zeros(0, dtype=np.float16)))
    # single row, single entry, last column
    cases.append(synthetic.CSR(1, 70000, np.array([0, 1], dtype=np.int32), np.array([69999], dtype=np.int32), np.array([1.5], dtype=np.float16)))
    # M = 0
    cases.append(synthetic.CSR(0, 10, np.zeros(1, dtype=np.int32), np.zeros(0, dtype=np.int32), np.zeros(0, dtype=np.float16)))
    # dense rows (every column), M not a multiple of V
    M, K = 19, 96
    ptr = (np.arange(M + 1) * K).astype(np.int32)
    cases.append(synthetic.CSR(M, K, ptr, np.tile(np.arange(K, dtype=np.int32), M), rng.uniform(-1, 1, M * K).astype(np.float16)))
    # exactly at the growth thresholds of the hash table: 4, 5, 18, 19, 76, 77, 306, 307 distinct keys, wide key range
    for u in (4, 5, 18, 19, 76, 77, 306, 307, 1228, 1229):
        cols = rng.permutation(200000)[:u].astype(np.int32)
        cases.append(synthetic.CSR(1, 200000, np.array([0, u], dtype=np.int32), cols, rng.uniform(-1, 1, u).astype(np.float16)))
    # colliding keys: all congruent modulo every small table length
    cols = (np.arange(30, dtype=np.int32) * 8192 + 5)
    lens = [10, 0, 8, 12] + [0] * (V - 4)
    ptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    cases.append(synthetic.CSR(V, 30 * 8192, ptr, rng.permutation(cols).astype(np.int32), rng.uniform(-1, 1, 30).astype(np.float16)))
    for a in cases:
        check_against_oracle(a, V)


def test_svc_rejects_bad_column(lib):
    a = synthetic.CSR(2, 10, np.array([0, 1, 2], dtype=np.int32), np.array([3, 10], dtype=np.int32), np.ones(2, dtype=np.float16))
    from sspmm_b200 import capi
    with pytest.raises(capi.SspmmError):
        run_gpu(a, 8)
    # the library stays usable afterwards
    ok = synthetic.CSR(2, 10, np.array([0, 1, 2], dtype=np.int32), np.array([3, 9], dtype=np.int32), np.ones(2, dtype=np.float16))
    check_against_oracle(ok, 8)


def test_all_zero_vector_count_entry_point(lib):
    from sspmm_b200 import sparse_matrix_format as smf
    a, V = CASES["config1_v8"]
    om = smf.OriginMatrix(a.M, a.K, a.row_ptr, a.col_idx)
    assert smf.return_all_zero_vec(V, a.M, a.K, om) == int(GOLD["config1_v8/all_zero_vec_cnt"][0])


def test_sorted_row_swizzle(lib):
    a = synthetic.power_law(4096, np.random.default_rng(5))
    r = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), 8)
    d = torch.tensor(r.vec_row_ptr, dtype=torch.int32, device="cuda:0")
    got = ops.sorted_row_swizzle(d).cpu().numpy()
    assert np.array_equal(got, svc_oracle.sorted_row_swizzle(r.vec_row_ptr))


@pytest.mark.parametrize("m_vec", [8192, 8193, 100_000, 262_144])
def test_sorted_row_swizzle_many_rows(lib, m_vec):
    """Around and far above the row count where the rank loop gives way to the sort: order = length descending, row id
    ascending among equal lengths (many ties: lengths are drawn from 0..40), a permutation of all rows."""
    rng = np.random.default_rng(m_vec)
    lens = rng.integers(0, 41, m_vec)
    lens[rng.integers(0, m_vec, 5)] = rng.integers(1000, 100000, 5)
    ptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    got = ops.sorted_row_swizzle(torch.from_numpy(ptr).to("cuda:0")).cpu().numpy()
    want = np.lexsort((np.arange(m_vec), -lens))
    assert np.array_equal(got, want)


def test_svc_full_size_properties(lib):
    """n = 65536 power-law matrix (largest sweep size): checked through
    size-independent properties instead of the slow CPU oracle."""
    a = synthetic.power_law(65536, np.random.default_rng(2024))
    V = 8
    ptr, col, val, _ = run_gpu(a, V)
    m_vec = a.M // V
    assert ptr[0] == 0 and np.all(np.diff(ptr) >= 0) and ptr[-1] == col.size
    # each vector row holds exactly the distinct columns of its V rows
    grp = np.repeat(np.arange(a.M) // V, np.diff(a.row_ptr)).astype(np.int64)
    key_in = np.unique(grp * a.K + a.col_idx)
    key_out = np.repeat(np.arange(m_vec, dtype=np.int64), np.diff(ptr)) * a.K + col
    assert key_out.size == key_in.size and np.array_equal(np.sort(key_out), key_in)
    # value vectors carry every original value once and zeros elsewhere
    assert np.isclose(val.astype(np.float64).sum(), a.values.astype(np.float64).sum(), atol=1e-6)
    assert np.count_nonzero(val) == np.count_nonzero(a.values)
    # spot-check a slice of vector rows against the oracle, including order
    sub = synthetic.CSR(512, a.K, (a.row_ptr[:513] - a.row_ptr[0]).astype(np.int32), a.col_idx[a.row_ptr[0]:a.row_ptr[512]], a.values[a.row_ptr[0]:a.row_ptr[512]])
    r = svc_oracle.cvse(sub.M, sub.K, sub.nnz, sub.row_lists(), V)
    assert np.array_equal(col[: ptr[64]], np.asarray(r.vec_colInd_list, dtype=np.int32))


def test_generate_cvse_file_batch_driver(lib, tmp_path):
    """The batch entry point row_merge.py calls (reference :190-250): files in, files + CSV rows out."""
    import csv
    from sspmm_b200 import sparse_matrix_format as smf
    names = ["config1_v8", "ffn_512x2048_s98_v8"]
    src, dest = tmp_path / "dlmc", tmp_path / "dlmc-v8"
    (src / "sub").mkdir(parents=True)
    listing = []
    for n in names:
        a, _ = CASES[n]
        rel = f"sub/{n}.smtx"
        svc_oracle.write_smtx(str(src / rel), a.M, a.K, a.nnz, a.row_ptr.tolist(), a.col_idx.tolist())
        listing.append(rel)
    (tmp_path / "paths.txt").write_text("\n".join(listing) + "\n")
    smf.generate_CVSE_file(str(src) + "/", str(dest) + "/", str(tmp_path / "paths.txt"), 8, csv_dir=str(tmp_path / "csv_data"))
    rows = list(csv.reader(open(tmp_path / "csv_data" / "RowMerge_V8.csv")))
    assert len(rows) == len(names)
    for i, n in enumerate(names):
        a, V = CASES[n]
        m, k, nnz, ptr, col = svc_oracle.read_smtx(str(dest / listing[i]))
        assert (m, k, nnz) == ((a.M + 7) // 8, a.K, a.nnz)
        assert ptr == GOLD[n + "/vec_row_ptr"].tolist() and col == GOLD[n + "/vec_colInd_list"].tolist()
        zero = int(GOLD[n + "/all_zero_vec_cnt"][0])
        exp = [str(i), str(a.M), str(a.K), str(a.nnz), str(svc_oracle.new_sparsity(8, a.M, a.K, a.nnz, zero)), str(zero)] + \
              [str(x) for x in GOLD[n + "/storage"].tolist()]
        assert rows[i] == exp


def test_svc_batch_equals_one_by_one(lib):
    """Several matrices of different shapes compressed in one stacked pass give exactly what separate
    calls give (and therefore what the reference gives)."""
    dev = torch.device("cuda:0")
    names = ["ragged_unsorted_v8", "powerlaw_4096_v8", "config1_v8", "ffn_512x2048_s98_v8"]
    mats = []
    for n in names:
        a, _ = CASES[n]
        mats.append((torch.from_numpy(a.row_ptr).to(dev), torch.from_numpy(a.col_idx).to(dev),
                     torch.from_numpy(a.values).to(dev), a.M, a.K))
    res, replayed = ops.svc_batch(mats, 8)
    assert replayed > 0
    for n, (p, c, v) in zip(names, res):
        a, _ = CASES[n]
        assert np.array_equal(p.cpu().numpy(), GOLD[n + "/vec_row_ptr"])
        assert np.array_equal(c.cpu().numpy(), GOLD[n + "/vec_colInd_list"])
        dense = svc_oracle.densify(p.numel() - 1, 8, a.K, p.cpu().tolist(), c.cpu().tolist(), v.cpu().numpy())
        assert np.array_equal(dense[: a.M].view(np.uint16), a.dense().view(np.uint16))


def test_reader_rows_take_the_array_path_through_the_python_entry_point(lib, tmp_path):
    """CVSE fed with the reader's row sequence (CSR arrays handed over without list conversion) equals CVSE fed
    with plain lists of lists, and both equal the oracle."""
    from sspmm_b200 import sparse_matrix_format as smf
    a = synthetic.power_law(3000, np.random.default_rng(77))
    p = str(tmp_path / "p.smtx")
    smf.write_smtx(p, a.M, a.K, a.nnz, a.row_ptr, a.col_idx)
    m = smf.sparse_matrix(p)
    fast = smf.CVSE(m.M, m.N, m.nnz, m.colInd_list_array(), 8)
    slow = smf.CVSE(a.M, a.K, a.nnz, a.row_lists(), 8)
    r = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), 8)
    assert fast.vec_row_ptr == slow.vec_row_ptr == r.vec_row_ptr
    assert fast.vec_colInd_list == slow.vec_colInd_list == r.vec_colInd_list
    assert fast.tile_num == r.tile_num and fast.vec_colInd_list_array == r.vec_colInd_list_array
    assert fast.return_TCF_storage() == r.return_TCF_storage() and fast.return_SRBCSR_storage() == r.return_SRBCSR_storage()
