"""TEST INFRASTRUCTURE -- CPU oracle for sparse vector compression (SVC).

Only the test suite, the smoke check and the benchmark's CPU-baseline leg may
import this module; the product package never does.

It restates, function by function, the reference's Python preprocessing
(RowMerge/sparse_matrix_format.py).  Two restatements of the compression are
kept side by side:

* ``cvse`` follows the reference literally, including its use of the built-in
  ``set`` (so on the same CPython it is the reference's behaviour by
  construction);
* ``cvse_emulated`` replaces the built-in ``set`` by ``IntSetModel``, an explicit
  model of how CPython 3.12 orders a set of small non-negative ints.  The CUDA
  kernels implement that model, so the tests first check the model against the
  real ``set`` and then the kernels against either.

Parity pin: tests/golden/*.npz hold outputs of the unmodified reference module
(imported from the reference checkout by tests/golden/make_golden.py) on seeded
synthetic inputs; tests/test_oracle.py checks both restatements against them.
The reference's row-reorder stage (reorder.py / row_merge_reorder.py) is absent
from the reference checkout, so for that stage parity is unpinned.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Sequence, Tuple

import numpy as np

# --------------------------------------------------------------------------- #
# .smtx reading / writing
# --------------------------------------------------------------------------- #


def read_smtx(path: str) -> Tuple[int, int, int, List[int], List[int]]:
    """Three-line text format "M, K, nnz" / row pointers / column ids
    (RowMerge/sparse_matrix_format.py:8-25; the same layout is read back for the
    compressed form by SSpMM/sspmm_test.cpp:28-64)."""
    with open(path) as f:
        head = f.readline()
        ptr = f.readline().split()
        col = f.readline().split()
    m, k, nnz = head.split(", ")
    return int(m), int(k), int(nnz), [int(x) for x in ptr], [int(x) for x in col]


def write_smtx(path: str, m: int, k: int, nnz: int, row_ptr: Sequence[int], col: Sequence[int]) -> None:
    """Writer of the same three-line layout, no trailing newline after the column
    ids (RowMerge/sparse_matrix_format.py:152-175)."""
    with open(path, "w") as f:
        f.write(f"{m}, {k}, {nnz}\n")
        f.write(" ".join(str(int(x)) for x in row_ptr))
        f.write("\n")
        f.write(" ".join(str(int(x)) for x in col))


def col_lists(m: int, row_ptr: Sequence[int], col_idx: Sequence[int]) -> List[List[int]]:
    """Per-row lists of column ids (RowMerge/sparse_matrix_format.py:41-53)."""
    return [[int(c) for c in col_idx[row_ptr[i]:row_ptr[i + 1]]] for i in range(m)]


# --------------------------------------------------------------------------- #
# Model of CPython's ordering of a set of non-negative ints
# --------------------------------------------------------------------------- #

_MINSIZE = 8          # initial table length
_LINEAR_PROBES = 9    # slots examined after the first one before jumping
_PERTURB_SHIFT = 5


class IntSetModel:
    """Open-addressing table that reproduces the slot order of a CPython 3.12
    ``set`` holding non-negative ints smaller than 2**61-1 (for which
    ``hash(x) == x``), when elements are only ever added.

    The table length is a power of two.  An element starts at ``hash & mask``;
    if the slot is taken, up to nine following slots are tried, but only when
    the whole window lies inside the table; otherwise the start jumps to
    ``(5*i + 1 + perturb) & mask`` with ``perturb`` shifted right by five bits
    each time.  After an insertion that makes ``5*fill >= 3*mask`` the table is
    rebuilt with the smallest power-of-two length above ``4*used`` (``2*used``
    beyond 50 000 elements), re-inserting the old entries in slot order.
    Iteration walks the slots in index order."""

    __slots__ = ("mask", "table", "used")

    def __init__(self) -> None:
        self.mask = _MINSIZE - 1
        self.table = [-1] * _MINSIZE
        self.used = 0

    @staticmethod
    def _place(table: List[int], mask: int, key: int) -> int:
        """Slot that ``key`` occupies or would occupy: first empty slot, or the
        slot already holding ``key``, along the probe sequence."""
        perturb = key
        i = key & mask
        while True:
            window = _LINEAR_PROBES if i + _LINEAR_PROBES <= mask else 0
            for s in range(i, i + window + 1):
                e = table[s]
                if e == -1 or e == key:
                    return s
            perturb >>= _PERTURB_SHIFT
            i = (i * 5 + 1 + perturb) & mask

    def add(self, key: int) -> None:
        s = self._place(self.table, self.mask, key)
        if self.table[s] == key:
            return
        self.table[s] = key
        self.used += 1
        if self.used * 5 >= self.mask * 3:
            self._grow(self.used * 2 if self.used > 50000 else self.used * 4)

    def _grow(self, minused: int) -> None:
        size = _MINSIZE
        while size <= minused:
            size <<= 1
        new = [-1] * size
        for e in self.table:
            if e != -1:
                new[self._place(new, size - 1, e)] = e
        self.table = new
        self.mask = size - 1

    def ordered(self) -> List[int]:
        return [e for e in self.table if e != -1]


def set_order(seq: Iterable[int]) -> List[int]:
    """``list(set(seq))`` according to :class:`IntSetModel`."""
    s = IntSetModel()
    for x in seq:
        s.add(int(x))
    return s.ordered()


def final_table_len(distinct: int) -> int:
    """Table length after adding ``distinct`` different keys to an empty set."""
    size = _MINSIZE
    while True:
        mask = size - 1
        trig = -(-3 * mask // 5)            # smallest fill with 5*fill >= 3*mask
        if distinct < trig:
            return size
        minused = trig * 2 if trig > 50000 else trig * 4
        new = _MINSIZE
        while new <= minused:
            new <<= 1
        size = new


# --------------------------------------------------------------------------- #
# The compression itself
# --------------------------------------------------------------------------- #


class CVSEResult:
    """Field names follow the reference class (sparse_matrix_format.py:93-123)."""

    def __init__(self, M, K, nnz, vec_len, lists):
        self.M, self.K, self.nnz, self.vec_len = M, K, nnz, vec_len
        self.num_vec_row = math.ceil(M / vec_len)
        self.vec_colInd_list_array = lists
        self.vec_row_ptr = [0]
        self.tile_num = []
        for l in lists:
            self.vec_row_ptr.append(self.vec_row_ptr[-1] + len(l))
            self.tile_num.append(math.ceil(len(l) / 32))
        self.num_vec = self.vec_row_ptr[-1]
        self.vec_colInd_list = [c for l in lists for c in l]

    # storage models, sparse_matrix_format.py:124-150 (4-byte index, 2-byte value)
    def return_CSR_storage(self):
        return self.nnz * (2 + 4) + (self.M + 1) * 4

    def return_CVSE_storage(self):
        return self.num_vec * self.vec_len * 2 + (self.num_vec_row + 1) * 4 + self.num_vec * 4

    def return_TCF_storage(self):
        return self.nnz * 2 + self.nnz * 3 * 4 + (self.M + 1) * 4 + sum(self.tile_num) * 32 * 4

    def return_SRBCSR_storage(self):
        return self.num_vec * self.vec_len * 2 + (self.num_vec_row + 1) * 4 + sum(self.tile_num) * 32 * 4


def _cvse(M, K, nnz, rows, V, order_fn) -> CVSEResult:
    """sparse_matrix_format.py:100-114: vector row i covers matrix rows
    V*i .. V*i+V-1 (those below M); its column list is rebuilt V times as
    ``list(set(previous + row))``."""
    lists = []
    for i in range(math.ceil(M / V)):
        cur: List[int] = []
        for j in range(V):
            if V * i + j < M:
                cur = order_fn(cur + list(rows[V * i + j]))
        lists.append(cur)
    return CVSEResult(M, K, nnz, V, lists)


def cvse(M, K, nnz, rows, V) -> CVSEResult:
    return _cvse(M, K, nnz, rows, V, lambda seq: list(set(seq)))


def cvse_emulated(M, K, nnz, rows, V) -> CVSEResult:
    return _cvse(M, K, nnz, rows, V, set_order)


def all_zero_vec_count(V: int, M: int, K: int, rows: Sequence[Sequence[int]]) -> int:
    """Number of (vector row, column) pairs with no non-zero in any of the V rows
    (sparse_matrix_format.py:177-188, restated on column lists instead of a dense
    0/1 matrix)."""
    cnt = 0
    for i in range(math.ceil(M / V)):
        seen = set()
        for j in range(V):
            if V * i + j < M:
                seen.update(rows[V * i + j])
        cnt += K - len(seen)
    return cnt


def new_sparsity(V: int, M: int, K: int, nnz: int, zero_cnt: int) -> float:
    """sparse_matrix_format.py:218-222."""
    vec_cnt = math.ceil(M / V) * K - zero_cnt
    return 1.0 if vec_cnt == 0 else 1.0 - nnz / (vec_cnt * V)


# --------------------------------------------------------------------------- #
# Value vectors and row swizzle (pinned by their consumers only)
# --------------------------------------------------------------------------- #


def pack_values(M, V, row_ptr, col_idx, vals_f16, res: CVSEResult) -> np.ndarray:
    """values[(vec_row_ptr[i]+p)*V + v] = A[i*V+v, cols_i[p]], zero elsewhere
    (layout read by SSpMM/sspmm_test.cpp:84-90 and by
    end2end/sspmm_e2e/verify/static_mask.py:29-45).  Duplicate (row, column)
    entries keep the last one."""
    out = np.zeros(res.num_vec * V, dtype=np.float16)
    for i, cols in enumerate(res.vec_colInd_list_array):
        pos = {c: p for p, c in enumerate(cols)}
        base = res.vec_row_ptr[i]
        for v in range(V):
            r = i * V + v
            if r >= M:
                break
            for e in range(row_ptr[r], row_ptr[r + 1]):
                out[(base + pos[int(col_idx[e])]) * V + v] = vals_f16[e]
    return out


def densify(m_vec, V, K, vec_row_ptr, vec_col, values) -> np.ndarray:
    """Inverse of pack_values: dense [m_vec*V, K] fp16."""
    a = np.zeros((m_vec * V, K), dtype=np.float16)
    vals = np.asarray(values).reshape(-1, V)
    for i in range(m_vec):
        for j in range(vec_row_ptr[i], vec_row_ptr[i + 1]):
            a[i * V:(i + 1) * V, vec_col[j]] = vals[j]
    return a


def sorted_row_swizzle(vec_row_ptr: Sequence[int]) -> np.ndarray:
    """Vector rows by decreasing length (SSpMM/include/bm_test_utils.h:210-225).
    The reference uses std::sort, whose order among equal lengths is
    unspecified; this restatement breaks ties by increasing row id."""
    ptr = np.asarray(vec_row_ptr, dtype=np.int64)
    length = ptr[1:] - ptr[:-1]
    return np.argsort(-length, kind="stable").astype(np.int32)


def spmm_numpy(m_vec, V, N, vec_row_ptr, vec_col, values, rhs) -> np.ndarray:
    """float64 evaluation of the same sum, used only for error analysis of the
    fp32 oracle (not the parity target)."""
    out = np.zeros((m_vec * V, N), dtype=np.float64)
    vals = np.asarray(values, dtype=np.float64).reshape(-1, V)
    rhs = np.asarray(rhs, dtype=np.float64)
    ptr = np.asarray(vec_row_ptr)
    col = np.asarray(vec_col)
    for i in range(m_vec):
        s, e = ptr[i], ptr[i + 1]
        if e > s:
            out[i * V:(i + 1) * V] = vals[s:e].T @ rhs[col[s:e]]
    return out
