"""Python entry points of the preprocessing stage, with the compression running
on the GPU.

Same names, arguments and attributes as the reference module
RowMerge/sparse_matrix_format.py, so that its scripts (row_merge.py:16,18;
suit_sparse_matrix.py:211) run unchanged with ``import sparse_matrix_format``
resolving to this file:

* ``sparse_matrix(path)``                      reader, reference :7-39
* ``CVSE(ROW, COL, NNZ, colInd_list_array, V)`` compression, reference :93-175
* ``return_all_zero_vec(V, ROW, COL, origin)`` reference :177-188
* ``generate_CVSE_file(src, dest, paths, V)``  batch driver, reference :190-250

The compression itself is ``svc_begin``/``svc_finish`` of libsspmm_b200.so; there
is no CPU implementation here, and a missing library or GPU is an error."""
from __future__ import annotations

import csv
import functools
import itertools
import math
import os
from collections.abc import Sequence
from typing import List, Optional

import numpy as np
import torch

from . import capi, ops


def read_smtx(path):
    """(rows, cols, nnz, row_ptr int32[], col_idx int32[]) through the library's C++ parser."""
    import ctypes as C
    lib = capi.lib()
    rows, cols, nnz = C.c_int(), C.c_int(), C.c_int()
    n1, n2 = C.c_int64(), C.c_int64()
    capi.check(lib.smtx_read_header(os.fsencode(path), C.byref(rows), C.byref(cols), C.byref(nnz), C.byref(n1), C.byref(n2)))
    row_ptr = np.empty(n1.value, dtype=np.int32)
    col = np.empty(n2.value, dtype=np.int32)
    capi.check(lib.smtx_read(os.fsencode(path), row_ptr.ctypes.data, n1.value, col.ctypes.data, n2.value))
    return rows.value, cols.value, nnz.value, row_ptr, col


def write_smtx(path, rows, cols, nnz, row_ptr, col_idx):
    rp = np.ascontiguousarray(row_ptr, dtype=np.int32)
    ci = np.ascontiguousarray(col_idx, dtype=np.int32)
    capi.check(capi.lib().smtx_write(os.fsencode(path), int(rows), int(cols), int(nnz), rp.ctypes.data, rp.size,
                                     ci.ctypes.data, ci.size))


def _device() -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("sspmm_b200 needs a CUDA device: the compression runs on the GPU only")
    return torch.device("cuda", torch.cuda.current_device())


class sparse_matrix:
    """Three-line .smtx reader: "M, N, nnz" / row pointers / column ids
    (reference :8-39).  Attributes M, N, nnz, rowPtr, colInd, rowInd."""

    def __init__(self, path):
        self.M, self.N, self.nnz, self._row_ptr, self._col = read_smtx(path)

    # list attributes of the reference, built on first use
    @functools.cached_property
    def rowPtr(self):
        return self._row_ptr.tolist()

    @functools.cached_property
    def colInd(self):
        return self._col.tolist()

    @functools.cached_property
    def rowInd(self):
        return np.repeat(np.arange(self.M), np.diff(self._row_ptr[: self.M + 1])).tolist()

    def colInd_list_array(self):
        """Per-row column lists (reference :41-53) as a sequence that also carries the CSR arrays, so
        that CVSE can skip the list -> array conversion."""
        return _CsrRows(self._row_ptr[: self.M + 1], self._col)

    def origin_matrix(self):
        """The reference returns a dense M x N list of 0/1 lists (:55-67) whose only
        consumer is ``return_all_zero_vec``; here it is a light view over the CSR
        arrays that indexes like that list."""
        return OriginMatrix(self.M, self.N, self._row_ptr, self._col)

    def sparsity(self):
        return 1.0 - self.nnz / self.M / self.N


class OriginMatrix:
    def __init__(self, M, N, row_ptr, col):
        self.M, self.N, self.row_ptr, self.col = M, N, row_ptr, col

    def __len__(self):
        return self.M

    def __getitem__(self, i):
        row = [0] * self.N
        for c in self.col[self.row_ptr[i]:self.row_ptr[i + 1]]:
            row[c] = 1
        return row


class _CsrRows(Sequence):
    """Read-only sequence of per-row column lists over CSR arrays; rows are cut on access."""

    def __init__(self, row_ptr, col):
        self.csr = (row_ptr, col)

    def __len__(self):
        return len(self.csr[0]) - 1

    def __getitem__(self, i):
        p, c = self.csr
        if isinstance(i, slice):
            return [c[p[k]:p[k + 1]].tolist() for k in range(*i.indices(len(self)))]
        if i < 0:
            i += len(self)
        if not 0 <= i < len(self):
            raise IndexError(i)
        return c[p[i]:p[i + 1]].tolist()

    def __eq__(self, other):
        return len(self) == len(other) and all(a == b for a, b in zip(self, other))


def _csr_from_lists(rows: Sequence[Sequence[int]]):
    lens = np.fromiter(map(len, rows), dtype=np.int64, count=len(rows))
    row_ptr = np.zeros(len(rows) + 1, dtype=np.int64)
    np.cumsum(lens, out=row_ptr[1:])
    col = np.fromiter(itertools.chain.from_iterable(rows), dtype=np.int64, count=int(row_ptr[-1]))
    if row_ptr[-1] >= 2 ** 31 or (col.size and (col.min() < 0 or col.max() >= 2 ** 31)):
        raise ValueError("matrix does not fit 32-bit indices")
    return row_ptr.astype(np.int32), col.astype(np.int32)


class CVSE:
    """Attributes as in the reference (:96-123): M, K, nnz, vec_len, num_vec_row,
    tile_num, vec_colInd_list_array, num_vec, vec_row_ptr, vec_colInd_list."""

    def __init__(self, ROW, COL, NNZ, colInd_list_array, vec_len, values=None):
        self.M, self.K, self.nnz, self.vec_len = ROW, COL, NNZ, vec_len
        self.num_vec_row = math.ceil(ROW / vec_len)
        csr = getattr(colInd_list_array, "csr", None)
        if csr is not None and len(colInd_list_array) == ROW:
            row_ptr, col = np.ascontiguousarray(csr[0], dtype=np.int32), np.ascontiguousarray(csr[1], dtype=np.int32)
        else:
            row_ptr, col = _csr_from_lists(colInd_list_array[:ROW])
        dev = _device()
        d_ptr = torch.from_numpy(row_ptr).to(dev)
        d_col = torch.from_numpy(col).to(dev)
        d_val = None
        if values is not None:
            d_val = torch.from_numpy(np.ascontiguousarray(values, dtype=np.float16)).to(dev)
        vec_ptr, vec_col, vec_val, replayed = ops.svc(d_ptr, d_col, d_val, ROW, COL, vec_len)
        self.replayed_rows = replayed
        self.d_vec_row_ptr, self.d_vec_col, self.d_vec_values = vec_ptr, vec_col, vec_val
        self._ptr = vec_ptr.cpu().numpy()
        self._cols = vec_col.cpu().numpy()
        self.num_vec = int(self._ptr[-1])
        self.values = None if vec_val is None else vec_val.cpu().numpy()

    # The list attributes of the reference are built on first use: turning a million column ids into
    # Python ints costs more than the compression itself.
    @functools.cached_property
    def vec_row_ptr(self):
        return self._ptr.tolist()

    @functools.cached_property
    def vec_colInd_list(self):
        return self._cols.tolist()

    @functools.cached_property
    def tile_num(self):
        return (-(-np.diff(self._ptr) // 32)).tolist()

    @functools.cached_property
    def vec_colInd_list_array(self):
        l, p = self.vec_colInd_list, self.vec_row_ptr
        return [l[p[i]:p[i + 1]] for i in range(self.num_vec_row)]

    # storage models (reference :124-150): 4-byte indices, 2-byte values
    def return_CSR_storage(self):
        return self.nnz * (2 + 4) + (self.M + 1) * 4

    def return_CVSE_storage(self):
        return self.num_vec * self.vec_len * 2 + (self.num_vec_row + 1) * 4 + self.num_vec * 4

    def return_TCF_storage(self):
        return self.nnz * 2 + self.nnz * 3 * 4 + (self.M + 1) * 4 + self._tiles() * 32 * 4

    def return_SRBCSR_storage(self):
        return self.num_vec * self.vec_len * 2 + (self.num_vec_row + 1) * 4 + self._tiles() * 32 * 4

    def _tiles(self):
        return int((-(-np.diff(self._ptr) // 32)).sum())

    def CVSE_out(self, new_dir):
        """"m_vec, K, nnz" / vector row pointers / column ids, space separated, no
        trailing newline (reference :152-175)."""
        write_smtx(new_dir, self.num_vec_row, self.K, self.nnz, self._ptr, self._cols)


def return_all_zero_vec(vec_len, ROW, COL, origin_matrix):
    """Number of (vector row, column) positions with no non-zero in any of the
    vec_len rows (reference :177-188) = ceil(ROW/vec_len)*COL - nvec; nvec comes
    from the GPU counting pass."""
    if isinstance(origin_matrix, OriginMatrix):
        row_ptr, col = origin_matrix.row_ptr, origin_matrix.col
    else:
        dense = np.asarray(origin_matrix)[:ROW, :COL] != 0
        row_ptr = np.zeros(ROW + 1, dtype=np.int32)
        np.cumsum(dense.sum(axis=1), out=row_ptr[1:])
        col = np.nonzero(dense)[1].astype(np.int32)
    dev = _device()
    vec_ptr, _, _, _ = ops.svc(torch.from_numpy(np.ascontiguousarray(row_ptr[: ROW + 1])).to(dev),
                               torch.from_numpy(np.ascontiguousarray(col)).to(dev), None, ROW, COL, vec_len)
    return math.ceil(ROW / vec_len) * COL - int(vec_ptr[-1].item())


def _stats_row(i, m0: sparse_matrix, vec_len, c: CVSE):
    zero = math.ceil(m0.M / vec_len) * m0.N - c.num_vec
    vec_cnt = c.num_vec
    new_sparsity = 1.0 if vec_cnt == 0 else 1.0 - m0.nnz / (vec_cnt * vec_len)
    return [str(i), str(m0.M), str(m0.N), str(m0.nnz), str(new_sparsity), str(zero), str(c.return_CSR_storage()),
            str(c.return_CVSE_storage()), str(c.return_TCF_storage()), str(c.return_SRBCSR_storage())]


def generate_CVSE_file(src_dir, dest_dir, paths_txt, vec_len, csv_dir="./csv_data", limit: Optional[int] = None):
    """Batch driver (reference :190-250): for every path listed in ``paths_txt``
    read ``src_dir + name``, compress, write ``dest_dir + name`` and append one
    statistics row to ``<csv_dir>/RowMerge_V<V>.csv`` (columns: NO, ROW, COL, NNZ,
    new_sparsity, all_zero_vec_cnt, CSR/CVSE/TCF/SR-BCSR bytes).  The reference
    reads exactly 2688 lines; this reads the whole list (or ``limit`` lines)."""
    os.makedirs(csv_dir, exist_ok=True)
    with open(paths_txt) as f:
        names = [ln.split()[0] for ln in f if ln.strip()]
    if limit is not None:
        names = names[:limit]
    with open(os.path.join(csv_dir, f"RowMerge_V{vec_len}.csv"), "a", newline="") as fcsv:
        writer = csv.writer(fcsv)
        for i, name in enumerate(names):
            m0 = sparse_matrix(src_dir + name)
            c = CVSE(m0.M, m0.N, m0.nnz, m0.colInd_list_array(), vec_len)
            ok = c.num_vec_row + 1 == c._ptr.size and c.num_vec == int(c._ptr[-1]) == c._cols.size
            if not ok:
                print("NO.", i, "  format error")
                break
            os.makedirs(os.path.dirname(dest_dir + name) or ".", exist_ok=True)
            c.CVSE_out(dest_dir + name)
            print("No.", i, "  OK")
            print(dest_dir + name)
            writer.writerow(_stats_row(i, m0, vec_len, c))
    print("Row-Merge (V = ", vec_len, ") format transformation finish")
