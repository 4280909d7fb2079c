"""SuiteSparse side of the preprocessing stage, with the compression on the GPU.

Same names and arguments as the reference module RowMerge/suit_sparse_matrix.py for the part that
feeds the compression:

* ``suite_matrix(path)``         Matrix Market reader, reference :85-151 (M, K, nnz, ``coo2csr``,
                                 ``colInd_list_array``, ``sparsity``)
* ``generate_suitesparse_CVSE_file(src_dir, dest_dir, paths_txt, vec_len)``   batch driver, reference :181-221:
  for every line of ``paths_txt`` read ``src_dir + line`` (.mtx), write the CSR next to it as
  ``*_csr.mtx`` (three-line text format), compress, write ``dest_dir + line`` with ``.mtx`` replaced by
  ``.smtx``.

Reading and the COO -> CSR conversion use scipy exactly as the reference does, so duplicate entries are
summed and the column order inside a row is scipy's; the compression is ``sparse_matrix_format.CVSE``
(GPU only, no CPU implementation here)."""
from __future__ import annotations

import os

import numpy as np
from scipy.io import mmread
from scipy.sparse import coo_matrix

from . import sparse_matrix_format


class suite_matrix:
    def __init__(self, path):
        coo = coo_matrix(mmread(path))
        self.path = path
        self.coo = coo
        self.M, self.K = coo.shape
        self.nnz = coo.nnz
        self._csr = None

    def _csr_arrays(self):
        if self._csr is None:
            csr = self.coo.tocsr()
            self._csr = (np.asarray(csr.indptr, dtype=np.int32), np.asarray(csr.indices, dtype=np.int32))
        return self._csr

    def coo2csr(self, gen=0):
        """(row pointers, column ids); with ``gen == 1`` also writes ``<path without .mtx>_csr.mtx`` in the
        three-line text format (reference :109-137)."""
        row_ptr, col = self._csr_arrays()
        if gen == 1:
            new_filename = self.path.replace(".mtx", "_csr.mtx")
            sparse_matrix_format.write_smtx(new_filename, self.M, self.K, self.nnz, row_ptr, col)
            print("Gnerate _csr.mtx File: ", new_filename)
        return row_ptr, col

    def colInd_list_array(self):
        """Per-row column lists (reference :138-148) as a sequence over the CSR arrays."""
        row_ptr, col = self._csr_arrays()
        return sparse_matrix_format._CsrRows(row_ptr, col)

    def sparsity(self):
        return 1.0 - self.nnz / self.M / self.K

    def origin_matrix(self):
        row_ptr, col = self._csr_arrays()
        return sparse_matrix_format.OriginMatrix(self.M, self.K, row_ptr, col)


def generate_suitesparse_CVSE_file(src_dir, dest_dir, paths_txt, vec_len):
    with open(paths_txt, "r") as file:
        print("Begin to gen CSR-file and CVSE-file, vecLength=", vec_len)
        lines = [line.rstrip("\n") for line in file]
    lines = [ln for ln in lines if ln.strip()]
    print("Number of file is ", len(lines))
    for i, name in enumerate(lines):
        source_file_name = src_dir + name
        dest_file_name = (dest_dir + name).replace(".mtx", ".smtx")
        print("source: ", source_file_name)
        print("dest:   ", dest_file_name)
        m = suite_matrix(source_file_name)
        print(m.M, m.K, m.nnz, m.sparsity())
        m.coo2csr(1)
        c = sparse_matrix_format.CVSE(m.M, m.K, m.nnz, m.colInd_list_array(), vec_len)
        os.makedirs(os.path.dirname(dest_file_name) or ".", exist_ok=True)
        c.CVSE_out(dest_file_name)
        print("File-", i, " Finished")
