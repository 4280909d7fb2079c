"""TEST INFRASTRUCTURE -- CPU restatement of the row-reordering extension (sspmm_b200/csrc/reorder.cu).

PARITY UNPINNED: the reference's reorder.py / row_merge_reorder.py are absent from the reference
checkout (only its README.md:36 and the data-set paths in SSpMM/sspmm_test.cpp:313-319 mention the
stage), so this restates OUR algorithm, not the reference's; tests use it to pin the CUDA kernel and
check invariants (valid permutation, fewer or equal vectors on structured inputs, SpMM unchanged up to
the permutation)."""
from __future__ import annotations

import numpy as np

WINDOW = 256
SIG_BITS = 2048


def _sig_bit(c: np.ndarray, K: int) -> np.ndarray:
    if K <= SIG_BITS:
        return c.astype(np.int64)
    return ((c.astype(np.uint64) * np.uint64(2654435761)) & np.uint64(0xFFFFFFFF)) >> np.uint64(21)


def row_permutation(M: int, K: int, V: int, row_ptr, col) -> np.ndarray:
    row_ptr = np.asarray(row_ptr)
    col = np.asarray(col)
    perm = np.empty(M, dtype=np.int32)
    for w0 in range(0, M, WINDOW):
        wn = min(WINDOW, M - w0)
        sig = np.zeros((wn, SIG_BITS), dtype=bool)
        for r in range(wn):
            c = col[row_ptr[w0 + r]:row_ptr[w0 + r + 1]]
            c = c[(c >= 0) & (c < K)]
            sig[r, _sig_bit(c, K)] = True
        assigned = np.zeros(wn, dtype=bool)
        pos = 0
        while pos < wn:
            seed = int(np.argmin(assigned))             # first unassigned
            group = sig[seed].copy()
            assigned[seed] = True
            perm[w0 + pos] = w0 + seed
            pos += 1
            k = 1
            while k < V and pos < wn:
                growth = (sig & ~group).sum(axis=1).astype(np.int64)
                growth[assigned] = np.iinfo(np.int64).max
                best = int(np.argmin(growth))           # ties -> lowest row
                group |= sig[best]
                assigned[best] = True
                perm[w0 + pos] = w0 + best
                pos += 1
                k += 1
    return perm


def permute_rows(M, row_ptr, col, vals, perm):
    row_ptr = np.asarray(row_ptr, dtype=np.int64)
    lens = np.diff(row_ptr)[perm]
    new_ptr = np.zeros(M + 1, dtype=np.int32)
    np.cumsum(lens, out=new_ptr[1:])
    idx = np.concatenate([np.arange(row_ptr[r], row_ptr[r + 1]) for r in perm] + [np.zeros(0, dtype=np.int64)]).astype(np.int64)
    return new_ptr, np.asarray(col)[idx], (None if vals is None else np.asarray(vals)[idx])
