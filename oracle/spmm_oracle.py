"""TEST INFRASTRUCTURE -- loader of the C oracle for the vector-sparse SpMM
(oracle/spmm_host.c, a restatement of SSpMM/sspmm_test.cpp:75-95).  Never
imported by the product package."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(HERE, "_build", "liboracle_spmm.so")
_lib = None


def build() -> str:
    src = os.path.join(HERE, "spmm_host.c")
    if not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "_build/liboracle_spmm.so"], check=True, capture_output=True)
    return _SO


def _load():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.oracle_sspmm_rows.restype = None
        _lib.oracle_sspmm_rows.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int] + [C.c_void_p] * 5 + [C.c_int]
        _lib.oracle_half_to_float.restype = None
        _lib.oracle_half_to_float.argtypes = [C.c_void_p, C.c_void_p, C.c_int64]
    return _lib


def sspmm_host(V: int, row_offsets, col_indices, values_f16, rhs_f16, rows=None, threads: int = 1) -> np.ndarray:
    """fp32 [n_rows*V, N] for vector rows ``rows = (begin, end)`` (default all)."""
    lib = _load()
    ro = np.ascontiguousarray(row_offsets, dtype=np.int32)
    ci = np.ascontiguousarray(col_indices, dtype=np.int32)
    va = np.ascontiguousarray(values_f16, dtype=np.float16)
    rhs = np.ascontiguousarray(rhs_f16, dtype=np.float16)
    K, N = rhs.shape
    m_vec = ro.size - 1
    b, e = (0, m_vec) if rows is None else rows
    rhs32 = np.empty((K, N), dtype=np.float32)
    lib.oracle_half_to_float(rhs.ctypes.data, rhs32.ctypes.data, rhs.size)
    out = np.empty(((e - b) * V, N), dtype=np.float32)
    lib.oracle_sspmm_rows(b, e, V, N, ro.ctypes.data, ci.ctypes.data, va.ctypes.data, rhs32.ctypes.data,
                          out.ctypes.data, threads)
    return out
