"""TEST INFRASTRUCTURE -- binding of the reference's own GPU kernel library
(oracle/_ref/libsspmm_ref.so, compiled by oracle/Makefile from the reference's
SSpMM/src/sspmm.cu, unmodified).  Used as a second oracle and as the
"reference kernel on the same GPU" comparator; never by the product package.

The reference kernels assume N % 64 == 0 and their V=16 tile loader reads up to
31 vectors past the end of the last vector row (SSpMM/src/spmm_utils/
sspmm_sparse_tile.h:299-310), so callers must pad `values` and
`column_indices` by at least 32 vectors."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "_ref", "libsspmm_ref.so")
PAD_VECTORS = 64

_SYM_F32 = "_ZN4spmm5SSpMMEiiiiPKiS1_S1_PK6__halfS4_Pf"
_SYM_F16 = "_ZN4spmm5SSpMMEiiiiPKiS1_S1_PK6__halfS4_PS2_"


def available() -> bool:
    return os.path.exists(SO)


_lib = None


def _fn(f16_out: bool):
    global _lib
    if _lib is None:
        _lib = C.CDLL(SO)
    fn = getattr(_lib, _SYM_F16 if f16_out else _SYM_F32)
    fn.restype = C.c_int
    fn.argtypes = [C.c_int] * 4 + [C.c_void_p] * 6
    return fn


def sspmm_ref(m_vec, V, N, K, row_indices, row_offsets, column_indices, values, rhs, out) -> int:
    """All arguments after K are torch CUDA tensors; runs on the legacy default stream."""
    import torch
    if N % 64 != 0:
        raise ValueError("the reference kernel needs N % 64 == 0")
    fn = _fn(out.dtype == torch.float16)
    return fn(m_vec, V, N, K, row_indices.data_ptr(), row_offsets.data_ptr(), column_indices.data_ptr(),
              values.data_ptr(), rhs.data_ptr(), out.data_ptr())
