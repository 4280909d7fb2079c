"""Device-side operators on torch CUDA tensors.  torch is used for device
memory and streams only; every computation is a call into libsspmm_b200.so."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import capi

KERNEL_AUTO, KERNEL_GATHER, KERNEL_SIMT, KERNEL_BLOCK, KERNEL_GATHER_LSU = 0, 1, 2, 3, 4


def _stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _require(t: torch.Tensor, dtype, name: str) -> None:
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def set_kernel(which: int) -> None:
    capi.check(capi.lib().sspmm_set_kernel(which))


def device_status() -> int:
    import ctypes as C
    s = C.c_int(0)
    capi.check(capi.lib().sspmm_device_status(C.byref(s)))
    return s.value


def sspmm(row_offsets: torch.Tensor, column_indices: torch.Tensor, values: torch.Tensor, rhs: torch.Tensor,
          vec_length: int, row_indices: Optional[torch.Tensor] = None, out_dtype=torch.float16,
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C[m_vec*V, N] = A_vs @ rhs[K, N] (the call made at SSpMM/sspmm_test.cpp:189)."""
    _require(row_offsets, torch.int32, "row_offsets")
    _require(column_indices, torch.int32, "column_indices")
    _require(values, torch.float16, "values")
    _require(rhs, torch.float16, "rhs")
    if row_indices is not None:
        _require(row_indices, torch.int32, "row_indices")
    m_vec = row_offsets.numel() - 1
    K, N = rhs.shape
    if out is None:
        out = torch.empty((m_vec * vec_length, N), dtype=out_dtype, device=rhs.device)
    fn = capi.lib().sspmm_f16_f16 if out.dtype == torch.float16 else capi.lib().sspmm_f16_f32
    args = (m_vec, vec_length, N, K, _ptr(row_indices), row_offsets.data_ptr(), column_indices.data_ptr(),
            values.data_ptr(), rhs.data_ptr(), out.data_ptr())
    if torch.cuda.current_device() == rhs.device.index:
        rc = fn(*args, _stream_ptr())
    else:
        with torch.cuda.device(rhs.device):
            rc = fn(*args, _stream_ptr())
    if rc != 0:
        capi.check(rc)
    return out


def svc(row_ptr: torch.Tensor, col_idx: torch.Tensor, values: Optional[torch.Tensor], M: int, K: int,
        vec_length: int) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor], int]:
    """Sparse vector compression of a CSR matrix held on the GPU.
    Returns (vec_row_ptr[m_vec+1], vec_col[nvec], vec_values[nvec*V] or None, replayed_rows)."""
    import ctypes as C
    _require(row_ptr, torch.int32, "row_ptr")
    _require(col_idx, torch.int32, "col_idx")
    if values is not None:
        _require(values, torch.float16, "values")
    dev = row_ptr.device
    m_vec = (M + vec_length - 1) // vec_length
    job = C.c_void_p()
    nvec = C.c_int64(0)
    lib = capi.lib()
    with torch.cuda.device(dev):
        st = _stream_ptr()
        capi.check(lib.svc_begin(M, K, vec_length, row_ptr.data_ptr(), col_idx.data_ptr(), _ptr(values), st,
                                 C.byref(job), C.byref(nvec)))
        try:
            n = nvec.value
            vec_ptr = torch.empty(m_vec + 1, dtype=torch.int32, device=dev)
            vec_col = torch.empty(n, dtype=torch.int32, device=dev)
            vec_val = torch.empty(n * vec_length, dtype=torch.float16, device=dev) if values is not None else None
            replayed = C.c_int64(0)
            capi.check(lib.svc_replayed_rows(job, C.byref(replayed)))
            capi.check(lib.svc_finish(job, vec_ptr.data_ptr(), vec_col.data_ptr(), _ptr(vec_val), st))
        finally:
            lib.svc_free(job)
    return vec_ptr, vec_col, vec_val, replayed.value


def sorted_row_swizzle(row_offsets: torch.Tensor) -> torch.Tensor:
    _require(row_offsets, torch.int32, "row_offsets")
    m_vec = row_offsets.numel() - 1
    out = torch.empty(m_vec, dtype=torch.int32, device=row_offsets.device)
    with torch.cuda.device(row_offsets.device):
        capi.check(capi.lib().sspmm_sorted_row_swizzle(m_vec, row_offsets.data_ptr(), out.data_ptr(), _stream_ptr()))
    return out
