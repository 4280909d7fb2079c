"""Device-side operators on torch CUDA tensors.  torch is used for device
memory and streams only; every computation is a call into libsspmm_b200.so."""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import capi

KERNEL_AUTO, KERNEL_GATHER, KERNEL_SIMT, KERNEL_BLOCK, KERNEL_GATHER_LSU, KERNEL_BLOCK_SINGLE = 0, 1, 2, 3, 4, 5


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


def svc_batch(mats, vec_length: int, nnz=None):
    """Sparse vector compression of several independent CSR matrices in one pass (``svc_batch_begin`` /
    ``svc_batch_finish``): the matrices are stacked on the device and compressed together.

    ``mats`` is a list of (row_ptr, col_idx, values_or_None, M, K) with device tensors; ``nnz`` the list of
    their non-zero counts (taken from ``col_idx.numel()`` when omitted).  Returns a list of
    (vec_row_ptr, vec_col, vec_values_or_None) per matrix -- views into three buffers that hold all matrices
    one after another -- and the total number of replayed vector rows."""
    import ctypes as C
    if not mats:
        return [], 0
    V = vec_length
    n = len(mats)
    dev = mats[0][0].device
    with_vals = all(m[2] is not None for m in mats)
    if nnz is None:
        nnz = [int(m[1].numel()) for m in mats]
    for (rp, ci, va, M, K) in mats:
        _require(rp, torch.int32, "row_ptr")
        _require(ci, torch.int32, "col_idx")
        if with_vals:
            _require(va, torch.float16, "values")
    Ms = (C.c_int * n)(*[m[3] for m in mats])
    Ks = (C.c_int * n)(*[m[4] for m in mats])
    Zs = (C.c_int * n)(*nnz)
    p_ptr = (C.c_void_p * n)(*[m[0].data_ptr() for m in mats])
    p_col = (C.c_void_p * n)(*[m[1].data_ptr() for m in mats])
    p_val = (C.c_void_p * n)(*[m[2].data_ptr() for m in mats]) if with_vals else None
    nvec = (C.c_int64 * n)()
    job = C.c_void_p()
    lib = capi.lib()
    with torch.cuda.device(dev):
        st = _stream_ptr()
        capi.check(lib.svc_batch_begin(n, V, Ms, Ks, Zs, p_ptr, p_col, p_val, st, C.byref(job), nvec))
        try:
            replayed = C.c_int64(0)
            capi.check(lib.svc_batch_replayed_rows(job, C.byref(replayed)))
            m_vecs = [(m[3] + V - 1) // V for m in mats]
            total_vec = sum(nvec)
            vec_ptr = torch.empty(sum(m_vecs) + n, dtype=torch.int32, device=dev)
            vec_col = torch.empty(total_vec, dtype=torch.int32, device=dev)
            vec_val = torch.empty(total_vec * V, dtype=torch.float16, device=dev) if with_vals else None
            capi.check(lib.svc_batch_finish(job, vec_ptr.data_ptr(), vec_col.data_ptr(), _ptr(vec_val), st))
        finally:
            lib.svc_batch_free(job)
    out, po, vo = [], 0, 0
    for k in range(n):
        nv = nvec[k]
        out.append((vec_ptr[po: po + m_vecs[k] + 1], vec_col[vo: vo + nv], None if vec_val is None else vec_val[vo * V: (vo + nv) * V]))
        po += m_vecs[k] + 1
        vo += nv
    return out, replayed.value


def sorted_row_swizzle(row_offsets: torch.Tensor) -> torch.Tensor:
    _require(row_offsets, torch.int32, "row_offsets")
    m_vec = row_offsets.numel() - 1
    out = torch.empty(m_vec, dtype=torch.int32, device=row_offsets.device)
    with torch.cuda.device(row_offsets.device):
        capi.check(capi.lib().sspmm_sorted_row_swizzle(m_vec, row_offsets.data_ptr(), out.data_ptr(), _stream_ptr()))
    return out


class Plan:
    """Ahead-of-time part of the SpMM for one weight structure (``sspmm_plan_create``): with it the product runs
    as one kernel launch straight from the compressed operand, without scratch, allocation or host
    synchronisation.  Keeps ``row_offsets`` and ``column_indices`` alive; the values may change between calls."""

    def __init__(self, row_offsets: torch.Tensor, column_indices: torch.Tensor, vec_length: int, K: int):
        import ctypes as C
        _require(row_offsets, torch.int32, "row_offsets")
        _require(column_indices, torch.int32, "column_indices")
        self.row_offsets, self.column_indices = row_offsets, column_indices
        self.V, self.K = vec_length, K
        self.m_vec = row_offsets.numel() - 1
        self.device = row_offsets.device
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            capi.check(capi.lib().sspmm_plan_create(self.m_vec, vec_length, K, row_offsets.data_ptr(),
                                                    column_indices.data_ptr(), _stream_ptr(), C.byref(self._h)))
        nvec, one, asc, nbytes = C.c_int64(), C.c_int(), C.c_int(), C.c_int64()
        capi.check(capi.lib().sspmm_plan_info(self._h, C.byref(nvec), C.byref(one), C.byref(asc), C.byref(nbytes)))
        self.nvec, self.one_launch, self.ascending, self.device_bytes = nvec.value, bool(one.value), bool(asc.value), nbytes.value

    @property
    def handle(self):
        return self._h

    def close(self) -> None:
        if self._h:
            capi.lib().sspmm_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def sspmm_planned(plan: Plan, values: torch.Tensor, rhs: torch.Tensor, out_dtype=torch.float16,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A_vs @ rhs through ``sspmm_planned``: one launch, nothing allocated by the library."""
    _require(values, torch.float16, "values")
    _require(rhs, torch.float16, "rhs")
    K, N = rhs.shape
    if K != plan.K:
        raise ValueError(f"rhs has {K} rows, the plan was built for K = {plan.K}")
    if out is None:
        out = torch.empty((plan.m_vec * plan.V, N), dtype=out_dtype, device=rhs.device)
    with torch.cuda.device(rhs.device):
        rc = capi.lib().sspmm_planned(plan.handle, values.data_ptr(), rhs.data_ptr(), out.data_ptr(), N,
                                      1 if out.dtype == torch.float16 else 0, _stream_ptr())
    if rc != 0:
        capi.check(rc)
    return out


class Group:
    """Several products bound to their operands and run as ONE persistent launch (``sspmm_group_create`` /
    ``sspmm_group_run``).  ``products`` is a list of (plan, values, rhs, out); all outputs share one dtype.
    ``mode``: COMPRESSED builds the A tiles inside the kernel from the compressed operand (no scratch for A),
    EXPANDED lets the kernel's loader warps write dense copies of A while the first tiles are multiplied (faster per
    K step), PAIRS is EXPANDED with 256 x 256 tiles on CTA pairs, AUTO picks COMPRESSED or EXPANDED by the work per
    SM.  Every mode is one launch per run."""

    AUTO, COMPRESSED, EXPANDED, PAIRS = 0, 1, 2, 3

    def __init__(self, products, mode: int = 0):
        import ctypes as C
        if not products:
            raise ValueError("a group needs at least one product")
        self._keep = list(products)
        out_dtype = products[0][3].dtype
        arr = (capi.GroupItem * len(products))()
        for i, (plan, values, rhs, out) in enumerate(products):
            _require(values, torch.float16, "values")
            _require(rhs, torch.float16, "rhs")
            _require(out, out_dtype, "out")
            if rhs.shape[0] != plan.K or tuple(out.shape) != (plan.m_vec * plan.V, rhs.shape[1]):
                raise ValueError(f"product {i}: operand shapes do not match the plan")
            arr[i] = capi.GroupItem(plan.handle, values.data_ptr(), rhs.data_ptr(), out.data_ptr(), rhs.shape[1])
        self.device = products[0][2].device
        self._h = C.c_void_p()
        with torch.cuda.device(self.device):
            capi.check(capi.lib().sspmm_group_create(arr, len(products), 1 if out_dtype == torch.float16 else 0, mode, C.byref(self._h)))
        bn, items, ctas, launches, nbytes = C.c_int(), C.c_int(), C.c_int(), C.c_int(), C.c_int64()
        capi.check(capi.lib().sspmm_group_info(self._h, C.byref(bn), C.byref(items), C.byref(ctas), C.byref(launches), C.byref(nbytes)))
        self.tile_columns, self.work_items, self.ctas, self.scratch_bytes = bn.value, items.value, ctas.value, nbytes.value
        self.launches = launches.value

    def run(self) -> None:
        if torch.cuda.current_device() == self.device.index:
            rc = capi.lib().sspmm_group_run(self._h, _stream_ptr())
        else:
            with torch.cuda.device(self.device):
                rc = capi.lib().sspmm_group_run(self._h, _stream_ptr())
        if rc != 0:
            capi.check(rc)

    def close(self) -> None:
        if self._h:
            capi.lib().sspmm_group_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def workspace_bytes(m_vec: int, vec_length: int, N: int, K: int, nvec: int, out_is_f16: bool = True) -> int:
    """Scratch ``sspmm_ws`` would like for these sizes (``sspmm_workspace_bytes``)."""
    import ctypes as C
    b = C.c_int64(0)
    capi.check(capi.lib().sspmm_workspace_bytes(m_vec, vec_length, N, K, nvec, 1 if out_is_f16 else 0, C.byref(b)))
    return b.value


def sspmm_ws(row_offsets: torch.Tensor, column_indices: torch.Tensor, values: torch.Tensor, rhs: torch.Tensor,
             vec_length: int, nvec: int, workspace: Optional[torch.Tensor], out: Optional[torch.Tensor] = None,
             row_indices: Optional[torch.Tensor] = None) -> torch.Tensor:
    """C = A_vs @ rhs through ``sspmm_f16_f16_ws``: the caller passes the vector count and owns the scratch, so the
    library reads nothing back, allocates nothing and never synchronises."""
    m_vec = row_offsets.numel() - 1
    K, N = rhs.shape
    if out is None:
        out = torch.empty((m_vec * vec_length, N), dtype=torch.float16, device=rhs.device)
    ws_ptr = workspace.data_ptr() if workspace is not None else None
    ws_bytes = workspace.numel() * workspace.element_size() if workspace is not None else 0
    with torch.cuda.device(rhs.device):
        rc = capi.lib().sspmm_f16_f16_ws(m_vec, vec_length, N, K, _ptr(row_indices), row_offsets.data_ptr(),
                                         column_indices.data_ptr(), values.data_ptr(), rhs.data_ptr(), out.data_ptr(),
                                         nvec, ws_ptr, ws_bytes, _stream_ptr())
    if rc != 0:
        capi.check(rc)
    return out
