"""`sptrans.spmm` of the reference's PyTorch extension, on the B200 kernels.

Same functions, argument order and return convention as the pybind module
end2end/sspmm_e2e/src/cuda/spmm.cpp:11-47 (implementation spmm_kernel.cu:460-586):

    spmm (row_indices, row_offsets, column_indices, values, rhs_matrix, vec_length) -> [m, k]     fp16
    bspmm(row_indices, row_offsets, column_indices, values, rhs_matrix, vec_length) -> [b, m, k]  fp16

with m = (len(row_offsets) - 1) * vec_length, rhs_matrix = [n, k] (or [b, n, k]), values =
[nvec * vec_length] (or [b, nvec * vec_length], one value array per batch entry).  The output is
allocated here, as in the reference.  vec_length 8 or 16 (the reference's 4 and 2 are the
vectorSparse kernels, outside this library's path)."""
from __future__ import annotations

import torch

from .. import capi, ops


def spmm(row_indices, row_offsets, column_indices, values, rhs_matrix, vec_length):
    return ops.sspmm(row_offsets, column_indices, values.reshape(-1), rhs_matrix, vec_length,
                     row_indices=row_indices, out_dtype=torch.float16)


def bspmm(row_indices, row_offsets, column_indices, values, rhs_matrix, vec_length):
    for t, dt, name in ((row_indices, torch.int32, "row_indices"), (row_offsets, torch.int32, "row_offsets"),
                        (column_indices, torch.int32, "column_indices"), (values, torch.float16, "values"),
                        (rhs_matrix, torch.float16, "rhs_matrix")):
        ops._require(t, dt, name)
    m_vec = row_offsets.numel() - 1
    n, k = rhs_matrix.shape[-2], rhs_matrix.shape[-1]
    batch = rhs_matrix.numel() // (n * k) if n * k else 0
    nnz = column_indices.numel() * vec_length
    shared_values = values.numel() == nnz and batch != 1
    out = torch.empty((batch, m_vec * vec_length, k), dtype=torch.float16, device=rhs_matrix.device)
    with torch.cuda.device(rhs_matrix.device):
        capi.check(capi.lib().sspmm_f16_f16_batched(
            m_vec, vec_length, k, n, batch, row_indices.data_ptr(), row_offsets.data_ptr(), column_indices.data_ptr(),
            values.data_ptr(), 0 if shared_values else nnz, rhs_matrix.data_ptr(), n * k, out.data_ptr(),
            m_vec * vec_length * k, torch.cuda.current_stream().cuda_stream))
    return out
