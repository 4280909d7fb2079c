"""Row reordering before compression (extension of the path; the reference's own reorder stage,
`row_merge_reorder.py`, is not in its checkout, so parity is unpinned -- see csrc/reorder.cu).

    perm = row_permutation(row_ptr, col_idx, M, K, V)      # GPU, greedy grouping in 256-row windows
    row_ptr2, col2, vals2 = permute_rows(row_ptr, col_idx, vals, perm)
    ... ops.svc(row_ptr2, col2, vals2, M, K, V) ... ops.sspmm(...) -> rows of C in permuted order
    C_original_order[perm] = C_permuted[:M]
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import capi, ops


def row_permutation(row_ptr: torch.Tensor, col_idx: torch.Tensor, M: int, K: int, vec_length: int) -> torch.Tensor:
    ops._require(row_ptr, torch.int32, "row_ptr")
    ops._require(col_idx, torch.int32, "col_idx")
    perm = torch.empty(M, dtype=torch.int32, device=row_ptr.device)
    with torch.cuda.device(row_ptr.device):
        capi.check(capi.lib().svc_reorder(M, K, vec_length, row_ptr.data_ptr(), col_idx.data_ptr(), perm.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream))
    return perm


def permute_rows(row_ptr: torch.Tensor, col_idx: torch.Tensor, vals: Optional[torch.Tensor], perm: torch.Tensor
                 ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """CSR with rows in the order `perm` (row perm[r] becomes row r).  Device-side data movement only."""
    M = perm.numel()
    p = perm.to(torch.int64)
    starts = row_ptr[:M].to(torch.int64)[p]
    lens = (row_ptr[1: M + 1] - row_ptr[:M]).to(torch.int64)[p]
    new_ptr = torch.zeros(M + 1, dtype=torch.int64, device=row_ptr.device)
    torch.cumsum(lens, 0, out=new_ptr[1:])
    nnz = int(new_ptr[-1].item())
    row_of = torch.repeat_interleave(torch.arange(M, device=row_ptr.device), lens, output_size=nnz)
    src = starts[row_of] + (torch.arange(nnz, device=row_ptr.device) - new_ptr[:-1][row_of])
    return new_ptr.to(torch.int32), col_idx[src].contiguous(), (None if vals is None else vals[src].contiguous())
