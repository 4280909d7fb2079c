"""Multi-GPU use of the SpMM: the columns of the dense operand B (and of C) are
independent, so rank g owns the contiguous column range ``shard_bounds(N, G)[g]``
of both and runs the single-GPU kernel on it with a replicated A_vs.  No
collective is needed to produce the sharded C; ``gather_columns`` assembles a
replicated C with one all-gather when the caller asks for it.

The reference has no multi-GPU path (it launches on one device,
SSpMM/sspmm_test.cpp:108-127), so this module has no counterpart there."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

COLUMN_QUANTUM = 8   # keeps every shard's rows 16-byte aligned for the tensor-core path


def shard_bounds(N: int, world: int, quantum: int = COLUMN_QUANTUM) -> List[Tuple[int, int]]:
    """Contiguous, near-equal column ranges whose starts are multiples of
    ``quantum`` (the last shard takes the remainder)."""
    if world < 1:
        raise ValueError("world size must be positive")
    units = -(-N // quantum)
    base, extra = divmod(units, world)
    out, start = [], 0
    for g in range(world):
        n_units = base + (1 if g < extra else 0)
        end = min(N, start + n_units * quantum)
        out.append((start, end))
        start = end
    return out


def shard_matrices(sweep_ids: List[int], rank: int, world: int) -> List[int]:
    """Independent matrices of a sweep are dealt round-robin: id mod world == rank."""
    return [i for i in sweep_ids if i % world == rank]


def gather_columns(local: torch.Tensor, N: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """local: this rank's [rows, n_g] column shard (bounds from ``shard_bounds``).
    Returns the replicated [rows, N] matrix on every rank."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    bounds = shard_bounds(N, world)
    rows = local.shape[0]
    assert local.shape[1] == bounds[rank][1] - bounds[rank][0], "shard width does not match shard_bounds"
    widest = max(e - s for s, e in bounds)
    # equal-sized staging blocks so one all_gather_into_tensor moves everything
    stage = torch.zeros((rows, widest), dtype=local.dtype, device=local.device)
    stage[:, : local.shape[1]] = local
    flat = torch.empty((world * rows, widest), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(flat, stage, group=group)
    gathered = flat.view(world, rows, widest)
    out = torch.empty((rows, N), dtype=local.dtype, device=local.device)
    for g, (s, e) in enumerate(bounds):
        out[:, s:e] = gathered[g, :, : e - s]
    return out


def sharded_sspmm(row_offsets, column_indices, values, rhs_local, vec_length, N_total: int, replicate: bool = False,
                  row_indices=None, out_dtype=torch.float16, group: Optional[dist.ProcessGroup] = None):
    """SpMM on this rank's column shard of B; ``replicate=True`` adds the all-gather."""
    from . import ops
    c_local = ops.sspmm(row_offsets, column_indices, values, rhs_local, vec_length, row_indices=row_indices,
                        out_dtype=out_dtype)
    if not replicate or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return c_local
    return gather_columns(c_local, N_total, group)
