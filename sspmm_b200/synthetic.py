"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (the reference's DLMC / SuiteSparse files are not
redistributable here, so every test and benchmark draws its matrices from
these generators).

All matrices are returned in CSR (int32 row pointers, int32 ascending column
ids per row, float16 values), the form the reference's reader produces
(RowMerge/sparse_matrix_format.py:8-53)."""
from __future__ import annotations

import dataclasses
from typing import List, Tuple

import numpy as np


@dataclasses.dataclass
class CSR:
    M: int
    K: int
    row_ptr: np.ndarray  # int32 [M+1]
    col_idx: np.ndarray  # int32 [nnz]
    values: np.ndarray   # float16 [nnz]

    @property
    def nnz(self) -> int:
        return int(self.row_ptr[-1])

    def row_lists(self) -> List[List[int]]:
        c = self.col_idx.tolist()
        p = self.row_ptr.tolist()
        return [c[p[i]:p[i + 1]] for i in range(self.M)]

    def dense(self) -> np.ndarray:
        a = np.zeros((self.M, self.K), dtype=np.float16)
        rows = np.repeat(np.arange(self.M), np.diff(self.row_ptr))
        a[rows, self.col_idx] = self.values
        return a


def magnitude_pruned(M: int, K: int, sparsity: float, rng: np.random.Generator) -> CSR:
    """Dense N(0, 0.02) draw in fp16; keep exactly round((1-s)*M*K) entries of
    largest magnitude (ties go to the lower flat index)."""
    w = rng.normal(0.0, 0.02, (M, K)).astype(np.float16)
    keep = int(round((1.0 - sparsity) * M * K))
    flat = np.abs(w.astype(np.float32)).ravel()
    order = np.argsort(-flat, kind="stable")
    mask = np.zeros(M * K, dtype=bool)
    mask[order[:keep]] = True
    mask = mask.reshape(M, K)
    row_ptr = np.zeros(M + 1, dtype=np.int32)
    np.cumsum(mask.sum(axis=1), out=row_ptr[1:])
    r, c = np.nonzero(mask)
    return CSR(M, K, row_ptr, c.astype(np.int32), w[r, c])


def dense_rhs(K: int, N: int, rng: np.random.Generator) -> np.ndarray:
    return rng.normal(0.0, 1.0, (K, N)).astype(np.float16)


def power_law(n: int, rng: np.random.Generator, mean_nnz: float = 16.0) -> CSR:
    """Square n x n matrix whose row lengths follow a Zipf(2) law truncated at n
    and rescaled to a mean of ``mean_nnz``; column ids uniform without
    replacement (ascending inside a row); values U(-1, 1) in fp16."""
    z = rng.zipf(2.0, n).astype(np.float64)
    z = np.minimum(z, n)
    ln = np.clip(np.rint(mean_nnz * z / z.mean()), 1, n).astype(np.int64)
    row_ptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(ln, out=row_ptr[1:])
    cols = np.empty(int(row_ptr[-1]), dtype=np.int32)
    for r in range(n):
        l = int(ln[r])
        if l * 4 > n:
            pick = rng.permutation(n)[:l]
        else:
            pick = np.unique(rng.integers(0, n, l + 8))
            while pick.size < l:
                pick = np.unique(np.concatenate([pick, rng.integers(0, n, l)]))
            if pick.size > l:
                pick = rng.permutation(pick)[:l]
        pick.sort()
        cols[row_ptr[r]:row_ptr[r + 1]] = pick
    vals = rng.uniform(-1.0, 1.0, cols.size).astype(np.float16)
    return CSR(n, n, row_ptr.astype(np.int32), cols, vals)


def power_law_device(n: int, seed: int, device, mean_nnz: float = 16.0):
    """The distribution of ``power_law`` (row lengths from Zipf(2) truncated at n and rescaled to the mean, uniform
    column ids without replacement, ascending inside a row, values U(-1, 1) in fp16) drawn on the GPU with torch's
    seeded generator: a sweep of thousands of matrices is generated in seconds.  Returns device tensors
    (row_ptr int32 [n+1], col_idx int32 [nnz], values fp16 [nnz]).  Not the same matrices as ``power_law``."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    k = torch.arange(1, n + 1, device=device, dtype=torch.float64)
    cdf = torch.cumsum(k ** -2.0, 0)
    cdf /= cdf[-1].clone()
    z = (torch.searchsorted(cdf, torch.rand(n, device=device, dtype=torch.float64, generator=g)) + 1).clamp_(max=n).double()
    ln = torch.clamp(torch.round(mean_nnz * z / z.mean()), 1, n).long()
    heavy = ln * 4 > n
    want = torch.where(heavy, torch.zeros_like(ln), ln)
    # light rows: oversample, keep each row's distinct draws, thin the surplus at random
    over = torch.where(heavy, torch.zeros_like(ln), want + 8 + want // 4)
    rows = torch.repeat_interleave(torch.arange(n, device=device), over)
    keys = torch.unique(rows * n + torch.randint(0, n, (rows.numel(),), device=device, generator=g))
    krow = keys // n
    have = torch.bincount(krow, minlength=n)
    redo = heavy | (have < want)                              # heavy rows, and (rare) rows short of distinct draws
    prio = torch.rand(keys.numel(), device=device, generator=g)
    order = torch.argsort(krow.double() + prio)                # inside a row: random order (prio < 1)
    start = torch.cumsum(have, 0) - have
    ko = krow[order]
    rank = torch.arange(keys.numel(), device=device) - start[ko]
    keep = order[(rank < want[ko]) & ~redo[ko]]
    kept = keys[keep]
    extra = []
    for r in torch.nonzero(redo).flatten().tolist():
        pick = torch.randperm(n, device=device, generator=g)[: int(ln[r])]
        extra.append(r * n + pick)
    if extra:
        kept = torch.cat([kept] + extra)
    kept, _ = torch.sort(kept)
    row_ptr = torch.zeros(n + 1, device=device, dtype=torch.int64)
    row_ptr[1:] = torch.cumsum(torch.bincount(kept // n, minlength=n), 0)
    col = (kept % n).int()
    vals = (torch.rand(col.numel(), device=device, generator=g) * 2 - 1).half()
    return row_ptr.int(), col, vals


# ---- named configurations ------------------------------------------------- #

FFN_SHAPES = [(2048, 512), (512, 2048)]
FFN_SPARSITIES = [0.5, 0.7, 0.8, 0.9, 0.95, 0.98]

# (Cout, K): 3x3 layers with Cin = Cout (K = 9*Cin) and 1x1 layers (K = Cin)
CONV_LAYERS = [(64, 576), (128, 1152), (256, 2304), (512, 4608),
               (256, 64), (512, 128), (1024, 256), (2048, 512)]
CONV_SPARSITIES = [0.8, 0.9]
CONV_N = 8 * 56 * 56

# hidden 768, FFN 3072: Q, K, V, O, FFN1, FFN2
ENCODER_WEIGHTS = [(768, 768)] * 4 + [(3072, 768), (768, 3072)]
ENCODER_TOKENS = 32 * 512


def config1(seed: int = 1) -> Tuple[CSR, np.ndarray]:
    """512x512 at 70 % sparsity, dense operand 512x256."""
    rng = np.random.default_rng(seed)
    a = magnitude_pruned(512, 512, 0.7, rng)
    return a, dense_rhs(512, 256, rng)


def ffn(shape_id: int, sparsity_id: int, N: int = 256) -> Tuple[CSR, np.ndarray]:
    rng = np.random.default_rng(200 + 10 * shape_id + sparsity_id)
    M, K = FFN_SHAPES[shape_id]
    a = magnitude_pruned(M, K, FFN_SPARSITIES[sparsity_id], rng)
    return a, dense_rhs(K, N, rng)


def conv_weight(layer_id: int, sparsity_id: int) -> CSR:
    rng = np.random.default_rng(300 + 10 * layer_id + sparsity_id)
    M, K = CONV_LAYERS[layer_id]
    return magnitude_pruned(M, K, CONV_SPARSITIES[sparsity_id], rng)


def encoder_weight(weight_id: int) -> CSR:
    rng = np.random.default_rng(400 + weight_id)
    M, K = ENCODER_WEIGHTS[weight_id]
    return magnitude_pruned(M, K, 0.9, rng)


def sweep_size(matrix_id: int) -> int:
    """n is log-uniform in [4096, 65536], fixed by the matrix id alone."""
    rng = np.random.default_rng(5000 + matrix_id)
    return int(round(4096 * 16.0 ** rng.random()))


def sweep_matrix(matrix_id: int) -> CSR:
    rng = np.random.default_rng(5000 + matrix_id)
    n = int(round(4096 * 16.0 ** rng.random()))
    return power_law(n, rng)


def sweep_matrix_device(matrix_id: int, device):
    """Matrix `matrix_id` of the 2000-matrix sweep, drawn on the GPU: n from the same seed rule as ``sweep_matrix``."""
    n = sweep_size(matrix_id)
    return (n,) + tuple(power_law_device(n, 5000 + matrix_id, device))
