"""The entry point that allocates nothing, sspmm_f16_f16_noalloc, against the regular
sspmm_f16_f16 on the same operands.

It exists for callers that cannot allocate device memory at call time (a serving process whose
arena already owns all device memory, a latency-critical loop where an allocation may fail or stall
other streams); its scratch is one fixed array shared by every call, so the test makes two calls in
a row with different matrices and checks that neither sees anything of the other.

This file sorts last on purpose: a run that stops at the first failure has then already executed
every other test.  It also passes when run alone in a fresh process."""
import ctypes as C

import numpy as np
import pytest
import torch

from sspmm_b200 import capi, ops

DEV = "cuda:0"
MAX_SCRATCH = 8 << 20


def random_cvse(seed, m_vec, K, V, density):
    rng = np.random.default_rng(seed)
    lens = rng.binomial(K, density, m_vec)
    lens[rng.integers(0, m_vec)] = 0                       # one empty vector row
    ptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    col = np.concatenate([np.sort(rng.permutation(K)[:l]) for l in lens] + [np.zeros(0, dtype=np.int64)]).astype(np.int32)
    vals = rng.uniform(-1, 1, int(ptr[-1]) * V).astype(np.float16)
    return ptr, col, vals


def call_noalloc(lib, ptr, col, vals, rhs, V, out):
    m_vec = ptr.numel() - 1
    K, N = rhs.shape
    return lib.sspmm_f16_f16_noalloc(m_vec, V, N, K, None, ptr.data_ptr(), col.data_ptr(), vals.data_ptr(),
                                     rhs.data_ptr(), out.data_ptr(), torch.cuda.current_stream().cuda_stream)


def assert_same(got, ref):
    """Tolerance of the SpMM parity tests: 1e-2 relative with a per-row floor, relative RMS <= 2e-3."""
    got = got.float().cpu().numpy().astype(np.float64)
    ref = ref.float().cpu().numpy().astype(np.float64)
    assert np.isfinite(got).all()
    floor = 1e-3 * np.max(np.abs(ref), axis=1, keepdims=True) + 1e-30
    err = np.abs(got - ref) / np.maximum(np.abs(ref), floor)
    assert err.max() <= 1e-2, f"max rel err {err.max():.3e}"
    rms = np.sqrt(np.mean((got - ref) ** 2)) / (np.sqrt(np.mean(ref ** 2)) + 1e-30)
    assert rms <= 2e-3, f"relative RMS error {rms:.3e}"


@pytest.mark.gpu
def test_noalloc_matches_regular_entry_point_on_two_calls_in_a_row(lib):
    torch.cuda.set_device(0)
    cases = [
        # (seed, m_vec, K, V, density, N): the second problem is smaller and differently shaped, so stale
        # contents of the shared scratch would show up if they were ever read
        (1, 64, 1000, 16, 0.4, 264),
        (2, 24, 520, 8, 0.15, 136),
    ]
    prepared = []
    for seed, m_vec, K, V, density, N in cases:
        ptr, col, vals = random_cvse(seed, m_vec, K, V, density)
        rhs = np.random.default_rng(100 + seed).normal(0, 1, (K, N)).astype(np.float16)
        t = [torch.from_numpy(x).to(DEV) for x in (ptr, col, vals, rhs)]
        ref = ops.sspmm(t[0], t[1], t[2], t[3], V, out_dtype=torch.float16)      # existing entry point
        prepared.append((t, V, ref))
    torch.cuda.synchronize()
    outs = []
    for t, V, ref in prepared:                                                  # two calls in a row, one stream
        out = torch.full_like(ref, float("nan"))
        rc = call_noalloc(lib, t[0], t[1], t[2], t[3], V, out)
        assert rc == 0, lib.sspmm_last_error_string().decode()
        outs.append(out)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for out, (_, _, ref) in zip(outs, prepared):
        assert_same(out, ref)
    # and once more in the opposite order
    for (t, V, ref) in reversed(prepared):
        out = torch.full_like(ref, float("nan"))
        assert call_noalloc(lib, t[0], t[1], t[2], t[3], V, out) == 0
        torch.cuda.synchronize()
        assert_same(out, ref)
    # "allocates nothing": after these warm calls, further calls leave the device's free memory and the default
    # stream-ordered pool (the allocator the regular entry points use) exactly as they were
    from cuda.bindings import runtime as cudart
    err, pool = cudart.cudaDeviceGetDefaultMemPool(0)
    assert err == cudart.cudaError_t.cudaSuccess

    def pool_state():
        vals = []
        for attr in (cudart.cudaMemPoolAttr.cudaMemPoolAttrReservedMemCurrent, cudart.cudaMemPoolAttr.cudaMemPoolAttrUsedMemCurrent):
            e, v = cudart.cudaMemPoolGetAttribute(pool, attr)
            assert e == cudart.cudaError_t.cudaSuccess
            vals.append(int(v))
        return vals

    outs = [torch.full_like(ref, float("nan")) for (_, _, ref) in prepared]
    torch.cuda.synchronize()
    before_pool, before_free = pool_state(), torch.cuda.mem_get_info()[0]
    for _ in range(3):
        for out, (t, V, ref) in zip(outs, prepared):
            assert call_noalloc(lib, t[0], t[1], t[2], t[3], V, out) == 0
    torch.cuda.synchronize()
    assert pool_state() == before_pool
    assert torch.cuda.mem_get_info()[0] == before_free


def test_noalloc_rejects_what_does_not_fit(lib):
    """Size and shape checks happen before any CUDA call, so this part needs no GPU."""
    dummy = C.c_void_p(256)                 # never dereferenced: the call is rejected first
    # 2 * K * m_vec * V bytes just above the limit
    m_vec, V = 128, 16
    K = MAX_SCRATCH // (2 * m_vec * V) + 1
    rc = lib.sspmm_f16_f16_noalloc(m_vec, V, 64, K, None, dummy, dummy, dummy, dummy, dummy, None)
    assert rc == 1
    msg = lib.sspmm_last_error_string().decode()
    assert "exceeds the fixed scratch" in msg and str(MAX_SCRATCH) in msg
    assert lib.sspmm_f16_f16_noalloc(4, 12, 64, 64, None, dummy, dummy, dummy, dummy, dummy, None) == 1
    assert lib.sspmm_f16_f16_noalloc(4, 8, 50, 64, None, dummy, dummy, dummy, dummy, dummy, None) == 1     # N % 8
    assert "N % 8" in lib.sspmm_last_error_string().decode()
    assert lib.sspmm_f16_f16_noalloc(0, 8, 64, 64, None, None, None, None, None, None, None) == 0        # empty
