"""The bounded device-side waits, made to run out on purpose -- without a fault, a trap or an endless
loop: a one-thread kernel waits on an mbarrier that nobody arrives at, with the cycle budget shortened
to about a millisecond for that launch.  The wait must give up, the kernel must return normally, the
status word must carry the code, reading it must clear it, and the next regular call must work."""
import ctypes as C
import time

import numpy as np
import pytest
import torch

from oracle import spmm_oracle
from sspmm_b200 import ops

DEV = "cuda:0"
STATUS_SELFTEST = 6


@pytest.mark.gpu
def test_wait_gives_up_and_context_stays_usable(lib):
    torch.cuda.set_device(0)
    assert ops.device_status() == 0
    gave_up = C.c_int(-1)
    t0 = time.perf_counter()
    rc = lib.sspmm_selftest_wait_expiry(2_000_000, C.byref(gave_up))       # about 1 ms at 2 GHz
    dt = time.perf_counter() - t0
    assert rc == 0, lib.sspmm_last_error_string().decode()
    assert gave_up.value == 1
    assert dt < 1.0, f"the shortened wait took {dt:.3f} s"
    assert ops.device_status() == STATUS_SELFTEST
    assert ops.device_status() == 0                                        # reading cleared it
    # the context is healthy: a regular product still matches the oracle
    rng = np.random.default_rng(3)
    lens = [5, 0, 40, 17]
    ptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    col = np.concatenate([rng.permutation(64)[:l] for l in lens]).astype(np.int32)
    vals = rng.uniform(-1, 1, int(ptr[-1]) * 8).astype(np.float16)
    rhs = rng.normal(0, 1, (64, 128)).astype(np.float16)
    out = ops.sspmm(torch.from_numpy(ptr).to(DEV), torch.from_numpy(col).to(DEV), torch.from_numpy(vals).to(DEV),
                    torch.from_numpy(rhs).to(DEV), 8, out_dtype=torch.float32)
    torch.cuda.synchronize()
    ref = spmm_oracle.sspmm_host(8, ptr, col, vals, rhs)
    assert np.allclose(out.cpu().numpy(), ref, rtol=1e-3, atol=1e-3)
    assert ops.device_status() == 0


def test_selftest_rejects_bad_limits(lib):
    g = C.c_int(0)
    assert lib.sspmm_selftest_wait_expiry(0, C.byref(g)) == 1
    assert lib.sspmm_selftest_wait_expiry(2_000_000, None) == 1
