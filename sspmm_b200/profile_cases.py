"""Small, fixed workloads for profiler captures (one kernel, a few launches, inputs larger than L2
where bandwidth matters).

    python -m sspmm_b200.profile_cases gather_powerlaw      # gather SpMM, power-law n=65536, N=1024
    python -m sspmm_b200.profile_cases gather_conv          # gather SpMM forced on conv (2048,512) s=0.9 V=16
    python -m sspmm_b200.profile_cases svc_powerlaw         # SVC of a power-law n=65536 matrix
    python -m sspmm_b200.profile_cases block_conv_shard     # block SpMM, conv (512,4608) s=0.8 V=8 at the
                                                            # 8-GPU shard width N=3136 (L2 flushed between launches)
"""
from __future__ import annotations

import sys

import numpy as np
import torch

from . import ops, synthetic


def _dev(a):
    d = "cuda:0"
    return torch.from_numpy(a.row_ptr).to(d), torch.from_numpy(a.col_idx).to(d), torch.from_numpy(a.values).to(d)


def main(case: str) -> None:
    if case == "svc_powerlaw":
        a = synthetic.power_law(65536, np.random.default_rng(65536))
        p, c, v = _dev(a)
        for _ in range(3):
            ops.svc(p, c, v, a.M, a.K, 8)
    elif case in ("gather_powerlaw", "gather_conv"):
        if case == "gather_powerlaw":
            a, V, N = synthetic.power_law(65536, np.random.default_rng(65536)), 8, 1024
        else:
            a, V, N = synthetic.conv_weight(7, 1), 16, synthetic.CONV_N
        p, c, v = _dev(a)
        vp, vc, vv, _ = ops.svc(p, c, v, a.M, a.K, V)
        rhs = torch.randn(a.K, N, device="cuda:0", dtype=torch.float16)
        out = torch.empty((vp.numel() - 1) * V, N, device="cuda:0", dtype=torch.float16)
        ops.set_kernel(ops.KERNEL_GATHER_LSU)
        for _ in range(4):
            ops.sspmm(vp, vc, vv, rhs, V, out=out)
        ops.set_kernel(ops.KERNEL_AUTO)
    elif case == "block_conv_shard":
        a, V, N = synthetic.conv_weight(3, 0), 8, synthetic.CONV_N // 8
        p, c, v = _dev(a)
        vp, vc, vv, _ = ops.svc(p, c, v, a.M, a.K, V)
        rhs = torch.randn(a.K, N, device="cuda:0", dtype=torch.float16)
        out = torch.empty((vp.numel() - 1) * V, N, device="cuda:0", dtype=torch.float16)
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda:0")
        ops.set_kernel(ops.KERNEL_BLOCK)
        for _ in range(4):
            flush.zero_()
            ops.sspmm(vp, vc, vv, rhs, V, out=out)
        ops.set_kernel(ops.KERNEL_AUTO)
    else:
        raise SystemExit(__doc__)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    print("done", case)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "")
