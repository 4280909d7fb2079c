"""GPU parity tests of the one-launch SpMM (plans and groups), called through the C ABI, against the CPU
oracle (fp32 restatement of the reference's host loop, SSpMM/sspmm_test.cpp:75-95).  Tolerances are the
ones of test_spmm_gpu.py."""
import numpy as np
import pytest
import torch

from oracle import spmm_oracle
from sspmm_b200 import ops, synthetic
from tests.test_spmm_gpu import assert_close, compress, random_cvse

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(*arrays):
    return [torch.from_numpy(np.ascontiguousarray(a)).to(DEV) for a in arrays]


def planned(ptr, col, vals, rhs, V, out_dtype):
    d_ptr, d_col, d_val, d_rhs = dev(ptr, col, vals, rhs)
    plan = ops.Plan(d_ptr, d_col, V, rhs.shape[0])
    out = ops.sspmm_planned(plan, d_val, d_rhs, out_dtype=out_dtype)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    return plan, out.float().cpu().numpy()


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("V", [8, 16])
def test_config1_planned(lib, V, out_dtype):
    a, rhs = synthetic.config1()
    ptr, col, vals = compress(a, V)
    ref = spmm_oracle.sspmm_host(V, ptr, col, vals, rhs)
    plan, got = planned(ptr, col, vals, rhs, V, out_dtype)
    assert plan.one_launch and plan.ascending and plan.nvec == col.size
    assert_close(got, ref, fp32=out_dtype == torch.float32)


@pytest.mark.parametrize("shape_id", [0, 1])
@pytest.mark.parametrize("sparsity_id", [0, 1, 2, 3, 4, 5])
def test_ffn_v16_planned_and_grouped(lib, shape_id, sparsity_id):
    """All twelve FFN cases: the planned call (static tiles) and a group of one (queue, K cut into parts)."""
    a, rhs = synthetic.ffn(shape_id, sparsity_id)
    ptr, col, vals = compress(a, 16)
    ref = spmm_oracle.sspmm_host(16, ptr, col, vals, rhs, threads=8)
    plan, got = planned(ptr, col, vals, rhs, 16, torch.float16)
    if not plan.one_launch:
        assert col.size < ptr.size * a.K / 16          # only very sparse structures are left to the gather kernels
    assert_close(got, ref)
    if plan.one_launch:
        d_val, d_rhs = dev(vals, rhs)
        for dt, mode in ((torch.float16, ops.Group.COMPRESSED), (torch.float32, ops.Group.COMPRESSED), (torch.float16, ops.Group.EXPANDED),
                         (torch.float16, ops.Group.PAIRS), (torch.float32, ops.Group.PAIRS)):
            out = torch.full((a.M, rhs.shape[1]), float("nan"), dtype=dt, device=DEV)
            g = ops.Group([(plan, d_val, d_rhs, out)], mode=mode)
            assert g.launches == 1
            for _ in range(3):                         # the queue and the arrival counters reset themselves
                out.fill_(float("nan"))
                g.run()
            torch.cuda.synchronize()
            assert ops.device_status() == 0
            assert_close(out.float().cpu().numpy(), ref, fp32=dt == torch.float32)


@pytest.mark.parametrize("V", [8, 16])
@pytest.mark.parametrize("N", [8, 64, 72, 136, 200, 256, 520])
def test_ragged_unsorted_rows_and_tails(lib, V, N):
    """Unsorted column lists (the permutation path), empty rows, a partial last row tile, K and N tails."""
    rng = np.random.default_rng(300 + N + V)
    lens = [0, 1, 2, 3, 15, 16, 17, 31, 33, 63, 64, 65, 0, 127, 129, 200, 0, 70, 5]
    K = 300
    ptr, col, vals = random_cvse(rng, len(lens), K, V, lens)
    rhs = rng.normal(0, 1, (K, N)).astype(np.float16)
    ref = spmm_oracle.sspmm_host(V, ptr, col, vals, rhs)
    for dt in (torch.float32, torch.float16):
        plan, got = planned(ptr, col, vals, rhs, V, dt)
        assert plan.one_launch and not plan.ascending
        assert_close(got, ref, fp32=dt == torch.float32)


def test_irregular_structure_falls_back(lib):
    """A column listed twice in a vector row: the plan carries no metadata and the call still gives the
    reference's answer (both vectors count), through the regular entry point."""
    ptr = np.array([0, 3, 5], dtype=np.int32)
    col = np.array([4, 9, 4, 0, 63], dtype=np.int32)
    rng = np.random.default_rng(5)
    vals = rng.uniform(-1, 1, 5 * 8).astype(np.float16)
    rhs = rng.normal(0, 1, (64, 64)).astype(np.float16)
    ref = spmm_oracle.sspmm_host(8, ptr, col, vals, rhs)
    plan, got = planned(ptr, col, vals, rhs, 8, torch.float32)
    assert not plan.one_launch
    assert_close(got, ref, fp32=True)
    d_val, d_rhs = dev(vals, rhs)
    with pytest.raises(Exception):
        ops.Group([(plan, d_val, d_rhs, torch.empty((16, 64), dtype=torch.float16, device=DEV))])


@pytest.mark.parametrize("mode", [ops.Group.COMPRESSED, ops.Group.EXPANDED, ops.Group.PAIRS])
def test_group_of_mixed_products(lib, mode):
    """Products of different shapes, V = 8 and 16, K from 64 to 2304, column counts with partial tiles, in one
    group (A tiles built in the kernel, or fetched from dense copies written at every run); every product against
    the oracle; replays give bit-identical results."""
    rng = np.random.default_rng(77)
    shapes = [(256, 2304, 16, 0.9, 1000), (64, 576, 8, 0.8, 1000), (512, 128, 16, 0.8, 1000), (256, 64, 8, 0.9, 1000),
              (1024, 256, 8, 0.9, 328), (128, 1152, 16, 0.8, 328)]
    prods, refs = [], []
    for (M, K, V, s, N) in shapes:
        a = synthetic.magnitude_pruned(M, K, s, rng)
        ptr, col, vals = compress(a, V)
        rhs = rng.normal(0, 1, (K, N)).astype(np.float16)
        d_ptr, d_col, d_val, d_rhs = dev(ptr, col, vals, rhs)
        plan = ops.Plan(d_ptr, d_col, V, K)
        assert plan.one_launch
        out = torch.full((M, N), float("nan"), dtype=torch.float16, device=DEV)
        prods.append((plan, d_val, d_rhs, out))
        refs.append(spmm_oracle.sspmm_host(V, ptr, col, vals, rhs, threads=8))
    g = ops.Group(prods, mode=mode)
    g.run()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    first = [p[3].clone() for p in prods]
    for (plan, _, _, out), ref in zip(prods, refs):
        assert_close(out.float().cpu().numpy(), ref)
    for _ in range(2):
        for p in prods:
            p[3].fill_(float("nan"))
        g.run()
        torch.cuda.synchronize()
        for p, f in zip(prods, first):
            assert torch.equal(p[3], f)
    assert ops.device_status() == 0


@pytest.mark.parametrize("N", [3136, 25088])
def test_conv_layer_planned_wide(lib, N):
    """Conv layer (512, 4608) at the 8-GPU shard width and at full width: planned call and group against the
    oracle on sampled vector rows, and against each other everywhere."""
    a = synthetic.conv_weight(3, 1)
    V = 16
    ptr, col, vals = compress(a, V)
    rng = np.random.default_rng(15)
    rhs = rng.normal(0, 1, (a.K, N)).astype(np.float16)
    d_ptr, d_col, d_val, d_rhs = dev(ptr, col, vals, rhs)
    plan = ops.Plan(d_ptr, d_col, V, a.K)
    assert plan.one_launch
    got = ops.sspmm_planned(plan, d_val, d_rhs)
    out = torch.full_like(got, float("nan"))
    out2 = torch.full_like(got, float("nan"))
    g = ops.Group([(plan, d_val, d_rhs, out)], mode=ops.Group.COMPRESSED)
    g2 = ops.Group([(plan, d_val, d_rhs, out2)], mode=ops.Group.EXPANDED)
    out3 = torch.full_like(got, float("nan"))
    g3 = ops.Group([(plan, d_val, d_rhs, out3)], mode=ops.Group.PAIRS)
    g.run()
    g2.run()
    g3.run()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    a_np, b_np = got.float().cpu().numpy(), out.float().cpu().numpy()
    assert_close(b_np, a_np)
    assert_close(out2.float().cpu().numpy(), a_np)
    assert_close(out3.float().cpu().numpy(), a_np)
    for rows in ((0, 2), (15, 17), (a.M // V - 2, a.M // V)):
        ref = spmm_oracle.sspmm_host(V, ptr, col, vals, rhs, rows=rows, threads=8)
        assert_close(a_np[rows[0] * V: rows[1] * V], ref)
        assert_close(b_np[rows[0] * V: rows[1] * V], ref)
