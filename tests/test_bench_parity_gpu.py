"""Parity of everything the benchmark times, at the benchmark's own sizes, against the CPU oracle
(oracle/spmm_host.c, the restatement of SSpMM/sspmm_test.cpp:75-95, and oracle/svc_oracle.py, the
restatement of RowMerge/sparse_matrix_format.py:94-123): all 32 conv products as one group at the
8-GPU shard width and at full width, the encoder layer at its stated size, and the long vector rows of
the largest sweep matrix.  The CPU computes sampled vector rows only (the full products would take
minutes); tolerances are those of test_spmm_gpu.py."""
import numpy as np
import pytest
import torch

from oracle import spmm_oracle, svc_oracle
from sspmm_b200 import ops, synthetic
from tests.test_spmm_gpu import assert_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def conv_products():
    return [(l, s, V) for s in range(len(synthetic.CONV_SPARSITIES)) for V in (8, 16) for l in range(len(synthetic.CONV_LAYERS))]


@pytest.mark.parametrize("N", [3136, 25088])
def test_all_conv_products_as_one_group(lib, N):
    """The benchmark step: 32 products (8 layers x 2 sparsities x V 8/16) in one group run, operands
    compressed by the GPU SVC.  Every product: SVC structure bit-equal to the oracle's, two sampled vector rows
    (first and last) of the result against the oracle over all N columns."""
    torch.cuda.set_device(0)
    rng = np.random.default_rng(2025)
    host_B, dev_B, cache = {}, {}, {}
    prods = []
    for (l, s, V) in conv_products():
        if (l, s) not in cache:
            cache[(l, s)] = synthetic.conv_weight(l, s)
        a = cache[(l, s)]
        if a.K not in host_B:
            host_B[a.K] = rng.normal(0, 1, (a.K, N)).astype(np.float16)
            dev_B[a.K] = torch.from_numpy(host_B[a.K]).to(DEV)
        vp, vc, vv, _ = ops.svc(torch.from_numpy(a.row_ptr).to(DEV), torch.from_numpy(a.col_idx).to(DEV),
                                torch.from_numpy(a.values).to(DEV), a.M, a.K, V)
        plan = ops.Plan(vp, vc, V, a.K)
        assert plan.one_launch
        out = torch.full(((vp.numel() - 1) * V, N), float("nan"), dtype=torch.float16, device=DEV)
        prods.append(dict(a=a, V=V, vp=vp, vc=vc, vv=vv, plan=plan, out=out))
    group = ops.Group([(p["plan"], p["vv"], dev_B[p["a"].K], p["out"]) for p in prods])
    group.run()
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    for p in prods:
        a, V = p["a"], p["V"]
        r = svc_oracle.cvse(a.M, a.K, a.nnz, a.row_lists(), V)
        ptr, col = p["vp"].cpu().numpy(), p["vc"].cpu().numpy()
        assert ptr.tolist() == r.vec_row_ptr and col.tolist() == r.vec_colInd_list
        vals = p["vv"].cpu().numpy()
        m_vec = ptr.size - 1
        got = p["out"]
        assert torch.isfinite(got).all()
        for rows in ((0, 1), (m_vec - 1, m_vec)):
            ref = spmm_oracle.sspmm_host(V, ptr, col, vals, host_B[a.K], rows=rows, threads=8)
            assert_close(got[rows[0] * V: rows[1] * V].float().cpu().numpy(), ref)


def test_encoder_layer_at_stated_size(lib):
    """hidden 768, FFN 3072, 12 heads, seq 512, batch 32: every linear of the grouped forward pass against the oracle
    on sampled vector rows (its input taken from the layer's own activation buffer), and the whole layer against
    the dense evaluation."""
    from sspmm_b200.encoder import SparseEncoderLayer
    torch.manual_seed(0)
    layer = SparseEncoderLayer(hidden=768, ffn=3072, heads=12, sparsity=0.9, vec_length=16, device=DEV)
    batch, seq = 32, 512
    x = torch.randn(768, batch * seq, device=DEV, dtype=torch.float16)
    y = layer.forward_grouped(x, batch, seq)
    torch.cuda.synchronize()
    assert ops.device_status() == 0
    assert layer.groups is not None
    b = layer.buf
    pairs = [(0, "ln1", "q"), (1, "ln1", "k"), (2, "ln1", "v"), (3, "att", "o"), (4, "ln2", None), (5, "h", "y")]
    for i, src, dst in pairs:
        lin = layer.linears[i]
        ptr, col, vals = lin.row_offsets.cpu().numpy(), lin.col.cpu().numpy(), lin.values.cpu().numpy()
        rhs = b[src].cpu().numpy()
        if dst is None:
            # FFN1 writes "h", which then receives its bias in place: recompute the product alone
            got_full = ops.sspmm_planned(lin.plan, lin.values, b[src])
        else:
            got_full = b[dst]
        m_vec = ptr.size - 1
        for rows in ((0, 1), (m_vec // 2, m_vec // 2 + 1)):
            ref = spmm_oracle.sspmm_host(16, ptr, col, vals, rhs, rows=rows, threads=8)
            assert_close(got_full[rows[0] * 16: rows[1] * 16].float().cpu().numpy(), ref)
    y_dense = layer.forward(x, batch, seq, dense=True)
    err = (y.float() - y_dense.float()).abs().max().item()
    scale = y_dense.float().abs().max().item()
    assert err <= 2e-2 * scale, (err, scale)


def test_svc_long_vector_rows_of_the_largest_sweep_size(lib):
    """n = 65536 power-law matrix, V = 8: the vector rows with the most columns (the ones that take the
    hash-order replay with large tables) and a random sample of the others, column order included, against the
    oracle run on exactly those row groups."""
    a = synthetic.power_law(65536, np.random.default_rng(2024))
    V = 8
    d = lambda t: torch.from_numpy(t).to(DEV)
    vp, vc, vv, replayed = ops.svc(d(a.row_ptr), d(a.col_idx), d(a.values), a.M, a.K, V)
    ptr, col, val = vp.cpu().numpy(), vc.cpu().numpy(), vv.cpu().numpy()
    assert replayed > 0
    lens = np.diff(ptr)
    longest = np.argsort(-lens)[:24]
    rng = np.random.default_rng(7)
    sample = np.unique(np.concatenate([longest, rng.integers(0, lens.size, 200)]))
    for i in sample.tolist():
        r0, r1 = i * V, min(i * V + V, a.M)
        rows = [a.col_idx[a.row_ptr[r]:a.row_ptr[r + 1]].tolist() for r in range(r0, r1)]
        nnz = int(a.row_ptr[r1] - a.row_ptr[r0])
        r = svc_oracle.cvse(r1 - r0, a.K, nnz, rows, V)
        assert col[ptr[i]:ptr[i + 1]].tolist() == r.vec_colInd_list, f"vector row {i} ({lens[i]} columns)"
        sub_ptr = (a.row_ptr[r0:r1 + 1] - a.row_ptr[r0]).astype(np.int32)
        packed = svc_oracle.pack_values(r1 - r0, V, sub_ptr, a.col_idx[a.row_ptr[r0]:a.row_ptr[r1]], a.values[a.row_ptr[r0]:a.row_ptr[r1]], r)
        assert np.array_equal(val[ptr[i] * V: ptr[i + 1] * V].view(np.uint16), np.asarray(packed).view(np.uint16))
    assert lens[longest[0]] > 4914            # the sample reaches the classes with tables beyond shared-memory lists


def test_workspace_entry_point_matches_regular(lib):
    """sspmm_f16_f16_ws (caller-owned scratch, vector count passed in) against sspmm_f16_f16 on a sweep matrix
    (row-gather kernel, long rows split) and on a dense-ish one (block kernel), and its size checks."""
    for a, V, N in ((synthetic.sweep_matrix(3), 8, 128), (synthetic.conv_weight(1, 0), 16, 200)):
        d = lambda t: torch.from_numpy(t).to(DEV)
        vp, vc, vv, _ = ops.svc(d(a.row_ptr), d(a.col_idx), d(a.values), a.M, a.K, V)
        rhs = torch.randn(a.K, N, device=DEV, dtype=torch.float16)
        ref = ops.sspmm(vp, vc, vv, rhs, V)
        need = ops.workspace_bytes(vp.numel() - 1, V, N, a.K, vc.numel())
        ws = torch.empty(max(need, 256), dtype=torch.uint8, device=DEV)
        got = ops.sspmm_ws(vp, vc, vv, rhs, V, vc.numel(), ws)
        torch.cuda.synchronize()
        assert_close(got.float().cpu().numpy(), ref.float().cpu().numpy())
        # without scratch the sparse operand still works (rows are not split); the dense-ish one is rejected
        if need == 0 or V == 8:
            got2 = ops.sspmm_ws(vp, vc, vv, rhs, V, vc.numel(), None)
            torch.cuda.synchronize()
            assert_close(got2.float().cpu().numpy(), ref.float().cpu().numpy())
        else:
            with pytest.raises(Exception):
                ops.sspmm_ws(vp, vc, vv, rhs, V, vc.numel(), None)
    assert ops.device_status() == 0
