"""Encoder layer with pruned, SVC-compressed weights against the same layer evaluated with dense
matrices (torch.matmul on the densified pruned weights)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sparse_encoder_layer_matches_dense_evaluation(lib):
    from sspmm_b200.encoder import SparseEncoderLayer
    torch.manual_seed(0)
    layer = SparseEncoderLayer(hidden=256, ffn=1024, heads=4, sparsity=0.9, vec_length=16)
    batch, seq = 4, 128
    x = torch.randn(256, batch * seq, device="cuda:0", dtype=torch.float16)
    y_sparse = layer.forward(x, batch, seq)
    y_dense = layer.forward(x, batch, seq, dense=True)
    torch.cuda.synchronize()
    assert y_sparse.shape == (256, batch * seq) and torch.isfinite(y_sparse).all()
    err = (y_sparse.float() - y_dense.float()).abs().max().item()
    scale = y_dense.float().abs().max().item()
    assert err <= 2e-2 * scale, (err, scale)
    rms = ((y_sparse.float() - y_dense.float()).pow(2).mean().sqrt() / y_dense.float().pow(2).mean().sqrt()).item()
    assert rms < 5e-3
