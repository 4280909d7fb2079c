"""Transformer encoder layer whose six weight matrices (Q, K, V, O, FFN1, FFN2) are magnitude-pruned,
compressed by the GPU SVC and applied with the vector-sparse SpMM; attention itself and LayerNorm
stay dense PyTorch ops.

Block structure follows the reference's end-to-end script (end2end/sspmm_e2e/end_to_end.py:44-75:
LayerNorm -> attention -> residual -> LayerNorm -> linear1 -> linear2 -> residual, no activation
between the two linears), with the sparsity moved from the attention mask to the weights.

Activations are kept feature-major, x[features, tokens], because the SpMM computes
C[out_features, tokens] = W_vs[out_features, in_features] . B[in_features, tokens] with B row-major."""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch
import torch.nn.functional as F

from . import ops, synthetic


class SparseLinear:
    """y[out, tokens] = W_vs . x[in, tokens] + b, W pruned and held in the compressed format."""

    def __init__(self, weight: synthetic.CSR, vec_length: int, device, bias: Optional[torch.Tensor] = None):
        self.out_features, self.in_features, self.V = weight.M, weight.K, vec_length
        self.nnz = weight.nnz
        d = lambda a: torch.from_numpy(a).to(device)
        self.row_offsets, self.col, self.values, _ = ops.svc(d(weight.row_ptr), d(weight.col_idx), d(weight.values),
                                                             weight.M, weight.K, vec_length)
        self.row_indices = ops.sorted_row_swizzle(self.row_offsets)
        self.plan = ops.Plan(self.row_offsets, self.col, vec_length, weight.K)
        self.bias = bias
        self.dense = torch.from_numpy(weight.dense()).to(device)          # only for the dense comparison

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        y = ops.sspmm(self.row_offsets, self.col, self.values, x, self.V, row_indices=self.row_indices)
        y = y[: self.out_features]
        return y if self.bias is None else y + self.bias[:, None]

    def dense_forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.dense @ x
        return y if self.bias is None else y + self.bias[:, None]


class SparseEncoderLayer:
    def __init__(self, hidden=768, ffn=3072, heads=12, sparsity=0.9, vec_length=16, device="cuda:0", seed=400):
        self.hidden, self.ffn, self.heads, self.dev = hidden, ffn, heads, torch.device(device)
        shapes = [(hidden, hidden)] * 4 + [(ffn, hidden), (hidden, ffn)]
        self.linears = []
        g = torch.Generator(device="cpu").manual_seed(seed)
        for i, (m, k) in enumerate(shapes):
            w = synthetic.magnitude_pruned(m, k, sparsity, np.random.default_rng(seed + i))
            b = (0.02 * torch.randn(m, generator=g)).to(torch.float16).to(self.dev)
            self.linears.append(SparseLinear(w, vec_length, self.dev, b))
        self.ln1 = (torch.ones(hidden, dtype=torch.float16, device=self.dev), torch.zeros(hidden, dtype=torch.float16, device=self.dev))
        self.ln2 = (torch.ones(hidden, dtype=torch.float16, device=self.dev), torch.zeros(hidden, dtype=torch.float16, device=self.dev))

    @staticmethod
    def _layer_norm_fm(x, wb, eps=1e-5):
        xf = x.float()
        mu = xf.mean(dim=0, keepdim=True)
        var = xf.var(dim=0, unbiased=False, keepdim=True)
        return (((xf - mu) * torch.rsqrt(var + eps)) * wb[0].float()[:, None] + wb[1].float()[:, None]).to(x.dtype)

    def _attention(self, q, k, v, batch, seq):
        h, hd = self.heads, self.hidden // self.heads
        def split(t):            # [hidden, batch*seq] -> [batch, heads, seq, head_dim]
            return t.view(h, hd, batch, seq).permute(2, 0, 3, 1)
        o = F.scaled_dot_product_attention(split(q), split(k), split(v))
        return o.permute(1, 3, 0, 2).reshape(self.hidden, batch * seq)

    def _groups_for(self, tokens: int):
        """Activation buffers of fixed shape and, bound to them, one group per dependency level of the layer:
        {Q, K, V} share their input and run as one launch, then O, FFN1, FFN2."""
        if getattr(self, "_tokens", None) == tokens:
            return
        z = lambda rows: torch.empty((rows, tokens), dtype=torch.float16, device=self.dev)
        b = self.buf = {"ln1": z(self.hidden), "q": z(self.hidden), "k": z(self.hidden), "v": z(self.hidden),
                        "att": z(self.hidden), "o": z(self.hidden), "ln2": z(self.hidden), "h": z(self.ffn), "y": z(self.hidden)}
        L = self.linears
        item = lambda l, src, dst: (l.plan, l.values, b[src], b[dst])
        self.groups = None
        if all(l.plan.one_launch and l.out_features % l.V == 0 for l in L):
            self.groups = [ops.Group([item(L[0], "ln1", "q"), item(L[1], "ln1", "k"), item(L[2], "ln1", "v")]),
                           ops.Group([item(L[3], "att", "o")]), ops.Group([item(L[4], "ln2", "h")]),
                           ops.Group([item(L[5], "h", "y")])]
        self._tokens = tokens

    def forward_grouped(self, x: torch.Tensor, batch: int, seq: int) -> torch.Tensor:
        """Same layer with the linears run as groups (sspmm_group_run) on preallocated activation buffers."""
        self._groups_for(batch * seq)
        if self.groups is None:
            return self.forward(x, batch, seq)
        b, L, g = self.buf, self.linears, self.groups
        b["ln1"].copy_(self._layer_norm_fm(x, self.ln1))
        g[0].run()
        q, k, v = (b[n] + L[i].bias[:, None] for i, n in enumerate(("q", "k", "v")))
        b["att"].copy_(self._attention(q, k, v, batch, seq))
        g[1].run()
        out = b["o"] + L[3].bias[:, None] + x
        b["ln2"].copy_(self._layer_norm_fm(out, self.ln2))
        g[2].run()
        b["h"] += L[4].bias[:, None]
        g[3].run()
        return b["y"] + L[5].bias[:, None] + out

    def forward(self, x: torch.Tensor, batch: int, seq: int, dense: bool = False) -> torch.Tensor:
        """x: [hidden, batch*seq] fp16, feature-major (token t of sequence b is column b*seq + t)."""
        lin = [(l.dense_forward if dense else l) for l in self.linears]
        out = self._layer_norm_fm(x, self.ln1)
        q, k, v = lin[0](out), lin[1](out), lin[2](out)
        att = lin[3](self._attention(q, k, v, batch, seq).contiguous())
        out = att + x
        y = self._layer_norm_fm(out, self.ln2)
        y = lin[5](lin[4](y))
        return y + out
