"""Operator namespace of the reference's PyTorch extension (`sptrans`), SpMM part only."""
