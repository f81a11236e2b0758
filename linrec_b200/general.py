"""The wider signature of the reference's Python operator, `linrec(inputs, coeffs, logc=False,
dim=-1, reverse=False)` (linrec/impl/python/ops.py:8-61), on top of the CUDA scan.

`dim`   the scan runs along `dim`; other than the last dimension this costs a transposed copy in and
        out (the kernels scan contiguous rows).
`logc`  coefficients are given as logarithms: c = exp(coeffs).  The gradient with respect to the
        logarithm is d_coeffs * c.  (The reference's own backward multiplies by the SHIFTED
        coefficients, linrec/impl/python/ops.py:33-38, which is not the derivative of its forward;
        this implementation follows the forward.)
Both are compositions around the scan operator, so autograd needs nothing extra.
"""
from __future__ import annotations

import torch

from .ops import linrec_pipe

__all__ = ["linrec_general"]


def linrec_general(inputs: torch.Tensor, coeffs: torch.Tensor, logc: bool = False, dim: int = -1,
                   reverse: bool = False) -> torch.Tensor:
    if logc:
        coeffs = torch.exp(coeffs)
    last = inputs.dim() - 1
    d = dim % inputs.dim() if inputs.dim() else 0
    if d != last:
        x = inputs.transpose(d, last).contiguous()
        c = coeffs.transpose(d, last).contiguous()
        return linrec_pipe(x, c, reverse).transpose(d, last)
    if coeffs.stride() != inputs.stride():
        coeffs = torch.empty_like(inputs).copy_(coeffs)
    return linrec_pipe(inputs, coeffs, reverse)
