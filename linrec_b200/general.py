"""The wider signature of the reference's Python operator, `linrec(inputs, coeffs, logc=False,
dim=-1, reverse=False)` (linrec/impl/python/ops.py:8-61), on top of the CUDA scan.

`dim`   the scan runs along `dim`.  For a dimension other than the last, dense 16-byte aligned
        tensors whose trailing extent is a whole number of 16-byte chunks are scanned where they lie
        (a kernel that walks down the axis, neighbouring channels on neighbouring threads), unless
        there are only a handful of columns; anything else costs a transposed copy in and out.
`logc`  coefficients are given as logarithms: c = exp(coeffs).  The gradient with respect to the
        logarithm is d_coeffs * c.  (The reference's own backward multiplies by the SHIFTED
        coefficients, linrec/impl/python/ops.py:33-38, which is not the derivative of its forward;
        this implementation follows the forward.)
Both are compositions around the scan operator, so autograd needs nothing extra.
"""
from __future__ import annotations

import torch

from .ops import dim_eligible, dim_worthwhile, linrec_dim_bwd, linrec_dim_fwd, linrec_pipe

__all__ = ["linrec_general"]


class _LinrecDimFn(torch.autograd.Function):
    """Scan along a non-last dimension of dense tensors; same saved tensors and gradient formulas
    as the last-dimension operator (linrec/impl/cuda/ops.py:17-21,54-59)."""

    @staticmethod
    def forward(ctx, inputs, coeffs, dim, reverse):
        outputs = linrec_dim_fwd(inputs, coeffs, dim, reverse)
        ctx.save_for_backward(coeffs, outputs)
        ctx.dim, ctx.reverse = dim, reverse
        return outputs

    @staticmethod
    def backward(ctx, d_outputs):
        coeffs, outputs = ctx.saved_tensors
        d_outputs = d_outputs.contiguous()
        if not dim_eligible(d_outputs, ctx.dim):
            d_outputs = d_outputs.clone(memory_format=torch.contiguous_format)
        d_inputs, d_coeffs = linrec_dim_bwd(d_outputs, coeffs, outputs, ctx.dim, ctx.reverse)
        return d_inputs, d_coeffs, None, None


def linrec_general(inputs: torch.Tensor, coeffs: torch.Tensor, logc: bool = False, dim: int = -1,
                   reverse: bool = False) -> torch.Tensor:
    if logc:
        coeffs = torch.exp(coeffs)
    last = inputs.dim() - 1
    d = dim % inputs.dim() if inputs.dim() else 0
    if d != last:
        if (inputs.shape == coeffs.shape and inputs.dtype == coeffs.dtype and dim_worthwhile(inputs, d)
                and dim_eligible(coeffs, d)):
            return _LinrecDimFn.apply(inputs, coeffs, d, bool(reverse))
        x = inputs.transpose(d, last).contiguous()
        c = coeffs.transpose(d, last).contiguous()
        return linrec_pipe(x, c, reverse).transpose(d, last)
    if coeffs.stride() != inputs.stride():
        coeffs = torch.empty_like(inputs).copy_(coeffs)
    return linrec_pipe(inputs, coeffs, reverse)
