"""The wider signature of the reference's Python operator, `linrec(inputs, coeffs, logc=False,
dim=-1, reverse=False)` (linrec/impl/python/ops.py:8-61), on top of the CUDA scan.

`dim`   the scan runs along `dim`.  For a dimension other than the last, dense 16-byte aligned
        tensors whose trailing extent is a whole number of 16-byte chunks are scanned where they lie
        (a kernel that walks down the axis, neighbouring channels on neighbouring threads), unless
        there are only a handful of columns; anything else costs a transposed copy in and out.
`logc`  coefficients are given as logarithms: c = exp(coeffs).  The kernels apply exp as they load
        the coefficients and the backward kernels return the gradient with respect to the logarithm,
        d_coeffs * c, so neither exp(coeffs) nor d_coeffs is ever written to memory (option
        `logCoeffs` of the C ABI).  (The reference's own backward multiplies by the SHIFTED
        coefficients, linrec/impl/python/ops.py:33-38, which is not the derivative of its forward;
        this implementation follows the forward.)
"""
from __future__ import annotations

import torch

from .ops import _C, _empty_like_rows, dim_eligible, dim_worthwhile, linrec_dim_bwd, linrec_dim_fwd, linrec_pipe

__all__ = ["linrec_general"]


class _LinrecDimFn(torch.autograd.Function):
    """Scan along a non-last dimension of dense tensors; same saved tensors and gradient formulas
    as the last-dimension operator (linrec/impl/cuda/ops.py:17-21,54-59)."""

    @staticmethod
    def forward(ctx, inputs, coeffs, dim, reverse, logc):
        kw = {"logCoeffs": 1} if logc else {}
        outputs = linrec_dim_fwd(inputs, coeffs, dim, reverse, **kw)
        ctx.save_for_backward(coeffs, outputs)
        ctx.dim, ctx.reverse, ctx.kw = dim, reverse, kw
        return outputs

    @staticmethod
    def backward(ctx, d_outputs):
        coeffs, outputs = ctx.saved_tensors
        d_outputs = d_outputs.contiguous()
        if not dim_eligible(d_outputs, ctx.dim):
            d_outputs = d_outputs.clone(memory_format=torch.contiguous_format)
        d_inputs, d_coeffs = linrec_dim_bwd(d_outputs, coeffs, outputs, ctx.dim, ctx.reverse, **ctx.kw)
        return d_inputs, d_coeffs, None, None, None


class _LinrecLogcFn(torch.autograd.Function):
    """Last-dimension scan with logarithmic coefficients, exp fused into the kernels."""

    @staticmethod
    def forward(ctx, inputs, logcoeffs, reverse):
        outputs = _C.linrec_pipe_fwd(inputs=inputs, coeffs=logcoeffs, reverse=reverse, logCoeffs=1)
        ctx.save_for_backward(logcoeffs, outputs)
        ctx.reverse = reverse
        return outputs

    @staticmethod
    def backward(ctx, d_outputs):
        logcoeffs, outputs = ctx.saved_tensors
        if d_outputs.stride() != outputs.stride():
            d_outputs = _empty_like_rows(outputs).copy_(d_outputs)
        d_inputs, d_log = _C.linrec_pipe_bwd(d_outputs=d_outputs, coeffs=logcoeffs, outputs=outputs,
                                             reverse=ctx.reverse, logCoeffs=1)
        return d_inputs, d_log, None


def linrec_general(inputs: torch.Tensor, coeffs: torch.Tensor, logc: bool = False, dim: int = -1,
                   reverse: bool = False) -> torch.Tensor:
    last = inputs.dim() - 1
    d = dim % inputs.dim() if inputs.dim() else 0
    logc, reverse = bool(logc), bool(reverse)
    if d != last:
        if (inputs.shape == coeffs.shape and inputs.dtype == coeffs.dtype and dim_worthwhile(inputs, d)
                and dim_eligible(coeffs, d)):
            return _LinrecDimFn.apply(inputs, coeffs, d, reverse, logc)
        x = inputs.transpose(d, last).contiguous()
        c = coeffs.transpose(d, last).contiguous()
        y = _LinrecLogcFn.apply(x, c, reverse) if logc else linrec_pipe(x, c, reverse)
        return y.transpose(d, last)
    if coeffs.stride() != inputs.stride():
        coeffs = _empty_like_rows(inputs).copy_(coeffs)
    if logc:
        return _LinrecLogcFn.apply(inputs, coeffs, reverse)
    return linrec_pipe(inputs, coeffs, reverse)
