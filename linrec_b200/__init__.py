"""linrec_b200 -- the linear-recurrence scan  y[i] = y[i-1]*c[i] + x[i]  for NVIDIA B200 (sm_100a).

Drop-in for the hot path of safelix/linrec: `linrec(inputs, coeffs, reverse=False)` with autograd,
the `linreccuda::*` custom ops and the `_C` introspection object, backed by hand-written CUDA
kernels behind a C ABI (include/linrec_b200.h).  CUDA only: importing this package on a machine
where the shared library cannot be loaded raises, and the operators reject CPU tensors
(the reference's package falls back to Triton or eager Python, linrec/__init__.py:3-11; this
one deliberately has a single implementation).
"""
from .ops import (  # noqa: F401
    _C,
    check_status,
    linrec_pipe,
    linrec_pipe_bwd,
    linrec_pipe_fwd,
    linrec_ref,
    linrec_ref_bwd,
    linrec_ref_fwd,
    linrec_tile,
    linrec_tile_bwd,
    linrec_tile_fwd,
)

from .general import linrec_general  # noqa: E402,F401

linrec = linrec_pipe

__version__ = "0.2.0"
__all__ = ["linrec", "linrec_ref", "linrec_tile", "linrec_pipe", "linrec_general", "check_status"]
