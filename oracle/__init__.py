"""CPU oracle for the linear-recurrence scan -- TEST INFRASTRUCTURE ONLY.

Only tests/, `__graft_entry__.smoke()` and the CPU-baseline / reference legs of bench.py may
import this package, and only as the checker (or as the thing timed on the host cores).  The
shipped package `linrec_b200` never imports it and has no CPU path of its own.

Three checkers live here:

* `fwd_f32 / bwd_f32`   the C restatement (oracle/linrec_oracle.c) of the reference's sequential
                        algorithm, separately rounded multiply and add, bit-identical to the
                        reference's Python implementation on the committed golden fixtures.
* `fwd_f64 / bwd_f64`   the same recurrences evaluated in double precision from fp32 inputs.
* `pyloop_fwd / pyloop_bwd`  a torch restatement of the reference's Python loop (one vectorised
                        torch multiply and add per time step, across all rows) -- this is the
                        shape of the reference's CPU path and is what the benchmark times on the
                        host cores.

Parity pin: tests/test_oracle_golden.py checks all of them against tests/golden/*.npz, which
were produced by importing the unmodified reference (tests/golden/make_golden.py).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build

_LIB = None


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is None:
        path = _build.build_oracle()
        L = ctypes.CDLL(path)
        i64, p, i32 = ctypes.c_int64, ctypes.c_void_p, ctypes.c_int
        L.linrec_oracle_fwd_f32.argtypes = [p, p, p, i64, i64, i64, i32]
        L.linrec_oracle_fwd_f64.argtypes = [p, p, p, i64, i64, i64, i32]
        L.linrec_oracle_bwd_f32.argtypes = [p, p, p, p, p, i64, i64, i64, i32]
        L.linrec_oracle_bwd_f64.argtypes = [p, p, p, p, p, i64, i64, i64, i32]
        for f in (L.linrec_oracle_fwd_f32, L.linrec_oracle_fwd_f64,
                  L.linrec_oracle_bwd_f32, L.linrec_oracle_bwd_f64):
            f.restype = None
        L.linrec_oracle_threads.restype = i32
        L.linrec_oracle_set_threads.argtypes = [i32]
        _LIB = L
    return _LIB


def _as2d(a, dtype) -> np.ndarray:
    a = np.ascontiguousarray(np.asarray(a, dtype=dtype))
    if a.ndim == 0:
        raise ValueError("need at least one dimension")
    return a


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def fwd_f32(x, c, reverse: bool = False) -> np.ndarray:
    x, c = _as2d(x, np.float32), _as2d(c, np.float32)
    assert x.shape == c.shape
    y = np.empty_like(x)
    L = x.shape[-1]
    n = x.size // L if L else 0
    lib().linrec_oracle_fwd_f32(_ptr(x), _ptr(c), _ptr(y), n, L, L, int(bool(reverse)))
    return y


def bwd_f32(dy, c, y, reverse: bool = False):
    dy, c, y = _as2d(dy, np.float32), _as2d(c, np.float32), _as2d(y, np.float32)
    assert dy.shape == c.shape == y.shape
    dx, dc = np.empty_like(dy), np.empty_like(dy)
    L = dy.shape[-1]
    n = dy.size // L if L else 0
    lib().linrec_oracle_bwd_f32(_ptr(dy), _ptr(c), _ptr(y), _ptr(dx), _ptr(dc), n, L, L,
                                int(bool(reverse)))
    return dx, dc


def fwd_f64(x, c, reverse: bool = False) -> np.ndarray:
    x, c = _as2d(x, np.float32), _as2d(c, np.float32)
    y = np.empty(x.shape, dtype=np.float64)
    L = x.shape[-1]
    n = x.size // L if L else 0
    lib().linrec_oracle_fwd_f64(_ptr(x), _ptr(c), _ptr(y), n, L, L, int(bool(reverse)))
    return y


def bwd_f64(dy, c, y64, reverse: bool = False):
    dy, c = _as2d(dy, np.float32), _as2d(c, np.float32)
    y64 = _as2d(y64, np.float64)
    dx, dc = np.empty(dy.shape, np.float64), np.empty(dy.shape, np.float64)
    L = dy.shape[-1]
    n = dy.size // L if L else 0
    lib().linrec_oracle_bwd_f64(_ptr(dy), _ptr(c), _ptr(y64), _ptr(dx), _ptr(dc), n, L, L,
                                int(bool(reverse)))
    return dx, dc


def threads() -> int:
    return int(lib().linrec_oracle_threads())


def set_threads(n: int) -> None:
    lib().linrec_oracle_set_threads(int(n))


# ---------------------------------------------------------------------------------------------
# torch restatement of the reference's Python loop (linrec/impl/python/ops.py:8-40).  One rounded
# multiply and one rounded add per step, vectorised over the rows by torch -- the cost profile of
# the reference's CPU path: seqlen sequential steps, each a pair of elementwise torch kernels.
# ---------------------------------------------------------------------------------------------
def pyloop_fwd(x, c, reverse: bool = False):
    import torch
    y = torch.zeros_like(x)
    prev = torch.zeros_like(x[..., 0])
    L = x.shape[-1]
    steps = range(L - 1, -1, -1) if reverse else range(L)
    for i in steps:
        prev = prev * c[..., i] + x[..., i]
        y[..., i] = prev
    return y


def _shifted(t, by: int):
    """`by`=+1 moves data towards higher indices, -1 towards lower; vacated slots are 0."""
    import torch
    out = torch.zeros_like(t)
    if t.shape[-1] > 1:
        if by > 0:
            out[..., 1:] = t[..., :-1]
        else:
            out[..., :-1] = t[..., 1:]
    return out


def pyloop_bwd(dy, c, y, reverse: bool = False):
    cs = _shifted(c, +1 if reverse else -1)
    dx = pyloop_fwd(dy, cs, reverse=not reverse)
    dc = dx * _shifted(y, -1 if reverse else +1)
    return dx, dc
