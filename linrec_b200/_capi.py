"""ctypes binding of the C ABI declared in include/linrec_b200.h.

This is the whole "extension layer": Python hands raw device pointers, sizes and the current CUDA
stream to the shared library; all host logic (checks, regime selection, tensor maps, launches)
is C++ inside the library.  It stands where the reference has its pybind11 module
(linrec/impl/cuda/extension.cpp:36-72).

There is no CPU path: if the shared library cannot be loaded, importing this module raises.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

OK = 0
ERR_INVALID_ARG = -1
ERR_WORKSPACE = -2
ERR_NOT_IMPLEMENTED = -3
ERR_CUDA = -4
ERR_TIMEOUT = -5
ERR_TOO_LONG = -6
ERR_UNALIGNED = -7
ERR_SCRATCH_LIMIT = -8

DTYPE_F32, DTYPE_BF16, DTYPE_F16, DTYPE_F64 = 0, 1, 2, 3
KIND_REF, KIND_TILE, KIND_PIPE = 0, 1, 2


class LinrecOpts(ctypes.Structure):
    _fields_ = [("n_opts", ctypes.c_int),
                ("names", ctypes.POINTER(ctypes.c_char_p)),
                ("values", ctypes.POINTER(ctypes.c_int))]


def _load() -> ctypes.CDLL:
    path = _build.LIB_PATH
    try:
        _build.build_library()          # no-op when the library is newer than its sources
    except Exception as exc:            # no nvcc on this machine, compile error, ...
        if not os.path.exists(path):
            raise ImportError(
                f"linrec_b200: the CUDA library {path} is missing and could not be built ({exc}). "
                "Build it with `python -m linrec_b200.build`; there is no fallback implementation."
            ) from exc
    lib = ctypes.CDLL(path)
    i32, i64, vp, sz = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p, ctypes.c_size_t
    po = ctypes.POINTER(LinrecOpts)
    lib.linrec_b200_workspace_size.argtypes = [i64, i64, i32]
    lib.linrec_b200_workspace_size.restype = sz
    lib.linrec_b200_fwd.argtypes = [i32, vp, vp, vp, i64, i64, i64, i32, i32, po, vp, sz, vp]
    lib.linrec_b200_fwd.restype = i32
    lib.linrec_b200_bwd.argtypes = [i32, vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, po, vp, sz, vp]
    lib.linrec_b200_bwd.restype = i32
    lib.linrec_b200_status.argtypes = [vp, vp]
    lib.linrec_b200_status.restype = i32
    lib.linrec_b200_attrs.argtypes = [i32, i32, i32, po, ctypes.POINTER(ctypes.c_char_p),
                                      ctypes.POINTER(i32), i32]
    lib.linrec_b200_attrs.restype = i32
    lib.linrec_b200_config_names.argtypes = [ctypes.POINTER(ctypes.c_char_p), i32]
    lib.linrec_b200_config_names.restype = i32
    lib.linrec_b200_config_list.argtypes = [ctypes.POINTER(i32), i32]
    lib.linrec_b200_config_list.restype = i32
    lib.linrec_b200_fwd_carry.argtypes = [vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, i32, po, vp, sz, vp]
    lib.linrec_b200_fwd_carry.restype = i32
    lib.linrec_b200_fwd_fixup.argtypes = [vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, i32, vp]
    lib.linrec_b200_fwd_fixup.restype = i32
    lib.linrec_b200_bwd_carry.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, i32, po, vp, sz, vp]
    lib.linrec_b200_bwd_carry.restype = i32
    lib.linrec_b200_bwd_fixup.argtypes = [vp, vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, i32, vp]
    lib.linrec_b200_bwd_fixup.restype = i32
    pp = ctypes.POINTER(ctypes.c_void_p)
    lib.linrec_b200_exchange_size.argtypes = [i64, i32]
    lib.linrec_b200_exchange_size.restype = sz
    lib.linrec_b200_exchange_init.argtypes = [vp, pp, i32, i32, i64, vp]
    lib.linrec_b200_exchange_init.restype = i32
    lib.linrec_b200_fwd_seq_p2p.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, i32, i32, vp, ctypes.c_uint32, po, vp, sz, vp]
    lib.linrec_b200_fwd_seq_p2p.restype = i32
    lib.linrec_b200_bwd_seq_p2p.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, i32, i32, vp, ctypes.c_uint32, po,
                                            vp, sz, vp]
    lib.linrec_b200_bwd_seq_p2p.restype = i32
    lib.linrec_b200_dim_workspace_size.argtypes = [i32, i64, i64, i64, i32, po]
    lib.linrec_b200_dim_workspace_size.restype = sz
    lib.linrec_b200_fwd_dim.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, po, vp, sz, vp]
    lib.linrec_b200_fwd_dim.restype = i32
    lib.linrec_b200_bwd_dim.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i32, i32, po, vp, sz, vp]
    lib.linrec_b200_bwd_dim.restype = i32
    lib.linrec_b200_fwd_static.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, vp]
    lib.linrec_b200_fwd_static.restype = i32
    lib.linrec_b200_static_workspace.argtypes = [pp, ctypes.POINTER(sz)]
    lib.linrec_b200_static_workspace.restype = i32
    lib.linrec_b200_launch_count.argtypes = []
    lib.linrec_b200_launch_count.restype = ctypes.c_uint64
    lib.linrec_b200_last_cuda_error.argtypes = []
    lib.linrec_b200_last_cuda_error.restype = ctypes.c_char_p
    lib.linrec_b200_strerror.argtypes = [i32]
    lib.linrec_b200_strerror.restype = ctypes.c_char_p
    lib.linrec_b200_version.argtypes = []
    lib.linrec_b200_version.restype = i32
    return lib


lib = _load()


def strerror(code: int) -> str:
    return lib.linrec_b200_strerror(code).decode()


def make_opts(kwargs: dict):
    """dict[str, int] -> (LinrecOpts, keep-alive objects); None for no options."""
    if not kwargs:
        return None, None
    n = len(kwargs)
    names = (ctypes.c_char_p * n)(*[k.encode() for k in kwargs])
    values = (ctypes.c_int * n)(*[int(v) for v in kwargs.values()])
    o = LinrecOpts(n, ctypes.cast(names, ctypes.POINTER(ctypes.c_char_p)),
                   ctypes.cast(values, ctypes.POINTER(ctypes.c_int)))
    return ctypes.byref(o), (o, names, values)


def raise_for(code: int, what: str) -> None:
    """Error translation: the reference raises RuntimeError from TORCH_CHECK and NotImplementedError
    for an unknown compile-time configuration (linrec/impl/cuda/dispatch.h:70-71)."""
    if code == OK:
        return
    msg = f"{what}: {strerror(code)} (status {code})"
    if code == ERR_CUDA:
        msg += f" [{lib.linrec_b200_last_cuda_error().decode()}]"
    if code == ERR_NOT_IMPLEMENTED:
        raise NotImplementedError(msg)
    raise RuntimeError(msg)


def config_names():
    n = lib.linrec_b200_config_names(None, 0)
    buf = (ctypes.c_char_p * n)()
    lib.linrec_b200_config_names(buf, n)
    return [b.decode() for b in buf]


def config_list():
    ncol = lib.linrec_b200_config_names(None, 0)
    nrow = lib.linrec_b200_config_list(None, 0)
    buf = (ctypes.c_int * (nrow * ncol))()
    lib.linrec_b200_config_list(buf, nrow)
    return [tuple(buf[r * ncol + c] for c in range(ncol)) for r in range(nrow)]


def attrs(kind: int, fwd: bool, dtype: int, kwargs: dict) -> dict:
    cap = 32
    names = (ctypes.c_char_p * cap)()
    values = (ctypes.c_int * cap)()
    opts, keep = make_opts(kwargs)
    n = lib.linrec_b200_attrs(kind, int(bool(fwd)), dtype, opts, names, values, cap)
    if n < 0:
        raise_for(n, "linrec_b200_attrs")
    return {names[i].decode(): int(values[i]) for i in range(n)}


def launch_count() -> int:
    return int(lib.linrec_b200_launch_count())
