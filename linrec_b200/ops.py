"""Python operator surface: the same names, signatures and error behaviour as the reference's
linrec/impl/cuda/ops.py:11-101 -- three operator families (`linrec_ref`, `linrec_tile`,
`linrec_pipe`), each a `torch.library` custom op pair `*_fwd` / `*_bwd` in the `linreccuda`
namespace with fake implementations and autograd registration -- on top of the C ABI.

    y = linrec_pipe(inputs, coeffs, reverse=False)        # y[i] = y[i-1]*coeffs[i] + inputs[i]

Differences from the reference, all widening: bfloat16 and float16 storage are accepted next to float32
(arithmetic stays fp32); rows may have a stride larger than their length; tensors whose leading
dimensions cannot be described by one row stride are made contiguous instead of being read as if
they were; element counts are 64-bit.
"""
from __future__ import annotations

import contextlib
import functools
import os
import threading
from types import SimpleNamespace
from typing import Tuple

import torch
from torch.autograd.function import FunctionCtx

from . import _capi

__all__ = ["linrec_ref", "linrec_tile", "linrec_pipe"]

_DTYPES = {torch.float32: _capi.DTYPE_F32, torch.bfloat16: _capi.DTYPE_BF16, torch.float16: _capi.DTYPE_F16,
           torch.float64: _capi.DTYPE_F64}   # float64: linrec_ref, and linrec_pipe / linrec_tile by one CTA per row
_CHECK_EVERY_CALL = os.environ.get("LINREC_B200_CHECK", "0") not in ("0", "")

# ---- workspace cache: one scratch buffer per (device, stream) --------------------------------------
_ws_lock = threading.Lock()
_workspaces: dict = {}


def _workspace(device: torch.device, stream_ptr: int, nbytes: int) -> torch.Tensor:
    key = (device.index, stream_ptr)
    with _ws_lock:
        ws = _workspaces.get(key)
        if ws is None or ws.numel() < nbytes:
            # zeroed once; every launch leaves the workspace ready for the next one
            ws = torch.zeros(max(nbytes, 1 << 16), dtype=torch.uint8, device=device)
            _workspaces[key] = ws
        return ws


@functools.lru_cache(maxsize=256)
def _workspace_size(numseq: int, seqlen: int, dtype: int) -> int:
    return int(_capi.lib.linrec_b200_workspace_size(numseq, seqlen, dtype))


def _on_device(device: torch.device):
    """Context that makes `device` current; free when it already is (the usual case)."""
    if torch.cuda.current_device() == device.index:
        return contextlib.nullcontext()
    return torch.cuda.device(device)


def check_status(device=None) -> None:
    """Synchronise and raise if a bounded device-side wait gave up in an earlier call."""
    with _ws_lock:
        items = list(_workspaces.items())
    for (dev, stream_ptr), ws in items:
        if device is not None and torch.device(device).index not in (None, dev):
            continue
        with torch.cuda.device(dev):
            rc = _capi.lib.linrec_b200_status(ws.data_ptr(), stream_ptr)
        _capi.raise_for(rc, "linrec_b200 device status")


# ---- argument handling -----------------------------------------------------------------------------
def _check_same(*ts: torch.Tensor) -> None:
    """The reference's preconditions (linrec/impl/cuda/linrec_pipe.cu:17-22,35)."""
    a = ts[0]
    for b in ts[1:]:
        if a.size() != b.size():
            raise RuntimeError("linrec: tensors must have the same sizes")
        if a.stride() != b.stride():
            raise RuntimeError("linrec: tensors must have the same strides")
        if a.device != b.device:
            raise RuntimeError("linrec: tensors must be on the same device")
        if a.dtype != b.dtype:
            raise RuntimeError("linrec: tensors must have the same dtype")
    if not all(t.is_cuda for t in ts):
        raise RuntimeError("linrec: tensors must be CUDA tensors (there is no CPU implementation)")
    if a.dtype not in _DTYPES:
        raise RuntimeError(f"linrec: dtype {a.dtype} is not supported (float32, bfloat16, float16, float64)")
    if a.dim() == 0:
        raise RuntimeError("linrec: need at least one dimension")
    if a.numel() > 0 and a.stride(-1) != 1:
        raise RuntimeError("linrec: the innermost dimension must have stride 1")


def _row_layout(t: torch.Tensor):
    """(numseq, seqlen, row_stride) if `t` is a set of rows at one uniform stride, else None."""
    L = t.size(-1)
    n = t.numel() // L if L else 0
    dims = [(sz, st) for sz, st in zip(t.shape[:-1], t.stride()[:-1]) if sz != 1]
    if not dims:
        return n, L, L
    row_stride = dims[-1][1]
    if row_stride < L:
        return None
    expect = row_stride
    for sz, st in reversed(dims):
        if st != expect:
            return None
        expect = st * sz
    return n, L, row_stride


def _empty_like_rows(t: torch.Tensor) -> torch.Tensor:
    """A result tensor with the LAYOUT of `t`.  `torch.empty_like` keeps the strides of dense tensors
    only; for rows that are padded (row stride larger than the row) it returns a contiguous tensor,
    and a kernel that is handed one row stride for all its tensors would then write outside it.  Rows
    at one uniform stride keep their strides here; anything else gets a contiguous result."""
    if t.numel() and _row_layout(t) is not None:
        return _empty_strided_like(t, t.size(), t.stride())
    return torch.empty(t.size(), dtype=t.dtype, device=t.device)


def _empty_strided_like(ref: torch.Tensor, size, stride) -> torch.Tensor:
    """`torch.empty_strided`, but starting as far from a 16-byte boundary as `ref` does: the kernel that
    takes rows of any alignment walks all tensors of a call in the same 16-byte chunks, and a view that
    starts inside a wider tensor would otherwise get a result that starts on a boundary."""
    skew = ref.data_ptr() & 15
    if skew == 0 or skew % ref.element_size():
        return torch.empty_strided(size, stride, dtype=ref.dtype, device=ref.device)
    skew //= ref.element_size()
    n = 1 + sum((sz - 1) * st for sz, st in zip(size, stride))
    return torch.empty(n + skew, dtype=ref.dtype, device=ref.device).as_strided(size, stride, skew)


# Signature (shape, strides, dtype, device) of tensors that passed every check before -> their row
# layout.  A training loop calls with the same signatures over and over; for them the preconditions
# reduce to "all tensors of the call have the signature of the first, and that one is known".
_known_layouts: dict = {}


def _launch(kind: int, bwd: bool, ins, reverse: bool, kwargs: dict, outs=None):
    """One forward or backward call.  `outs` (optional) are caller-provided result tensors with the
    layout of the inputs; without them the results are allocated like the inputs."""
    ref = ins[0]
    n_out = 2 if bwd else 1
    sig = (ref.shape, ref.stride(), ref.dtype, ref.device)
    layout = _known_layouts.get(sig)
    if layout is not None and all((t.shape, t.stride(), t.dtype, t.device) == sig for t in ins[1:]) and (
            outs is None or (len(outs) == n_out and all((t.shape, t.stride(), t.dtype, t.device) == sig for t in outs))):
        if outs is None:
            outs = [_empty_strided_like(ref, sig[0], sig[1]) for _ in range(n_out)]
        work_ins, work_outs = ins, outs
    else:
        _check_same(*ins)
        if outs is None:
            outs = [_empty_like_rows(ref) for _ in range(n_out)]
        else:
            outs = list(outs)
            if len(outs) != n_out:
                raise RuntimeError("linrec: wrong number of result tensors")
            _check_same(ref, *outs)
        if ref.numel() == 0:
            return outs
        layout = _row_layout(ref)
        work_ins, work_outs = list(ins), outs
        if layout is None or any(o.stride() != ref.stride() for o in outs):
            work_ins = [t.contiguous() for t in ins]
            work_outs = [torch.empty_like(work_ins[0]) for _ in range(n_out)]
            layout = _row_layout(work_ins[0])
        elif len(_known_layouts) < 4096:
            _known_layouts[sig] = layout        # every tensor of this call has the signature of `ref`
    numseq, seqlen, row_stride = layout
    dtype = _DTYPES[ref.dtype]
    opts, keep = _capi.make_opts(kwargs)
    with _on_device(ref.device):
        stream = torch.cuda.current_stream(ref.device).cuda_stream
        ws = _workspace(ref.device, stream, _workspace_size(numseq, seqlen, dtype))
        if not bwd:
            rc = _capi.lib.linrec_b200_fwd(kind, work_ins[0].data_ptr(), work_ins[1].data_ptr(),
                                           work_outs[0].data_ptr(), numseq, seqlen, row_stride,
                                           int(bool(reverse)), dtype, opts, ws.data_ptr(), ws.numel(), stream)
        else:
            rc = _capi.lib.linrec_b200_bwd(kind, work_ins[0].data_ptr(), work_ins[1].data_ptr(),
                                           work_ins[2].data_ptr(), work_outs[0].data_ptr(),
                                           work_outs[1].data_ptr(), numseq, seqlen, row_stride,
                                           int(bool(reverse)), dtype, opts, ws.data_ptr(), ws.numel(), stream)
        _capi.raise_for(rc, "linrec_b200_bwd" if bwd else "linrec_b200_fwd")
        if _CHECK_EVERY_CALL:
            _capi.raise_for(_capi.lib.linrec_b200_status(ws.data_ptr(), stream), "linrec_b200 device status")
    if work_outs is not outs:
        for o, w in zip(outs, work_outs):
            o.copy_(w)
    return outs


def dim_eligible(t: torch.Tensor, dim: int) -> bool:
    """Can the scan run along `dim` of `t` in place of a transposed copy?  Needs a dense tensor,
    16-byte aligned, whose trailing extent (the product of the sizes after `dim`) is a whole number
    of 16-byte chunks."""
    if t.dtype not in _DTYPES or not t.is_cuda or not t.is_contiguous():
        return False
    inner = 1
    for s in t.shape[dim + 1:]:
        inner *= s
    return inner > 1 and (inner * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0


def dim_worthwhile(t: torch.Tensor, dim: int) -> bool:
    """Is scanning along `dim` where the tensor lies faster than transposed copies around the
    last-axis kernel?  Measured on B200: yes unless there are only a few columns (one column = 32
    channel words of one batch entry), where the kernel has to cut the sequence into chunks linked
    by look-back and reaches 0.7-1.5 TB/s against about 2 TB/s for the transposed path."""
    if not dim_eligible(t, dim):
        return False
    nb = 1
    for s in t.shape[:dim]:
        nb *= s
    nchan = 1
    for s in t.shape[dim + 1:]:
        nchan *= s
    per_col = 32 * (4 // t.element_size())
    return nb * -(-nchan // per_col) >= 128


def _launch_dim(bwd: bool, ins, dim: int, reverse: bool, kwargs: dict):
    """Forward or backward scan along `dim` (not the last) of dense tensors of one shape, through
    linrec_b200_fwd_dim / linrec_b200_bwd_dim: the tensors are taken as (nb, seqlen, nchan)."""
    ref = ins[0]
    for t in ins:
        if t.shape != ref.shape or t.dtype != ref.dtype or t.device != ref.device:
            raise RuntimeError("linrec: tensors must have the same shape, dtype and device")
        if not dim_eligible(t, dim):
            raise RuntimeError("linrec: scan along this dimension needs dense, 16-byte aligned tensors")
    outs = [torch.empty_like(ref) for _ in range(2 if bwd else 1)]
    if ref.numel() == 0:
        return outs
    nb = 1
    for s in ref.shape[:dim]:
        nb *= s
    seqlen = ref.shape[dim]
    nchan = ref.numel() // (nb * seqlen)
    dtype = _DTYPES[ref.dtype]
    opts, keep = _capi.make_opts(kwargs)
    with torch.cuda.device(ref.device):
        stream = torch.cuda.current_stream(ref.device).cuda_stream
        need = _capi.lib.linrec_b200_dim_workspace_size(int(bwd), nb, seqlen, nchan, dtype, opts)
        if need == 0:
            raise NotImplementedError("linrec: no compiled variant for these options")
        ws = _workspace(ref.device, stream, need)
        if not bwd:
            rc = _capi.lib.linrec_b200_fwd_dim(ins[0].data_ptr(), ins[1].data_ptr(), outs[0].data_ptr(), nb, seqlen,
                                               nchan, int(bool(reverse)), dtype, opts, ws.data_ptr(), ws.numel(), stream)
        else:
            rc = _capi.lib.linrec_b200_bwd_dim(ins[0].data_ptr(), ins[1].data_ptr(), ins[2].data_ptr(),
                                               outs[0].data_ptr(), outs[1].data_ptr(), nb, seqlen, nchan,
                                               int(bool(reverse)), dtype, opts, ws.data_ptr(), ws.numel(), stream)
        _capi.raise_for(rc, "linrec_b200_bwd_dim" if bwd else "linrec_b200_fwd_dim")
        if _CHECK_EVERY_CALL:
            _capi.raise_for(_capi.lib.linrec_b200_status(ws.data_ptr(), stream), "linrec_b200 device status")
    return outs


def linrec_dim_fwd(inputs, coeffs, dim, reverse=False, **kwargs):
    return _launch_dim(False, (inputs, coeffs), dim, reverse, kwargs)[0]


def linrec_dim_bwd(d_outputs, coeffs, outputs, dim, reverse=False, **kwargs):
    return tuple(_launch_dim(True, (d_outputs, coeffs, outputs), dim, reverse, kwargs))


def _fwd(kind):
    def f(inputs, coeffs, reverse=False, **kwargs):
        return _launch(kind, False, (inputs, coeffs), reverse, kwargs)[0]
    return f


def _bwd(kind):
    def f(d_outputs, coeffs, outputs, reverse=False, **kwargs):
        dx, dc = _launch(kind, True, (d_outputs, coeffs, outputs), reverse, kwargs)
        return dx, dc
    return f


def _attrs(kind):
    def f(fwd, dtype=torch.float32, **kwargs):
        return _capi.attrs(kind, fwd, _DTYPES[dtype], kwargs)
    return f


# The object that stands where the reference has its compiled module `_C`
# (functions of linrec/impl/cuda/extension.cpp:36-72, same names and keyword arguments; integer
# keyword arguments select a compiled variant as there).
_C = SimpleNamespace(
    linrec_ref_fwd=_fwd(_capi.KIND_REF), linrec_ref_bwd=_bwd(_capi.KIND_REF),
    linrec_tile_fwd=_fwd(_capi.KIND_TILE), linrec_tile_bwd=_bwd(_capi.KIND_TILE),
    linrec_pipe_fwd=_fwd(_capi.KIND_PIPE), linrec_pipe_bwd=_bwd(_capi.KIND_PIPE),
    linrec_tile_attrs=_attrs(_capi.KIND_TILE), linrec_pipe_attrs=_attrs(_capi.KIND_PIPE),
    linrec_ref_attrs=_attrs(_capi.KIND_REF),
    config_names=_capi.config_names(),
    config_list=_capi.config_list(),
    launch_count=_capi.launch_count,
)


# ---- fake (meta) implementations and autograd wiring -----------------------------------------------
def setup_context(ctx: FunctionCtx, inputs, output):
    _, coeffs, reverse = inputs
    ctx.save_for_backward(coeffs, output)
    ctx.reverse = reverse


def fake_fwd(inputs: torch.Tensor, coeffs: torch.Tensor, reverse: bool = False) -> torch.Tensor:
    assert inputs.size() == coeffs.size()
    assert inputs.stride() == coeffs.stride()
    assert inputs.device == coeffs.device
    assert inputs.dtype == coeffs.dtype
    assert inputs.stride(-1) == 1
    return _empty_like_rows(inputs)


def fake_bwd(d_outputs: torch.Tensor, coeffs: torch.Tensor, outputs: torch.Tensor,
             reverse: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    assert d_outputs.size() == coeffs.size() == outputs.size()
    assert d_outputs.stride() == coeffs.stride() == outputs.stride()
    assert d_outputs.device == coeffs.device == outputs.device
    assert d_outputs.dtype == coeffs.dtype == outputs.dtype
    assert d_outputs.stride(-1) == 1
    return _empty_like_rows(d_outputs), _empty_like_rows(coeffs)


def _register(family: str):
    c_fwd, c_bwd = getattr(_C, f"linrec_{family}_fwd"), getattr(_C, f"linrec_{family}_bwd")

    @torch.library.custom_op(f"linreccuda::linrec_{family}_fwd", mutates_args=(), device_types="cuda")
    def fwd(inputs: torch.Tensor, coeffs: torch.Tensor, reverse: bool = False) -> torch.Tensor:
        return c_fwd(inputs=inputs, coeffs=coeffs, reverse=reverse)

    @torch.library.custom_op(f"linreccuda::linrec_{family}_bwd", mutates_args=(), device_types="cuda")
    def bwd(d_outputs: torch.Tensor, coeffs: torch.Tensor, outputs: torch.Tensor,
            reverse: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        return c_bwd(d_outputs=d_outputs, coeffs=coeffs, outputs=outputs, reverse=reverse)

    fwd.register_fake(fake_fwd)
    bwd.register_fake(fake_bwd)

    def backward(ctx: FunctionCtx, d_outputs: torch.Tensor):
        coeffs, outputs = ctx.saved_tensors
        # The incoming gradient may have any layout; the saved tensors keep theirs.  Bring the
        # gradient to the layout of the saved tensors (the reference only fixes stride(-1) and
        # then fails its equal-strides check, linrec/impl/cuda/ops.py:55).
        if d_outputs.stride() != coeffs.stride():
            d_outputs = _empty_like_rows(coeffs).copy_(d_outputs)
        d_inputs, d_coeffs = bwd(d_outputs=d_outputs, coeffs=coeffs, outputs=outputs, reverse=ctx.reverse)
        return d_inputs, d_coeffs, None

    torch.library.register_autograd(f"linreccuda::linrec_{family}_fwd", backward, setup_context=setup_context)
    return fwd, bwd


linrec_ref_fwd, linrec_ref_bwd = _register("ref")
linrec_tile_fwd, linrec_tile_bwd = _register("tile")
linrec_pipe_fwd, linrec_pipe_bwd = _register("pipe")
linrec_ref = linrec_ref_fwd
linrec_tile = linrec_tile_fwd
linrec_pipe = linrec_pipe_fwd
