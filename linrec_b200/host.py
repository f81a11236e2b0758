"""Scan of tensors that live in (pinned) HOST memory, streamed through the GPU in row slabs.

Rows are independent, so a (numseq, seqlen) problem is cut into slabs of rows; slab i+1 is copied
to the device while slab i is being scanned and the results of slab i-1 travel back, on three
streams.  Device memory use is fixed (two sets of slab buffers) whatever the size of the tensors,
which also makes problems larger than the GPU's memory possible: the (8192, 2^20) fp32 forward +
backward needs 192 GiB for its six tensors, more than one B200 holds.

The reference has no such path (its operators take device tensors only); this is the entry point
the end-to-end measurement of bench.py times.
"""
from __future__ import annotations

import torch

from . import _capi
from .ops import _launch

__all__ = ["linrec_fwd_bwd_host", "linrec_fwd_host"]


def _check_host(*ts):
    a = ts[0]
    if a.dim() < 1:
        raise RuntimeError("linrec: need at least one dimension")
    for t in ts:
        if t.device.type != "cpu" or not t.is_contiguous() or t.shape != a.shape or t.dtype != a.dtype:
            raise RuntimeError("linrec host path: tensors must be contiguous CPU tensors of one shape and dtype")
    return a.reshape(-1, a.shape[-1]).shape


def _slabs(numseq: int, seqlen: int, itemsize: int, slab_rows):
    if slab_rows is None:
        # about 64 MiB per tensor and slab
        slab_rows = max(1, (64 << 20) // max(1, seqlen * itemsize))
    slab_rows = min(slab_rows, numseq)
    return [(r, min(r + slab_rows, numseq)) for r in range(0, numseq, slab_rows)], slab_rows


def _run(host_in, host_out, bwd_too: bool, reverse: bool, device, slab_rows):
    numseq, seqlen = _check_host(*host_in, *host_out)
    dev = torch.device(device if device is not None else "cuda")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    ins2d = [t.reshape(numseq, seqlen) for t in host_in]
    outs2d = [t.reshape(numseq, seqlen) for t in host_out]
    slabs, rows = _slabs(numseq, seqlen, host_in[0].element_size(), slab_rows)
    n_in, n_out = len(ins2d), len(outs2d)
    with torch.cuda.device(dev):
        s_in, s_run, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
        cur = torch.cuda.current_stream()
        for s in (s_in, s_run, s_out):
            s.wait_stream(cur)
        dbuf_in = [[torch.empty((rows, seqlen), dtype=host_in[0].dtype, device=dev) for _ in range(n_in)] for _ in range(2)]
        dbuf_out = [[torch.empty((rows, seqlen), dtype=host_in[0].dtype, device=dev) for _ in range(n_out)] for _ in range(2)]
        ev_in, ev_run, ev_out = {}, {}, {}
        for i, (r0, r1) in enumerate(slabs):
            n = r1 - r0
            b = i % 2
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(ev_run[i - 2])          # the scan of slab i-2 has read these buffers
                for k in range(n_in):
                    dbuf_in[b][k][:n].copy_(ins2d[k][r0:r1], non_blocking=True)
                ev_in[i] = s_in.record_event()
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[i])
                if i >= 2:
                    s_run.wait_event(ev_out[i - 2])         # the results of slab i-2 have left these buffers
                if bwd_too:
                    x, c, dy = (t[:n] for t in dbuf_in[b])
                    y, dx, dc = (t[:n] for t in dbuf_out[b])
                    _launch(_capi.KIND_PIPE, False, (x, c), reverse, {}, outs=(y,))
                    _launch(_capi.KIND_PIPE, True, (dy, c, y), reverse, {}, outs=(dx, dc))
                else:
                    x, c = (t[:n] for t in dbuf_in[b])
                    _launch(_capi.KIND_PIPE, False, (x, c), reverse, {}, outs=(dbuf_out[b][0][:n],))
                ev_run[i] = s_run.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[i])
                for k in range(n_out):
                    outs2d[k][r0:r1].copy_(dbuf_out[b][k][:n], non_blocking=True)
                ev_out[i] = s_out.record_event()
        for s in (s_in, s_run, s_out):
            cur.wait_stream(s)
    return host_out


def linrec_fwd_bwd_host(inputs, coeffs, d_outputs, reverse: bool = False, out=None, device=None, slab_rows=None):
    """Forward and backward of the scan for host tensors: returns (outputs, d_inputs, d_coeffs) on the
    host.  Pinned tensors make the copies asynchronous; `out` may hold three preallocated (pinned)
    result tensors.  The call returns after queueing; synchronise the current stream before reading."""
    if out is None:
        out = tuple(torch.empty_like(inputs, pin_memory=inputs.is_pinned()) for _ in range(3))
    _run((inputs, coeffs, d_outputs), tuple(out), True, reverse, device, slab_rows)
    return tuple(out)


def linrec_fwd_host(inputs, coeffs, reverse: bool = False, out=None, device=None, slab_rows=None):
    """Forward scan for host tensors (see linrec_fwd_bwd_host)."""
    if out is None:
        out = torch.empty_like(inputs, pin_memory=inputs.is_pinned())
    _run((inputs, coeffs), (out,), False, reverse, device, slab_rows)
    return out
