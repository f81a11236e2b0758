"""Multi-GPU modes of the scan (one process per GPU, `torch.distributed`).

The reference is single-device; both modes are additions, checked against the single-device result
on the unsharded tensor.

channel sharding   rows are independent: every rank scans its own rows with `linrec_b200.linrec`,
                   no communication at all (`linrec_channel_sharded` is literally that call).
sequence sharding  every rank holds the columns [rank*L, (rank+1)*L) of ALL rows.  Each rank scans
                   its shard locally and emits one small record per row, the records are
                   all-gathered once (NCCL over NVLink; 8 or 16 bytes per row and rank), and a fused
                   fix-up kernel folds the records of the earlier shards and adds
                   `carry * running product of c` to the local result, stopping along each row as
                   soon as that correction has underflowed to exactly zero (no later element can be changed by it).

`linrec_seq_sharded(x_shard, c_shard, reverse=False, group=None)` is differentiable; its backward
does the same three steps with the gradient scan.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _capi
from .ops import _DTYPES, _check_same, _empty_like_rows, _row_layout, _workspace, linrec_pipe

__all__ = ["linrec_channel_sharded", "linrec_seq_sharded", "seq_sharded_fwd", "seq_sharded_bwd", "PeerExchange"]


def linrec_channel_sharded(inputs: torch.Tensor, coeffs: torch.Tensor, reverse: bool = False) -> torch.Tensor:
    """Rows sharded over ranks: the local scan is the whole job."""
    return linrec_pipe(inputs, coeffs, reverse)


class CudaShardKernels:
    """The four C-ABI calls of sequence sharding on torch CUDA tensors."""

    @staticmethod
    def _prep(*ts):
        """Inputs brought to ONE row layout (numseq, seqlen, row_stride).  Every tensor of a call,
        results included, is addressed with that one row stride, so results are allocated with
        `_empty_like_rows` (the layout of the inputs): for padded rows a plain `empty_like` returns a
        contiguous tensor, which the kernels would overrun."""
        _check_same(*ts)
        ts = [t if _row_layout(t) is not None else t.contiguous() for t in ts]
        lay = _row_layout(ts[0])
        if any(_row_layout(t) != lay or t.stride() != ts[0].stride() for t in ts):
            ts = [t.contiguous() for t in ts]
            lay = _row_layout(ts[0])
        return ts, lay

    @staticmethod
    def _launch_env(ref, numseq, seqlen):
        stream = torch.cuda.current_stream(ref.device).cuda_stream
        dtype = _DTYPES[ref.dtype]
        need = _capi.lib.linrec_b200_workspace_size(numseq, seqlen, dtype)
        ws = _workspace(ref.device, stream, need)
        return stream, dtype, ws

    @staticmethod
    def _results(ref, out, n):
        """`n` result tensors with the layout of `ref`: the caller's (`out`) if they have it, else new ones."""
        if out is None:
            return [_empty_like_rows(ref) for _ in range(n)]
        out = list(out) if isinstance(out, (tuple, list)) else [out]
        if len(out) != n or any(o.shape != ref.shape or o.stride() != ref.stride() or o.dtype != ref.dtype or
                                o.device != ref.device for o in out):
            raise RuntimeError("linrec: result tensors must have the shape, strides, dtype and device of the inputs")
        return out

    def fwd_carry(self, x, c, reverse, shard, nshards, out=None):
        (x, c), (numseq, seqlen, stride) = self._prep(x, c)
        (y,) = self._results(x, out, 1)
        rec = torch.empty((numseq, 2), dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            stream, dtype, ws = self._launch_env(x, numseq, seqlen)
            rc = _capi.lib.linrec_b200_fwd_carry(x.data_ptr(), c.data_ptr(), y.data_ptr(), rec.data_ptr(), numseq,
                                                 seqlen, stride, int(bool(reverse)), dtype, shard, nshards, None,
                                                 ws.data_ptr(), ws.numel(), stream)
        _capi.raise_for(rc, "linrec_b200_fwd_carry")
        return y, rec

    def fwd_fixup(self, x, y, c, gathered, reverse, shard, nshards):
        numseq, seqlen, stride = _row_layout(y)
        with torch.cuda.device(y.device):
            stream = torch.cuda.current_stream(y.device).cuda_stream
            rc = _capi.lib.linrec_b200_fwd_fixup(x.data_ptr(), y.data_ptr(), c.data_ptr(), gathered.data_ptr(), numseq, seqlen,
                                                 stride, int(bool(reverse)), _DTYPES[y.dtype], shard, nshards, stream)
        _capi.raise_for(rc, "linrec_b200_fwd_fixup")

    def bwd_carry(self, dy, c, y, reverse, shard, nshards, out=None):
        (dy, c, y), (numseq, seqlen, stride) = self._prep(dy, c, y)
        dx, dc = self._results(dy, out, 2)
        rec = torch.empty((numseq, 4), dtype=torch.float32, device=dy.device)
        with torch.cuda.device(dy.device):
            stream, dtype, ws = self._launch_env(dy, numseq, seqlen)
            rc = _capi.lib.linrec_b200_bwd_carry(dy.data_ptr(), c.data_ptr(), y.data_ptr(), dx.data_ptr(), dc.data_ptr(),
                                                 rec.data_ptr(), numseq, seqlen, stride, int(bool(reverse)), dtype,
                                                 shard, nshards, None, ws.data_ptr(), ws.numel(), stream)
        _capi.raise_for(rc, "linrec_b200_bwd_carry")
        return dx, dc, rec, c, y, dy

    def bwd_fixup(self, dy, dx, dc, c, y, gathered, reverse, shard, nshards):
        numseq, seqlen, stride = _row_layout(dx)
        with torch.cuda.device(dx.device):
            stream = torch.cuda.current_stream(dx.device).cuda_stream
            rc = _capi.lib.linrec_b200_bwd_fixup(dy.data_ptr(), dx.data_ptr(), dc.data_ptr(), c.data_ptr(), y.data_ptr(),
                                                 gathered.data_ptr(), numseq, seqlen, stride, int(bool(reverse)),
                                                 _DTYPES[dx.dtype], shard, nshards, stream)
        _capi.raise_for(rc, "linrec_b200_bwd_fixup")


_CUDA_KERNELS = CudaShardKernels()


class PeerExchange:
    """Exchange buffers for sequence sharding without a collective call.

    Every rank allocates one buffer in symmetric (peer-mapped) memory; the scan kernels leave each
    row's record in their own buffer and flag all ranks when a launch is complete, and the fix-up
    kernels wait on the flags in their own buffer and read the records over NVLink from their
    owners, so a sharded scan is two kernel launches and nothing else.  Create one per
    process group and reuse it for every call (`linrec_seq_sharded(..., exchange=ex)`); calls are
    collective and must be made in the same order on all ranks.
    """

    def __init__(self, max_rows: int, group=None, device=None):
        import ctypes
        import torch.distributed._symmetric_memory as symm_mem
        self.max_rows = int(max_rows)
        self.epoch = 0
        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        nbytes = _capi.lib.linrec_b200_exchange_size(self.max_rows, self.world)
        dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=dev)
        handle = symm_mem.rendezvous(buf, group)
        ptrs = (ctypes.c_void_p * self.world)(*[int(p) for p in handle.buffer_ptrs])
        with torch.cuda.device(dev):
            rc = _capi.lib.linrec_b200_exchange_init(buf.data_ptr(), ptrs, self.rank, self.world, self.max_rows,
                                                     torch.cuda.current_stream(dev).cuda_stream)
        _capi.raise_for(rc, "linrec_b200_exchange_init")
        torch.cuda.synchronize(dev)
        handle.barrier()                   # every rank's buffer is initialised before anyone writes a flag into it
        self.buffer = buf
        self._keep = handle
        self._pending = None               # (event, pinned copy of the status word, workspace, stream) of the last call
        self._pinned = None

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    # A wait for another rank that ran out of its budget (option peerWaitBudgetMs, 30 s by default)
    # leaves wrong numbers and a bit in the status word of the workspace.  Reading that word means
    # waiting for the device, which the hot path must not do; so every call queues a copy of the word
    # into pinned memory behind its kernels, and the NEXT call looks at that copy if it has arrived.
    def _watch(self, ws, stream_obj):
        if self._pinned is None:
            self._pinned = torch.zeros(2, dtype=torch.int32, pin_memory=True)
        host = self._pinned[self.epoch & 1:(self.epoch & 1) + 1]    # the word is sticky, so losing an older copy loses nothing
        host.copy_(ws[4:8].view(torch.int32), non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(stream_obj)
        self._pending = (ev, host, ws, stream_obj)

    def poll(self, wait: bool = False) -> None:
        """Raise if an earlier call on this exchange gave up waiting for another rank.  Without `wait`
        only a result that has already arrived is looked at (no synchronisation)."""
        if self._pending is None:
            return
        ev, host, ws, stream_obj = self._pending
        if wait:
            ev.synchronize()
        elif not ev.query():
            return
        self._pending = None
        if int(host.item()) != 0:
            with torch.cuda.device(ws.device):
                rc = _capi.lib.linrec_b200_status(ws.data_ptr(), stream_obj.cuda_stream)   # reads and clears the word
            _capi.raise_for(rc if rc != 0 else _capi.ERR_TIMEOUT, "linrec_b200 peer exchange")

    def _env(self, ref, numseq, seqlen):
        stream = torch.cuda.current_stream(ref.device).cuda_stream
        dtype = _DTYPES[ref.dtype]
        ws = _workspace(ref.device, stream, _capi.lib.linrec_b200_workspace_size(numseq, seqlen, dtype))
        return stream, dtype, ws

    def fwd(self, x, c, reverse, opts=None, out=None):
        (x, c), (numseq, seqlen, stride) = CudaShardKernels._prep(x, c)
        if numseq > self.max_rows:
            raise RuntimeError("linrec: more rows than the peer exchange was created for")
        self.poll()
        (y,) = CudaShardKernels._results(x, out, 1)
        o, keep = _capi.make_opts(opts or {})
        with torch.cuda.device(x.device):
            stream, dtype, ws = self._env(x, numseq, seqlen)
            rc = _capi.lib.linrec_b200_fwd_seq_p2p(x.data_ptr(), c.data_ptr(), y.data_ptr(), numseq, seqlen, stride,
                                                   int(bool(reverse)), dtype, self.rank, self.world,
                                                   self.buffer.data_ptr(), self.next_epoch(), o, ws.data_ptr(), ws.numel(), stream)
            _capi.raise_for(rc, "linrec_b200_fwd_seq_p2p")
            self._watch(ws, torch.cuda.current_stream(x.device))
        return y

    def bwd(self, dy, c, y, reverse, opts=None, out=None):
        (dy, c, y), (numseq, seqlen, stride) = CudaShardKernels._prep(dy, c, y)
        if numseq > self.max_rows:
            raise RuntimeError("linrec: more rows than the peer exchange was created for")
        self.poll()
        dx, dc = CudaShardKernels._results(dy, out, 2)
        o, keep = _capi.make_opts(opts or {})
        with torch.cuda.device(dy.device):
            stream, dtype, ws = self._env(dy, numseq, seqlen)
            rc = _capi.lib.linrec_b200_bwd_seq_p2p(dy.data_ptr(), c.data_ptr(), y.data_ptr(), dx.data_ptr(), dc.data_ptr(),
                                                   numseq, seqlen, stride, int(bool(reverse)), dtype, self.rank, self.world,
                                                   self.buffer.data_ptr(), self.next_epoch(), o, ws.data_ptr(),
                                                   ws.numel(), stream)
            _capi.raise_for(rc, "linrec_b200_bwd_seq_p2p")
            self._watch(ws, torch.cuda.current_stream(dy.device))
        return dx, dc


def _gather(records: torch.Tensor, group) -> torch.Tensor:
    """All-gather of the per-row records in rank order: result[(rank, row, k)]."""
    world = dist.get_world_size(group)
    rows = records.shape[0]
    out = torch.empty((world * rows,) + tuple(records.shape[1:]), dtype=records.dtype, device=records.device)
    dist.all_gather_into_tensor(out, records.contiguous(), group=group)   # concatenation along dim 0
    return out.view((world, rows) + tuple(records.shape[1:]))


def seq_sharded_fwd(x: torch.Tensor, c: torch.Tensor, reverse: bool = False, group=None, kernels=None, exchange=None,
                    out=None):
    """Forward scan of a row that is split over the ranks of `group` (this rank holds shard `rank`).
    With `exchange` (a PeerExchange) the records are read from peer memory inside the kernels; without it
    by one all-gather.  `out` may hold a preallocated result with the layout of `x`."""
    kw = {} if out is None else {"out": out}
    if exchange is not None:
        return exchange.fwd(x, c, reverse, **kw)
    k = kernels or _CUDA_KERNELS
    shard, nshards = dist.get_rank(group), dist.get_world_size(group)
    y, rec = k.fwd_carry(x, c, reverse, shard, nshards, **kw)
    if nshards > 1:
        gathered = _gather(rec, group)
        same = lambda t: t if t.stride() == y.stride() else t.contiguous()
        k.fwd_fixup(same(x), y, same(c), gathered, reverse, shard, nshards)
    return y


def seq_sharded_bwd(dy: torch.Tensor, c: torch.Tensor, y: torch.Tensor, reverse: bool = False, group=None,
                    kernels=None, exchange=None, out=None):
    """Backward of `seq_sharded_fwd`: (dx, dc) of this rank's shard; `y` is the forward output shard.
    `out` may hold two preallocated results with the layout of `dy`."""
    kw = {} if out is None else {"out": out}
    if exchange is not None:
        return exchange.bwd(dy, c, y, reverse, **kw)
    k = kernels or _CUDA_KERNELS
    shard, nshards = dist.get_rank(group), dist.get_world_size(group)
    dx, dc, rec, c2, y2, dy2 = k.bwd_carry(dy, c, y, reverse, shard, nshards, **kw)
    if nshards > 1:
        gathered = _gather(rec, group)
        k.bwd_fixup(dy2, dx, dc, c2, y2, gathered, reverse, shard, nshards)
    return dx, dc


class _SeqShardedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, c, reverse, group, exchange):
        y = seq_sharded_fwd(x, c, reverse, group, exchange=exchange)
        ctx.save_for_backward(c, y)
        ctx.reverse, ctx.group, ctx.exchange = reverse, group, exchange
        return y

    @staticmethod
    def backward(ctx, dy):
        c, y = ctx.saved_tensors
        if dy.stride() != c.stride():
            dy = _empty_like_rows(c).copy_(dy)
        dx, dc = seq_sharded_bwd(dy, c, y, ctx.reverse, ctx.group, exchange=ctx.exchange)
        return dx, dc, None, None, None


def linrec_seq_sharded(inputs: torch.Tensor, coeffs: torch.Tensor, reverse: bool = False, group=None,
                       exchange=None) -> torch.Tensor:
    """Differentiable scan over a sequence that is sharded across the ranks of `group`; `exchange`
    (a PeerExchange) selects the peer-store path instead of the all-gather."""
    return _SeqShardedFn.apply(inputs, coeffs, reverse, group, exchange)
