"""Sequence sharding, host side: two gloo ranks on CPU run `seq_sharded_fwd/bwd` with the device
kernels replaced by a numpy stand-in that follows the same record contract as the C ABI
(forward record (P, Y); backward record (P, Y, c at the shard's scan-last element, y at its
scan-first element); fix-up = fold of the earlier shards' records + carry * running product).
The records travel as fp32 (their contract), hence the 5e-6 tolerance.  What is under test is everything around the kernels: shard/rank bookkeeping, the all-gather layout,
direction handling -- against the CPU oracle on the unsharded tensor."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class NumpyShardKernels:
    """float64 stand-in for the four device entry points (same argument and record conventions)."""

    @staticmethod
    def _scan(x, c, asc, first_coeff_counts):
        L = x.shape[-1]
        y = np.zeros_like(x)
        v = np.zeros(x.shape[:-1])
        P = np.ones(x.shape[:-1])
        order = range(L) if asc else range(L - 1, -1, -1)
        for n, i in enumerate(order):
            ci = c[..., i] if (n > 0 or first_coeff_counts) else np.zeros_like(c[..., i])
            v = v * ci + x[..., i]
            P = P * ci
            y[..., i] = v
        return y, P, v

    def fwd_carry(self, x, c, reverse, shard, nshards):
        asc = not reverse
        holds_start = shard == (0 if asc else nshards - 1)
        y, P, Y = self._scan(x.numpy().astype(np.float64), c.numpy().astype(np.float64), asc, not holds_start)
        return torch.from_numpy(y), torch.from_numpy(np.stack([P, Y], -1).astype(np.float32))

    def fwd_fixup(self, x, y, c, gathered, reverse, shard, nshards):
        asc = not reverse
        order = list(range(nshards)) if asc else list(range(nshards - 1, -1, -1))
        g = gathered.numpy().astype(np.float64)
        v = np.zeros(y.shape[0])
        for s in order[:order.index(shard)]:
            v = v * g[s, :, 0] + g[s, :, 1]
        yn, cn = y.numpy(), c.numpy().astype(np.float64)
        L = yn.shape[-1]
        for i in (range(L) if asc else range(L - 1, -1, -1)):
            v = v * cn[:, i]
            yn[:, i] += v

    def bwd_carry(self, dy, c, y, reverse, shard, nshards):
        asc = bool(reverse)
        holds_start = shard == (0 if asc else nshards - 1)
        cn, yn, dyn = (t.numpy().astype(np.float64) for t in (c, y, dy))
        L = cn.shape[-1]
        cs, ys = np.ones_like(cn), np.zeros_like(yn)
        if asc:
            cs[:, 1:] = cn[:, :-1]
            ys[:, :-1] = yn[:, 1:]
        else:
            cs[:, :-1] = cn[:, 1:]
            ys[:, 1:] = yn[:, :-1]
        dx, P, Y = self._scan(dyn, cs, asc, not holds_start)
        dc = dx * ys
        first, last = (0, L - 1) if asc else (L - 1, 0)
        rec = np.stack([P, Y, cn[:, last], yn[:, first]], -1).astype(np.float32)
        return torch.from_numpy(dx), torch.from_numpy(dc), torch.from_numpy(rec), c, y, dy

    def bwd_fixup(self, dy, dx, dc, c, y, gathered, reverse, shard, nshards):
        asc = bool(reverse)
        order = list(range(nshards)) if asc else list(range(nshards - 1, -1, -1))
        pos = order.index(shard)
        g = gathered.numpy().astype(np.float64)
        v = np.zeros(dx.shape[0])
        prev = None
        for s in order[:pos]:
            if prev is not None:
                v = v * g[prev, :, 2]
            v = v * g[s, :, 0] + g[s, :, 1]
            prev = s
        if prev is not None:
            v = v * g[prev, :, 2]
        dxn, dcn, cn, yn = dx.numpy(), dc.numpy(), c.numpy().astype(np.float64), y.numpy().astype(np.float64)
        L = dxn.shape[-1]
        idx = list(range(L)) if asc else list(range(L - 1, -1, -1))
        for n, i in enumerate(idx):
            if n > 0:
                v = v * cn[:, idx[n - 1]]
            dxn[:, i] += v
            if n + 1 < L:
                dcn[:, i] += v * yn[:, idx[n + 1]]
        if pos + 1 < nshards:
            dcn[:, idx[-1]] = dxn[:, idx[-1]] * g[order[pos + 1], :, 3]


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from linrec_b200 import sharded
        rows, L = 5, 96
        Ls = L // world
        g = torch.Generator().manual_seed(99)
        x = torch.randn(rows, L, generator=g, dtype=torch.float64)
        c = 0.6 + 0.4 * torch.rand(rows, L, generator=g, dtype=torch.float64)
        dy = torch.randn(rows, L, generator=g, dtype=torch.float64)
        k = NumpyShardKernels()
        sl = slice(rank * Ls, (rank + 1) * Ls)
        for rev in (False, True):
            y_full = oracle.fwd_f64(x.numpy().astype(np.float32), c.numpy().astype(np.float32), reverse=rev)
            x32, c32, dy32 = x.float().double(), c.float().double(), dy.float().double()
            y = sharded.seq_sharded_fwd(x32[:, sl].contiguous(), c32[:, sl].contiguous(), rev, None, k)
            np.testing.assert_allclose(y.numpy(), y_full[:, sl], rtol=5e-6, atol=5e-6)
            dx_full, dc_full = oracle.bwd_f64(dy.numpy().astype(np.float32), c.numpy().astype(np.float32), y_full, reverse=rev)
            ysh = torch.from_numpy(np.ascontiguousarray(y_full[:, sl]))
            dx, dc = sharded.seq_sharded_bwd(dy32[:, sl].contiguous(), c32[:, sl].contiguous(), ysh, rev, None, k)
            np.testing.assert_allclose(dx.numpy(), dx_full[:, sl], rtol=5e-6, atol=5e-6)
            np.testing.assert_allclose(dc.numpy(), dc_full[:, sl], rtol=5e-6, atol=5e-6)
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_sharding_host_logic_gloo(tmp_path, world):
    port = 29500 + (os.getpid() % 2000) + world
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_channel_sharding_is_the_plain_operator():
    from linrec_b200 import sharded
    import linrec_b200
    assert sharded.linrec_channel_sharded.__doc__
    # rows are independent: the sharded entry point must be the same operator, nothing added
    import inspect
    assert "linrec_pipe(inputs, coeffs, reverse)" in inspect.getsource(sharded.linrec_channel_sharded)
    assert linrec_b200.linrec is linrec_b200.linrec_pipe


def test_results_follow_the_row_layout_of_padded_inputs(monkeypatch):
    """Every tensor of a sharded call is addressed with ONE row stride.  Inputs whose rows are padded
    (row stride larger than the row) keep their layout, so the results must be allocated with that
    layout too; a contiguous result would be overrun by a kernel that steps from row to row with the
    inputs' stride.  Checked on CPU tensors with the CUDA-only precondition switched off."""
    from linrec_b200 import ops, sharded
    monkeypatch.setattr(sharded, "_check_same", lambda *ts: None)
    base = torch.zeros(5, 300)
    x, c = base[:, :256], torch.ones(5, 300)[:, :256]
    assert x.stride() == (300, 1) and torch.empty_like(x).stride() == (256, 1)   # what went wrong before
    (xp, cp), (numseq, seqlen, stride) = sharded.CudaShardKernels._prep(x, c)
    assert (numseq, seqlen, stride) == (5, 256, 300)
    for t in (xp, cp, ops._empty_like_rows(xp)):
        assert ops._row_layout(t) == (5, 256, 300)
    # batch dimensions in front of padded rows
    x3 = torch.zeros(2, 3, 40)[:, :, :32]
    out = ops._empty_like_rows(x3)
    assert out.stride() == x3.stride() and ops._row_layout(out) == (6, 32, 40)
    # no uniform row stride (a permuted batch): inputs are made contiguous, and so is the result
    xp = torch.zeros(4, 6, 8).permute(1, 0, 2)
    (a, b), lay = sharded.CudaShardKernels._prep(xp, xp.clone(memory_format=torch.preserve_format))
    assert lay == (24, 8, 8) and a.is_contiguous() and ops._empty_like_rows(a).is_contiguous()
    # inputs with different (individually valid) strides end up with one layout
    (a, b), lay = sharded.CudaShardKernels._prep(x, torch.zeros(5, 256))
    assert lay == (5, 256, 256) and a.stride() == b.stride()


def test_results_start_as_far_from_a_16_byte_boundary_as_their_inputs():
    """The kernel for rows of any alignment walks all tensors of a call in the same 16-byte chunks, so
    a result allocated for inputs that are views into a wider tensor has to start at the same offset
    from a 16-byte boundary (inside its own storage); aligned inputs get a plain allocation."""
    from linrec_b200 import ops
    for dtype, skew in ((torch.float32, 3), (torch.float32, 1), (torch.bfloat16, 5), (torch.bfloat16, 1), (torch.float64, 1)):
        wide = torch.zeros(6, 1000 + skew + 2, dtype=dtype)
        view = wide[:, skew:skew + 1000]
        if view.data_ptr() % 16 == 0:
            continue            # the allocation itself happened to start off a boundary by the same amount
        out = ops._empty_like_rows(view)
        assert out.shape == view.shape and out.stride() == view.stride() and out.dtype == dtype
        assert out.data_ptr() % 16 == view.data_ptr() % 16
        assert 0 < out.storage_offset() < 16
        out.fill_(1)            # every element is inside the allocation
        assert float(out.double().sum()) == 6 * 1000
    aligned = torch.zeros(6, 1000)
    out = ops._empty_like_rows(aligned)
    assert out.storage_offset() == 0 and out.stride() == aligned.stride()

