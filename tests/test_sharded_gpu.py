"""Sequence sharding on the GPU.

1. One GPU, all shards: the four C-ABI entry points are called for every shard in turn on slices of
   one tensor and the records are stacked by hand (what the all-gather would deliver).  No kernel
   waits for another launch, so this is safe on a single device.  Checked against the CPU oracle on
   the unsharded tensor at the fp32 tolerance of the suite.
2. Two or more GPUs (skipped otherwise): real ranks over NCCL through `linrec_seq_sharded` with
   autograd, checked against the single-device operator.
"""
import os
import sys

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-4, 1e-5
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _judge_against_f64(ours, seq32, truth64, what):
    """Acceptance for slowly decaying coefficients (c close to 1), where two valid fp32 evaluation
    orders already differ by more than rtol 1e-4 / atol 1e-5 near zero crossings: our error against
    the fp64 evaluation may be at most twice the sequential fp32 oracle's own error against it, and
    the share of elements that miss the nominal tolerance may be at most twice the sequential
    oracle's own share (or 1e-4, whichever is larger)."""
    err_ours = float(np.abs(ours - truth64).max())
    err_seq = float(np.abs(seq32 - truth64).max())
    assert err_ours <= 2.0 * err_seq + ATOL, f"{what}: error {err_ours:.3g} vs sequential fp32 error {err_seq:.3g}"
    miss = (np.abs(ours - truth64) > ATOL + RTOL * np.abs(truth64)).mean()
    miss_seq = (np.abs(seq32 - truth64) > ATOL + RTOL * np.abs(truth64)).mean()
    assert miss <= max(1e-4, 2.0 * miss_seq), f"{what}: {miss:.2e} of the elements miss the nominal tolerance (sequential fp32: {miss_seq:.2e})"


def _data(shape, clo, seed=5):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g), clo + (1 - clo) * torch.rand(shape, generator=g),
            torch.randn(shape, generator=g))


@pytest.mark.parametrize("rows,L,G,clo", [(6, 4 * 96, 4, 0.5), (3, 2 * 8192 * 3, 2, 0.9), (5, 3 * 2080, 3, 0.99),
                                          (130, 8 * 512, 8, 0.0), (2, 4 * 40001, 4, 0.999)],
                         ids=["short", "chained", "ragged", "many_rows", "slow_decay"])
@pytest.mark.parametrize("rev", [False, True])
def test_all_shards_on_one_gpu(rows, L, G, clo, rev):
    from linrec_b200.sharded import CudaShardKernels
    k = CudaShardKernels()
    dev = torch.device("cuda:0")
    x, c, dy = _data((rows, L), clo)
    Ls = L // G
    xs = [x[:, s * Ls:(s + 1) * Ls].contiguous().to(dev) for s in range(G)]
    cs = [c[:, s * Ls:(s + 1) * Ls].contiguous().to(dev) for s in range(G)]
    # forward
    ys, recs = zip(*[k.fwd_carry(xs[s], cs[s], rev, s, G) for s in range(G)])
    gathered = torch.stack(recs).contiguous()
    for s in range(G):
        k.fwd_fixup(xs[s], ys[s], cs[s], gathered, rev, s, G)
    y = torch.cat([t.cpu() for t in ys], dim=1).numpy()
    y_ref = oracle.fwd_f32(x.numpy(), c.numpy(), reverse=rev)
    y64 = oracle.fwd_f64(x.numpy(), c.numpy(), reverse=rev)
    if clo < 0.99:
        np.testing.assert_allclose(y, y_ref, rtol=RTOL, atol=ATOL)
    else:
        # slowly decaying coefficients: two valid fp32 orders differ by more than the nominal
        # tolerance near zero crossings, so the fp64 evaluation is the arbiter
        _judge_against_f64(y, y_ref, y64, "y")
    # backward, from the oracle's forward outputs
    yg = [torch.from_numpy(np.ascontiguousarray(y_ref[:, s * Ls:(s + 1) * Ls])).to(dev) for s in range(G)]
    dys = [dy[:, s * Ls:(s + 1) * Ls].contiguous().to(dev) for s in range(G)]
    outs = [k.bwd_carry(dys[s], cs[s], yg[s], rev, s, G) for s in range(G)]
    gathered = torch.stack([o[2] for o in outs]).contiguous()
    for s in range(G):
        k.bwd_fixup(dys[s], outs[s][0], outs[s][1], cs[s], yg[s], gathered, rev, s, G)
    dx = torch.cat([o[0].cpu() for o in outs], dim=1).numpy()
    dc = torch.cat([o[1].cpu() for o in outs], dim=1).numpy()
    if clo < 0.99:
        dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c.numpy(), y_ref, reverse=rev)
        np.testing.assert_allclose(dx, dx_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(dc, dc_ref, rtol=RTOL, atol=2 * ATOL * max(1.0, float(np.abs(y_ref).max())))
    else:
        dx64, dc64 = oracle.bwd_f64(dy.numpy(), c.numpy(), y_ref.astype(np.float64), reverse=rev)
        dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c.numpy(), y_ref, reverse=rev)
        _judge_against_f64(dx, dx_ref, dx64, "dx")
        scale = max(1.0, float(np.abs(y_ref).max()))   # dc = dx * y: judge it per unit of |y|
        _judge_against_f64(dc / scale, dc_ref / scale, dc64 / scale, "dc")
    import linrec_b200
    linrec_b200.check_status()


def _fwd_all_shards(x, c, G, rev=False):
    from linrec_b200.sharded import CudaShardKernels
    k = CudaShardKernels()
    dev = torch.device("cuda:0")
    Ls = x.shape[1] // G
    xs = [x[:, s * Ls:(s + 1) * Ls].contiguous().to(dev) for s in range(G)]
    cs = [c[:, s * Ls:(s + 1) * Ls].contiguous().to(dev) for s in range(G)]
    ys, recs = zip(*[k.fwd_carry(xs[s], cs[s], rev, s, G) for s in range(G)])
    gathered = torch.stack(recs).contiguous()
    for s in range(G):
        k.fwd_fixup(xs[s], ys[s], cs[s], gathered, rev, s, G)
    return torch.cat([t.cpu() for t in ys], dim=1).numpy()


@pytest.mark.parametrize("case", ["random", "impulse", "inf", "nan", "regrowth", "tiny_values"])
def test_the_walk_may_end_early_only_where_nothing_is_lost(case):
    """The fix-up walk along a row ends where the entering carry's remaining contribution is exactly zero or
    below a quarter ulp of the true value.  Shards of 32768 elements with c ~ U(0.99, 1): the second rule
    ends the walk after ~4 k elements.  The results must be as good as the unsharded operator's (judged
    against fp64), an impulse's tail must keep its relative accuracy down to 1e-37, a non-finite
    carry must travel on exactly as in the sequential evaluation, and a later stretch of c > 1 must not
    bring back anything that was dropped."""
    import linrec_b200
    rows, G, Ls = 4, 2, 32768
    L = G * Ls
    x, c, _ = _data((rows, L), 0.99, seed=11)
    rtol, atol = 1e-4, 1e-5
    if case == "impulse":
        x = torch.zeros_like(x)
        x[:, 5] = 1.0
        c = 0.998 + 0.1 * (c - 0.99)          # U(0.998, 0.999): the product over a row is ~ 2e-43, down in the subnormals,
        atol = 1e-37                          # where an fp32 chain stalls (y * c rounds back to y): judged above them
    elif case == "inf":
        x[1, Ls - 7] = float("inf")
    elif case == "nan":
        x[2, 3] = float("nan")
    elif case == "regrowth":
        c[:, Ls + 8000:Ls + 16000] = 1.002     # e^16 ~ 9e6 after the walk has ended
    elif case == "tiny_values":
        x[:, Ls:] *= 1e-30                     # behind the boundary the carry's tail is all there is for a long while
        atol = 1e-33
    y = _fwd_all_shards(x, c, G)
    y64 = oracle.fwd_f64(x.numpy(), c.numpy())
    y32 = oracle.fwd_f32(x.numpy(), c.numpy())
    if case in ("inf", "nan"):
        np.testing.assert_array_equal(np.isfinite(y), np.isfinite(y32))
        np.testing.assert_array_equal(np.isnan(y), np.isnan(y32))
        ok = np.isfinite(y32)
        _judge_against_f64(y[ok], y32[ok], y64[ok], "y (finite part)")
    elif case == "impulse":
        np.testing.assert_allclose(y, y64, rtol=rtol, atol=atol)
    elif case == "tiny_values":
        _judge_against_f64(y[:, :Ls], y32[:, :Ls], y64[:, :Ls], "y (first shard)")
        # second shard: the carry's tail (from ~10 down to where the 1e-29-sized local values take over) at
        # the relative tolerance all the way; 2048 elements behind the boundary are still dominated by
        # values of ordinary size with their ordinary absolute error
        np.testing.assert_allclose(y[:, Ls:Ls + 2048], y64[:, Ls:Ls + 2048], rtol=rtol, atol=1e-5)
        np.testing.assert_allclose(y[:, Ls + 2048:], y64[:, Ls + 2048:], rtol=rtol, atol=atol)
    else:
        if case == "random":
            _judge_against_f64(y, y32, y64, "y")
        # no worse than the unsharded operator on the device (through a stretch of c > 1 every tiled
        # evaluation loses more than the sequential one, sharded or not)
        dev = torch.device("cuda:0")
        y1 = linrec_b200._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=c.to(dev)).cpu().numpy()
        assert np.abs(y - y64).max() <= 1.5 * np.abs(y1 - y64).max() + 1e-6 * np.abs(y64).max()
    linrec_b200.check_status()


@pytest.mark.parametrize("rows,L,G,clo", [(6, 4 * 96, 4, 0.5), (3, 2 * 8192 * 3, 2, 0.9), (5, 3 * 2080, 3, 0.99), (40, 8 * 512, 8, 0.3)],
                         ids=["short", "chained", "ragged", "eight"])
def test_peer_exchange_all_ranks_on_one_gpu(rows, L, G, clo):
    """The peer-memory path with every "rank" on one device: G exchange buffers in local memory, scan
    phase of all ranks first, then the fix-up phase of all ranks (so no launch ever waits for a later
    one).  Four exchanges in a row (forward and backward, both directions) exercise slot reuse and the
    acknowledgements."""
    import ctypes
    from linrec_b200 import _capi
    dev = torch.device("cuda:0")
    nbytes = _capi.lib.linrec_b200_exchange_size(rows, G)
    assert nbytes > 0
    bufs = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(G)]
    x, c, dy = _data((rows, L), clo, seed=11)
    Ls = L // G
    cut = lambda t, s: t[:, s * Ls:(s + 1) * Ls].contiguous().to(dev)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(_capi.lib.linrec_b200_workspace_size(rows, Ls, 0), dtype=torch.uint8, device=dev)
    ptrs = (ctypes.c_void_p * G)(*[b.data_ptr() for b in bufs])
    for s in range(G):
        assert _capi.lib.linrec_b200_exchange_init(bufs[s].data_ptr(), ptrs, s, G, rows, stream) == 0
    epoch = 0
    for rev in (False, True, False):
        y_ref = oracle.fwd_f32(x.numpy(), c.numpy(), reverse=rev)
        dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c.numpy(), y_ref, reverse=rev)
        xs, cs, dys = ([cut(t, s) for s in range(G)] for t in (x, c, dy))
        ygs = [cut(torch.from_numpy(y_ref), s) for s in range(G)]
        ys = [torch.empty_like(t) for t in xs]
        dxs, dcs = [torch.empty_like(t) for t in xs], [torch.empty_like(t) for t in xs]
        epoch += 1
        for phase in (1, 2):
            o, keep = _capi.make_opts({"p2pPhase": phase})
            for s in range(G):
                rc = _capi.lib.linrec_b200_fwd_seq_p2p(xs[s].data_ptr(), cs[s].data_ptr(), ys[s].data_ptr(), rows, Ls, Ls,
                                                       int(rev), 0, s, G, bufs[s].data_ptr(), epoch, o, ws.data_ptr(), ws.numel(), stream)
                assert rc == 0, _capi.strerror(rc)
        epoch += 1
        for phase in (1, 2):
            o, keep = _capi.make_opts({"p2pPhase": phase})
            for s in range(G):
                rc = _capi.lib.linrec_b200_bwd_seq_p2p(dys[s].data_ptr(), cs[s].data_ptr(), ygs[s].data_ptr(), dxs[s].data_ptr(),
                                                       dcs[s].data_ptr(), rows, Ls, Ls, int(rev), 0, s, G, bufs[s].data_ptr(), epoch, o,
                                                       ws.data_ptr(), ws.numel(), stream)
                assert rc == 0, _capi.strerror(rc)
        torch.cuda.synchronize()
        assert _capi.lib.linrec_b200_status(ws.data_ptr(), stream) == 0
        cat = lambda ts: torch.cat([t.cpu() for t in ts], dim=1).numpy()
        np.testing.assert_allclose(cat(ys), y_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(cat(dxs), dx_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(cat(dcs), dc_ref, rtol=RTOL, atol=2 * ATOL * max(1.0, float(np.abs(y_ref).max())))


@pytest.mark.parametrize("rev", [False, True])
def test_padded_rows_stay_inside_their_allocation(rev):
    """Inputs whose rows are padded (row stride 300, row length 256): the sharded entry points must
    allocate their results with the same layout and leave the padding and everything around it alone.
    The padding of the inputs is poisoned with NaN, so a kernel that read it would show."""
    from linrec_b200.sharded import CudaShardKernels
    k = CudaShardKernels()
    dev = torch.device("cuda:0")
    rows, L, stride, G = 5, 2 * 256, 300, 2
    x, c, dy = _data((rows, L), 0.5, seed=21)
    Ls = L // G

    def padded(t):
        buf = torch.full((rows, stride), float("nan"), device=dev)
        buf[:, :Ls] = t.to(dev)
        return buf[:, :Ls]

    xs, cs, dys = ([padded(t[:, s * Ls:(s + 1) * Ls]) for s in range(G)] for t in (x, c, dy))
    ys, recs = zip(*[k.fwd_carry(xs[s], cs[s], rev, s, G) for s in range(G)])
    for y in ys:
        assert y.stride() == (stride, 1) and y.untyped_storage().nbytes() >= ((rows - 1) * stride + Ls) * 4
    gathered = torch.stack(recs).contiguous()
    for s in range(G):
        k.fwd_fixup(xs[s], ys[s], cs[s], gathered, rev, s, G)
    y_ref = oracle.fwd_f32(x.numpy(), c.numpy(), reverse=rev)
    np.testing.assert_allclose(torch.cat([t.cpu() for t in ys], dim=1).numpy(), y_ref, rtol=RTOL, atol=ATOL)
    yg = [padded(torch.from_numpy(y_ref[:, s * Ls:(s + 1) * Ls])) for s in range(G)]
    outs = [k.bwd_carry(dys[s], cs[s], yg[s], rev, s, G) for s in range(G)]
    gathered = torch.stack([o[2] for o in outs]).contiguous()
    for s in range(G):
        assert outs[s][0].stride() == (stride, 1) and outs[s][1].stride() == (stride, 1)
        k.bwd_fixup(dys[s], outs[s][0], outs[s][1], cs[s], yg[s], gathered, rev, s, G)
    dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c.numpy(), y_ref, reverse=rev)
    np.testing.assert_allclose(torch.cat([o[0].cpu() for o in outs], dim=1).numpy(), dx_ref, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(torch.cat([o[1].cpu() for o in outs], dim=1).numpy(), dc_ref, rtol=RTOL,
                               atol=2 * ATOL * max(1.0, float(np.abs(y_ref).max())))
    import linrec_b200
    linrec_b200.check_status()


@pytest.mark.parametrize("rev", [False, True])
def test_fixup_follows_a_carry_through_a_dip(rev):
    """The operator does not restrict its coefficients: a carry may shrink below the normal range
    (39 steps of c = 0.1) and grow back (39 steps of c = 10).  The fix-up walk must not give up while
    the carried value is merely tiny -- only at exact zero.  The second shard has x = 0, so everything
    it holds IS the correction."""
    from linrec_b200.sharded import CudaShardKernels
    k = CudaShardKernels()
    dev = torch.device("cuda:0")
    rows, Ls, G = 4, 256, 2
    g = torch.Generator(device="cpu").manual_seed(3)
    x = torch.randn(rows, G * Ls, generator=g)
    c = 0.5 + 0.5 * torch.rand(rows, G * Ls, generator=g)
    dip = torch.cat([torch.full((39,), 0.1), torch.full((39,), 10.0), torch.full((Ls - 78,), 0.9)])
    second = slice(0, Ls) if rev else slice(Ls, 2 * Ls)          # the shard that comes second in scan order
    x[:, second] = 0.0
    c[:, second] = dip.flip(0) if rev else dip
    cut = lambda t, s: t[:, s * Ls:(s + 1) * Ls].contiguous().to(dev)
    ys, recs = zip(*[k.fwd_carry(cut(x, s), cut(c, s), rev, s, G) for s in range(G)])
    gathered = torch.stack(recs).contiguous()
    for s in range(G):
        k.fwd_fixup(cut(x, s), ys[s], cut(c, s), gathered, rev, s, G)
    y = torch.cat([t.cpu() for t in ys], dim=1).numpy()
    y64 = oracle.fwd_f64(x.numpy(), c.numpy(), reverse=rev)
    # at the bottom of the dip the values are subnormal and keep only ~19 bits: rtol 1e-4 holds, atol does not apply
    np.testing.assert_allclose(y, y64, rtol=1e-4, atol=1e-37)
    far = y[:, 0] if rev else y[:, -1]
    assert np.all(np.abs(far) > 1e-12), "the carry was dropped inside the dip"


def test_wait_for_a_peer_gives_up_with_status():
    """The fix-up phase of the peer-memory path is run for shard 1 without anybody ever flagging shard
    0's records as complete: its bounded waits (option peerWaitBudgetMs, 20 ms here) must run out by themselves,
    set the status word of the workspace and leave the context usable."""
    import ctypes
    from linrec_b200 import _capi
    dev = torch.device("cuda:0")
    rows, Ls, G = 3, 4096, 2
    nbytes = _capi.lib.linrec_b200_exchange_size(rows, G)
    bufs = [torch.empty(nbytes, dtype=torch.uint8, device=dev) for _ in range(G)]
    ptrs = (ctypes.c_void_p * G)(*[b.data_ptr() for b in bufs])
    stream = torch.cuda.current_stream().cuda_stream
    for s in range(G):
        assert _capi.lib.linrec_b200_exchange_init(bufs[s].data_ptr(), ptrs, s, G, rows, stream) == 0
    ws = torch.zeros(_capi.lib.linrec_b200_workspace_size(rows, Ls, 0), dtype=torch.uint8, device=dev)
    x = torch.ones(rows, Ls, device=dev)
    y = torch.zeros_like(x)
    o, keep = _capi.make_opts({"p2pPhase": 2, "peerWaitBudgetMs": 20})
    rc = _capi.lib.linrec_b200_fwd_seq_p2p(x.data_ptr(), x.data_ptr(), y.data_ptr(), rows, Ls, Ls, 0, 0, 1, G,
                                           bufs[1].data_ptr(), 1, o, ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, _capi.strerror(rc)
    assert _capi.lib.linrec_b200_status(ws.data_ptr(), stream) == _capi.ERR_TIMEOUT
    assert _capi.lib.linrec_b200_status(ws.data_ptr(), stream) == 0
    import linrec_b200
    assert torch.isfinite(linrec_b200.linrec(x, x * 0.5)).all()
    linrec_b200.check_status()


def _nccl_worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import linrec_b200
        from linrec_b200.sharded import PeerExchange, linrec_seq_sharded
        rows, L = 1024, world * 3 * 4096
        exchange = PeerExchange(rows)
        Ls = L // world
        x, c, dy = _data((rows, L), 0.9, seed=77)
        c[rows // 2:] = 0.999 + 0.001 * c[rows // 2:]        # half of the rows decay slowly: carries cross whole shards
        sl = slice(rank * Ls, (rank + 1) * Ls)
        for rev in (False, True):
            xf, cf = x.to(dev).requires_grad_(True), c.to(dev).requires_grad_(True)
            y_full = linrec_b200.linrec(xf, cf, reverse=rev)
            gx_full, gc_full = torch.autograd.grad(y_full, (xf, cf), dy.to(dev))
            xs = x[:, sl].contiguous().to(dev).requires_grad_(True)
            cs = c[:, sl].contiguous().to(dev).requires_grad_(True)
            ys = linrec_seq_sharded(xs, cs, reverse=rev)
            gx, gc = torch.autograd.grad(ys, (xs, cs), dy[:, sl].contiguous().to(dev))
            h = rows // 2
            # slowly decaying rows reach |y| ~ 30: two valid fp32 evaluation orders differ by a few ulp of
            # that near zero crossings, so their absolute tolerance is scaled by the size of the values
            ymax = max(1.0, float(y_full[h:].abs().max()))
            gmax = max(1.0, float(gx_full[h:].abs().max()))

            def close(got, want, scale=1.0):
                torch.testing.assert_close(got[:h], want[:h], rtol=RTOL, atol=4 * ATOL)
                torch.testing.assert_close(got[h:], want[h:], rtol=RTOL, atol=ATOL * scale)

            close(ys, y_full[:, sl], ymax)
            close(gx, gx_full[:, sl], gmax)
            close(gc, gc_full[:, sl], 4 * ymax * gmax)
            # the same through peer memory instead of the all-gather (several exchanges in a row)
            for _ in range(3):
                xs2 = xs.detach().clone().requires_grad_(True)
                cs2 = cs.detach().clone().requires_grad_(True)
                ys2 = linrec_seq_sharded(xs2, cs2, reverse=rev, exchange=exchange)
                gx2, gc2 = torch.autograd.grad(ys2, (xs2, cs2), dy[:, sl].contiguous().to(dev))
                # same kernels, same records: bit-identical to the all-gather path
                assert torch.equal(ys2, ys) and torch.equal(gx2, gx) and torch.equal(gc2, gc)
        exchange.poll(wait=True)
        linrec_b200.check_status()
        open(os.path.join(tmp, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_real_ranks_over_nccl(tmp_path):
    world = torch.cuda.device_count()
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp
    port = 29600 + os.getpid() % 1000
    mp.spawn(_nccl_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
