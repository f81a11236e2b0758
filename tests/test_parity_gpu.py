"""Parity of the CUDA path with the CPU oracle (GPU only; every call goes through the C ABI).

Tolerances (from the task definition): fp32  rtol 1e-4, atol 1e-5 against the fp32 oracle;
bf16 storage  rtol 2^-7, atol 1e-5 against the fp32 oracle run on the bf16-rounded inputs.
dc = dx * y_shifted carries the rounding of both factors, so its absolute tolerance is doubled.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import GOLDEN_CASES

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5
SEED = 12334567890


def _ops():
    import linrec_b200
    return linrec_b200


def _data(shape, clo=0.0, chi=1.0, seed=SEED, bwd=False):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(shape, generator=g)
    c = clo + (chi - clo) * torch.rand(shape, generator=g)
    dy = torch.randn(shape, generator=g)
    return x, c, dy


def _check_fwd_bwd(x, c, dy, rev, family="pipe", rtol=RTOL, atol=ATOL, **kw):
    lb = _ops()
    dev = torch.device("cuda:0")
    fwd = getattr(lb._C, f"linrec_{family}_fwd")
    bwd = getattr(lb._C, f"linrec_{family}_bwd")
    xd, cd, dyd = x.to(dev), c.to(dev), dy.to(dev)
    y = fwd(inputs=xd, coeffs=cd, reverse=rev, **kw)
    y_ref = oracle.fwd_f32(x.numpy(), c.numpy(), reverse=rev)
    np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=rtol, atol=atol)
    # backward from the oracle's forward outputs, so that the two checks are independent
    yd = torch.from_numpy(y_ref).to(dev)
    dx, dc = bwd(d_outputs=dyd, coeffs=cd, outputs=yd, reverse=rev, **kw)
    dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c.numpy(), y_ref, reverse=rev)
    np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=rtol, atol=atol)
    np.testing.assert_allclose(dc.cpu().numpy(), dc_ref, rtol=rtol, atol=2 * atol)
    lb.check_status()


# ---- golden fixtures recorded from the reference ---------------------------------------------------
@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("rev", [False, True])
@pytest.mark.parametrize("family", ["ref", "tile", "pipe"])
def test_golden(golden, name, rev, family):
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = (torch.from_numpy(golden[f"{name}/{k}"]).to(dev) for k in ("x", "c", "dy"))
    tag = f"{name}/rev{int(rev)}"
    y = getattr(lb._C, f"linrec_{family}_fwd")(inputs=x, coeffs=c, reverse=rev)
    np.testing.assert_allclose(y.cpu().numpy(), golden[f"{tag}/y"], rtol=RTOL, atol=ATOL)
    yg = torch.from_numpy(golden[f"{tag}/y"]).to(dev)
    dx, dc = getattr(lb._C, f"linrec_{family}_bwd")(d_outputs=dy, coeffs=c, outputs=yg, reverse=rev)
    np.testing.assert_allclose(dx.cpu().numpy(), golden[f"{tag}/dx"], rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(dc.cpu().numpy(), golden[f"{tag}/dc"], rtol=RTOL, atol=2 * ATOL)
    lb.check_status()


# ---- shapes: short, ragged, tile-sized, chained, with every direction ------------------------------
SHAPES = [
    (1, 1), (7, 1), (5, 2), (3, 15), (3, 16), (3, 17), (4, 31), (9, 32), (9, 33), (2, 64), (11, 96),
    (6, 100), (300, 128), (37, 160), (129, 256), (5, 1000), (64, 1024), (3, 2047), (3, 2048), (3, 2049),
    (17, 4096), (2, 4097), (5, 4128), (3, 6144), (4, 8192), (2, 12288 + 32), (3, 20000), (2, 65536),
    (1, 1 << 18),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
def test_pipe_shapes(shape, rev):
    x, c, dy = _data(shape)
    _check_fwd_bwd(x, c, dy, rev)


@pytest.mark.parametrize("shape", [(512, 4096)], ids=["cfg1_512x4096"])
def test_config1_forward(shape):
    """The reference's own CPU-runnable case: forward, reverse=False, (512, 4096)."""
    x, c, dy = _data(shape)
    _check_fwd_bwd(x, c, dy, False)


@pytest.mark.parametrize("rev", [False, True])
def test_slow_decay_coefficients(rev):
    """c ~ U(0.9, 1): carries survive for thousands of steps, so chained tiles really matter."""
    x, c, dy = _data((6, 3 * 8192), clo=0.9, chi=1.0)
    _check_fwd_bwd(x, c, dy, rev)


def test_three_dim_batch_autograd():
    """(batch, channel, length) through autograd, against the oracle's analytic backward."""
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data((3, 5, 777), clo=0.9, chi=1.0)
    for rev in (False, True):
        xd = x.to(dev).requires_grad_(True)
        cd = c.to(dev).requires_grad_(True)
        y = lb.linrec(xd, cd, reverse=rev)
        gx, gc = torch.autograd.grad(y, (xd, cd), dy.to(dev))
        y_ref = oracle.fwd_f32(x.numpy(), c.numpy(), reverse=rev)
        dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c.numpy(), y_ref, reverse=rev)
        np.testing.assert_allclose(y.detach().cpu().numpy(), y_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(gx.cpu().numpy(), dx_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(gc.cpu().numpy(), dc_ref, rtol=RTOL, atol=2 * ATOL)


# ---- bf16 storage, fp32 arithmetic -----------------------------------------------------------------
BF16_RTOL = 2.0 ** -7


@pytest.mark.parametrize("shape", [(64, 512), (300, 64), (5, 3 * 8192), (3, 1000), (7, 4097), (16, 65536), (2, 2 * 8192 + 64)],
                         ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
def test_bf16_storage(shape, rev, dtype):
    """Inputs rounded to 2-byte storage; the oracle runs in fp32 on the upcast inputs; our outputs are
    fp32 accumulations rounded once to the storage type.  bf16 (8 significant bits, rounding <= 2^-9):
    rtol 2^-7 / atol 1e-5; fp16 (11 bits, rounding <= 2^-12): rtol 2^-9 / atol 1e-5."""
    lb = _ops()
    dev = torch.device("cuda:0")
    BF16_RTOL = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -9
    x, c, dy = (t.to(dtype) for t in _data(shape, clo=0.5, chi=1.0))
    y = lb._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=rev)
    assert y.dtype == dtype
    y_ref = oracle.fwd_f32(x.float().numpy(), c.float().numpy(), reverse=rev)
    np.testing.assert_allclose(y.float().cpu().numpy(), y_ref, rtol=BF16_RTOL, atol=ATOL)
    yb = torch.from_numpy(y_ref).to(dtype)
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy.to(dev), coeffs=c.to(dev), outputs=yb.to(dev), reverse=rev)
    dx_ref, dc_ref = oracle.bwd_f32(dy.float().numpy(), c.float().numpy(), yb.float().numpy(), reverse=rev)
    np.testing.assert_allclose(dx.float().cpu().numpy(), dx_ref, rtol=BF16_RTOL, atol=ATOL)
    np.testing.assert_allclose(dc.float().cpu().numpy(), dc_ref, rtol=BF16_RTOL, atol=2 * ATOL)
    # the sequential operator and every bulk-copy variant agree on bf16 as well
    y_seq = lb._C.linrec_ref_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=rev)
    np.testing.assert_allclose(y_seq.float().cpu().numpy(), y_ref, rtol=BF16_RTOL, atol=ATOL)
    lb.check_status()


def test_tile_family_refuses_rows_longer_than_a_tile():
    """The tile family keeps a whole row in one tile; the largest tile holds 8192 fp32 elements
    whichever loader the row's length and alignment select."""
    lb = _ops()
    dev = torch.device("cuda:0")
    for L, fits in [(2049, True), (2100, True), (8192 + 4, False), (8192 - 4, True), (8191, True), (8193, False)]:
        x, c, _ = _data((2, L))
        if fits:
            y = lb._C.linrec_tile_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=False)
            np.testing.assert_allclose(y.cpu().numpy(), oracle.fwd_f32(x.numpy(), c.numpy()), rtol=RTOL, atol=ATOL)
        else:
            with pytest.raises(RuntimeError, match="does not fit one tile"):
                lb._C.linrec_tile_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=False)


# ---- rows of whole 16-byte chunks that are not whole 128-byte lines: the cp.async kernel --------------
@pytest.mark.parametrize("shape", [(7, 100), (300, 36), (33, 1000), (5, 2100), (3, 10000), (2, 50004), (1, 4)],
                         ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
def test_async_copy_kernel(shape, rev):
    lb = _ops()
    x, c, dy = _data(shape, clo=0.5, chi=1.0)
    attrs = lb._C.linrec_pipe_attrs(fwd=True, memcode=2)
    assert attrs["memcode"] == 2 and attrs["kStages"] == 2
    for kw in ({}, {"memcode": 2}, {"memcode": 2, "kThreadsPerBlock": 128}, {"memcode": 2, "kThreadsPerBlock": 512},
               {"memcode": 0}):
        _check_fwd_bwd(x, c, dy, rev, **kw)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("shape", [(9, 200), (4, 4104), (2, 20008)], ids=lambda s: f"{s[0]}x{s[1]}")
def test_async_copy_kernel_two_byte(dtype, shape):
    """2-byte storage through the cp.async kernel against the plain-load kernel (same tile algebra,
    same tile size: bit for bit where a row is one tile) and against the oracle."""
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data(shape, clo=0.5, chi=1.0)
    xd, cd, dyd = x.to(dev, dtype), c.to(dev, dtype), dy.to(dev, dtype)
    for rev in (False, True):
        ya = lb._C.linrec_pipe_fwd(inputs=xd, coeffs=cd, reverse=rev, memcode=2, kThreadsPerBlock=128)
        yg = lb._C.linrec_pipe_fwd(inputs=xd, coeffs=cd, reverse=rev, memcode=0, kElemsPerThread=16)
        da = lb._C.linrec_pipe_bwd(d_outputs=dyd, coeffs=cd, outputs=yg, reverse=rev, memcode=2, kThreadsPerBlock=128)
        dg = lb._C.linrec_pipe_bwd(d_outputs=dyd, coeffs=cd, outputs=yg, reverse=rev, memcode=0, kElemsPerThread=16)
        if shape[1] <= 2048:
            # one tile per row: no look-back, whose order of combination depends on timing
            assert torch.equal(ya, yg)
            assert torch.equal(da[0], dg[0]) and torch.equal(da[1], dg[1])
        else:
            for a, b in ((ya, yg), (da[0], dg[0]), (da[1], dg[1])):
                np.testing.assert_allclose(a.float().cpu().numpy(), b.float().cpu().numpy(), rtol=2e-2, atol=2e-2)
        yd = lb._C.linrec_pipe_fwd(inputs=xd, coeffs=cd, reverse=rev)
        ref = oracle.fwd_f32(xd.float().cpu().numpy(), cd.float().cpu().numpy(), reverse=rev)
        np.testing.assert_allclose(yd.float().cpu().numpy(), ref, rtol=2e-2, atol=2e-2)
    lb.check_status()


def test_async_copy_kernel_refuses_unaligned_rows():
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, _ = _data((4, 1001))
    with pytest.raises(RuntimeError):
        lb._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=False, memcode=2)


# ---- rows of whole 4-byte words: the 4-byte cp.async kernel -------------------------------------------
@pytest.mark.parametrize("shape", [(7, 101), (300, 37), (33, 1001), (5, 2101), (3, 10001), (2, 50003), (1, 3), (9, 1),
                                   (2, 3 * 8192 + 1), (40, 4097)], ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
def test_word_copy_kernel(shape, rev):
    """fp32 rows of any length (here: odd lengths, which no 16-byte path can take) go through 4-byte
    cp.async copies (memcode 3, the default for them); every variant of that loader, the lazy-ticket
    mode and the plain-load kernel (memcode 0) must agree with the oracle."""
    lb = _ops()
    x, c, dy = _data(shape, clo=0.3)
    attrs = lb._C.linrec_pipe_attrs(fwd=True, memcode=3)
    assert attrs["memcode"] == 3 and attrs["kStages"] == 2
    for kw in ({}, {"memcode": 3, "kThreadsPerBlock": 128}, {"memcode": 3, "kThreadsPerBlock": 256},
               {"memcode": 3, "kThreadsPerBlock": 512}, {"memcode": 3, "kThreadsPerBlock": 512, "lazyTickets": 1},
               {"memcode": 0}):
        _check_fwd_bwd(x, c, dy, rev, **kw)


def test_word_copy_kernel_views_and_two_byte_rows():
    """Views that start at an odd element and rows with padding between them (fp32), and even-length
    rows of 2-byte elements at 4-byte aligned addresses; a 2-byte row that starts at an odd element
    has no 4-byte path and falls to the plain-load kernel."""
    lb = _ops()
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(17)
    for (rows, L, stride, off) in [(5, 255, 255, 1), (5, 1001, 1003, 3), (3, 9001, 9002, 1), (4, 20001, 20001, 0)]:
        big_x = torch.randn(rows * stride + off + 8, generator=g)
        big_c = torch.rand(rows * stride + off + 8, generator=g)
        big_dy = torch.randn(rows * stride + off + 8, generator=g)
        view = lambda t: torch.as_strided(t, (rows, L), (stride, 1), off)
        xh, ch, dyh = (view(t).contiguous() for t in (big_x, big_c, big_dy))
        for rev in (False, True):
            xv, cv, dyv = (view(t.to(dev)) for t in (big_x, big_c, big_dy))
            y = lb._C.linrec_pipe_fwd(inputs=xv, coeffs=cv, reverse=rev, memcode=3)
            y_ref = oracle.fwd_f32(xh.numpy(), ch.numpy(), reverse=rev)
            np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=RTOL, atol=ATOL)
            dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dyv, coeffs=cv, outputs=y, reverse=rev, memcode=3)
            dx_ref, dc_ref = oracle.bwd_f32(dyh.numpy(), ch.numpy(), y.cpu().numpy(), reverse=rev)
            np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=RTOL, atol=ATOL)
            np.testing.assert_allclose(dc.cpu().numpy(), dc_ref, rtol=RTOL, atol=2 * ATOL)
    for dtype in (torch.bfloat16, torch.float16):
        rtol = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -9
        for shape in [(9, 202), (4, 4102), (2, 20006)]:
            x, c, dy = (t.to(dtype) for t in _data(shape, clo=0.5))
            for rev in (False, True):
                y = lb._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=rev, memcode=3)
                y_ref = oracle.fwd_f32(x.float().numpy(), c.float().numpy(), reverse=rev)
                np.testing.assert_allclose(y.float().cpu().numpy(), y_ref, rtol=rtol, atol=ATOL)
                dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy.to(dev), coeffs=c.to(dev), outputs=y, reverse=rev, memcode=3)
                dx_ref, dc_ref = oracle.bwd_f32(dy.float().numpy(), c.float().numpy(), y.float().cpu().numpy(), reverse=rev)
                np.testing.assert_allclose(dx.float().cpu().numpy(), dx_ref, rtol=rtol, atol=ATOL)
                np.testing.assert_allclose(dc.float().cpu().numpy(), dc_ref, rtol=rtol, atol=2 * ATOL)
        odd = torch.zeros(2 * 101 + 1, dtype=dtype, device=dev)[1:].view(2, 101)
        with pytest.raises(RuntimeError):
            lb._C.linrec_pipe_fwd(inputs=odd, coeffs=odd, reverse=False, memcode=3)
        assert lb.linrec(odd, odd).shape == (2, 101)
    lb.check_status()


# ---- every compiled variant ------------------------------------------------------------------------
def _variants():
    lb = _ops()
    return lb._C.config_names, lb._C.config_list


@pytest.mark.parametrize("shape", [(40, 512), (3, 4096 * 5), (2, 8192 * 3 + 4096)], ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
def test_all_variants(shape, rev):
    names, configs = _variants()
    x, c, dy = _data(shape, clo=0.5, chi=1.0)
    assert len(configs) >= 4
    for cfg in configs:
        E, NT, S, OB, memcode = cfg
        if memcode == 1 and (E * NT * 4 * (3 * S + 2 * OB) + 1024 > 227 * 1024 or E * NT * 4 > 256 * 128):
            # the backward pass of this variant needs more shared memory than an SM has
            with pytest.raises(NotImplementedError):
                _check_fwd_bwd(x, c, dy, rev, **dict(zip(names, cfg)))
            continue
        _check_fwd_bwd(x, c, dy, rev, **dict(zip(names, cfg)))


def test_programmatic_launch_on_and_off_agree():
    """The scan kernels are launched so that their prologue may overlap the tail of the kernel before
    them (they wait before their first access to global memory).  Back-to-back launches that depend on
    each other -- forward, then backward on its output, repeated on one workspace, chained rows and rows
    that share a tile, super-chunks with their fix-up kernel -- must give bit-identical results with the
    overlap on (default) and off."""
    lb = _ops()
    dev = torch.device("cuda:0")
    for shape in [(300, 512), (64, 3 * 8192 + 64), (33, 1000), (7, 10001), (3, 1 << 18)]:
        x, c, dy = (t.to(dev) for t in _data(shape, clo=0.8))
        outs = {}
        for pdl in (1, 0):
            res = []
            for _ in range(4):
                y = lb._C.linrec_pipe_fwd(inputs=x, coeffs=c, reverse=False, programmaticLaunch=pdl)
                dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy, coeffs=c, outputs=y, reverse=False, programmaticLaunch=pdl)
                y2 = lb._C.linrec_pipe_fwd(inputs=dx, coeffs=c, reverse=True, programmaticLaunch=pdl)    # reads what was just written
                res.append((y, dx, dc, y2))
            torch.cuda.synchronize()
            for r in res[1:]:
                assert all(torch.equal(a, b) for a, b in zip(r, res[0]))
            outs[pdl] = res[0]
        assert all(torch.equal(a, b) for a, b in zip(outs[1], outs[0]))
        np.testing.assert_allclose(outs[1][0].cpu().numpy(), oracle.fwd_f32(x.cpu().numpy(), c.cpu().numpy()), rtol=RTOL, atol=ATOL)
    lb.check_status()


# ---- layouts ---------------------------------------------------------------------------------------
def test_unaligned_base_and_row_stride():
    """Views that start one element into an allocation and rows with padding between them."""
    lb = _ops()
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(7)
    for (rows, L, stride, off) in [(5, 256, 256, 1), (5, 256, 300, 0), (4, 4096, 4100, 3), (3, 9000, 9001, 1)]:
        big_x = torch.randn(rows * stride + off + 8, generator=g)
        big_c = torch.rand(rows * stride + off + 8, generator=g)
        xv = torch.as_strided(big_x.to(dev), (rows, L), (stride, 1), off)
        cv = torch.as_strided(big_c.to(dev), (rows, L), (stride, 1), off)
        xh = torch.as_strided(big_x, (rows, L), (stride, 1), off).contiguous()
        ch = torch.as_strided(big_c, (rows, L), (stride, 1), off).contiguous()
        for rev in (False, True):
            y = lb.linrec(xv, cv, reverse=rev)
            np.testing.assert_allclose(y.cpu().numpy(), oracle.fwd_f32(xh.numpy(), ch.numpy(), reverse=rev),
                                       rtol=RTOL, atol=ATOL)


def test_permuted_batch_dims():
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, _ = _data((4, 6, 200))
    xp, cp = x.to(dev).permute(1, 0, 2), c.to(dev).permute(1, 0, 2)
    y = lb.linrec(xp, cp)
    ref = oracle.fwd_f32(x.permute(1, 0, 2).contiguous().numpy(), c.permute(1, 0, 2).contiguous().numpy())
    np.testing.assert_allclose(y.cpu().numpy(), ref, rtol=RTOL, atol=ATOL)


def test_autograd_through_padded_rows():
    """Rows with a stride larger than their length, through autograd: outputs and gradients keep the
    layout of the inputs (the reference's backward fails its equal-strides check in this situation,
    linrec/impl/cuda/ops.py:55 with linrec_pipe.cu:98), and nothing is written into the padding."""
    lb = _ops()
    dev = torch.device("cuda:0")
    rows, L, stride = 6, 1000, 1024
    x, c, dy = _data((rows, L), clo=0.5)
    for rev in (False, True):
        bx = torch.full((rows, stride), -777.0, device=dev)
        bc = torch.full((rows, stride), -777.0, device=dev)
        bx[:, :L], bc[:, :L] = x.to(dev), c.to(dev)
        xd, cd = bx[:, :L].requires_grad_(True), bc[:, :L].requires_grad_(True)
        y = lb.linrec(xd, cd, reverse=rev)
        assert y.stride() == (stride, 1)
        gx, gc = torch.autograd.grad(y, (xd, cd), dy.to(dev))          # a contiguous incoming gradient
        y_ref = oracle.fwd_f32(x.numpy(), c.numpy(), reverse=rev)
        dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c.numpy(), y_ref, reverse=rev)
        np.testing.assert_allclose(y.detach().cpu().numpy(), y_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(gx.cpu().numpy(), dx_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(gc.cpu().numpy(), dc_ref, rtol=RTOL, atol=2 * ATOL)
    lb.check_status()


def test_guard_bands_untouched():
    """Outputs are written into the middle of a sentinel-filled allocation through the C ABI; the
    bytes before and after every row block must keep the sentinel (no out-of-row writes)."""
    import ctypes
    from linrec_b200 import _capi
    dev = torch.device("cuda:0")
    for (rows, L, stride) in [(7, 100, 100), (5, 4096, 4096), (3, 8192 + 64, 8192 + 64), (6, 333, 340)]:
        for bwd in (False, True):
            for rev in (False, True):
                x, c, dy = _data((rows, stride))
                pad = 1024
                n = rows * stride
                outs = [torch.full((n + 2 * pad,), -777.0, device=dev) for _ in range(2)]
                xd, cd, dyd = x.to(dev), c.to(dev), dy.to(dev)
                ws_bytes = _capi.lib.linrec_b200_workspace_size(rows, L, 0)
                ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)
                stream = torch.cuda.current_stream().cuda_stream
                o0 = outs[0].data_ptr() + 4 * pad
                o1 = outs[1].data_ptr() + 4 * pad
                if not bwd:
                    rc = _capi.lib.linrec_b200_fwd(_capi.KIND_PIPE, xd.data_ptr(), cd.data_ptr(), o0, rows, L, stride,
                                                   int(rev), 0, None, ws.data_ptr(), ws_bytes, stream)
                else:
                    rc = _capi.lib.linrec_b200_bwd(_capi.KIND_PIPE, dyd.data_ptr(), cd.data_ptr(), xd.data_ptr(), o0, o1,
                                                   rows, L, stride, int(rev), 0, None, ws.data_ptr(), ws_bytes, stream)
                assert rc == 0
                torch.cuda.synchronize()
                for o in outs[: 2 if bwd else 1]:
                    body = o[pad:pad + n].view(rows, stride)
                    assert torch.all(o[:pad] == -777.0) and torch.all(o[pad + n:] == -777.0)
                    if stride > L:
                        assert torch.all(body[:, L:] == -777.0)
                    assert not torch.any(body[:, :L] == -777.0)


def test_general_signature_logc_and_dim():
    """logc and dim of the reference's Python operator; gradients against fp64 autograd through the
    plain recurrence (the derivative of the forward that is actually computed)."""
    lb = _ops()
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(3)
    x = torch.randn(4, 300, 6, generator=g)
    logc = torch.log(0.5 + 0.5 * torch.rand(4, 300, 6, generator=g))
    dy = torch.randn(4, 300, 6, generator=g)
    for rev in (False, True):
        xd, ld = x.to(dev).requires_grad_(True), logc.to(dev).requires_grad_(True)
        y = lb.linrec_general(xd, ld, logc=True, dim=1, reverse=rev)
        gx, gl = torch.autograd.grad(y, (xd, ld), dy.to(dev))
        x64, l64 = x.double().requires_grad_(True), logc.double().requires_grad_(True)
        c64 = torch.exp(l64)
        prev = torch.zeros(4, 6, dtype=torch.float64)
        outs = [None] * 300
        for i in (range(299, -1, -1) if rev else range(300)):
            prev = prev * c64[:, i] + x64[:, i]
            outs[i] = prev
        y64 = torch.stack(outs, dim=1)
        rx, rl = torch.autograd.grad(y64, (x64, l64), dy.double())
        np.testing.assert_allclose(y.detach().cpu().numpy(), y64.detach().numpy(), rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(gx.cpu().numpy(), rx.numpy(), rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(gl.cpu().numpy(), rl.numpy(), rtol=RTOL, atol=2 * ATOL)


@pytest.mark.parametrize("shape", [(5, 64), (40, 512), (3, 4096 * 5), (7, 100), (33, 1000), (3, 10000), (5, 333), (2, 2101),
                                   (2, 8192 * 3 + 4096)], ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
def test_log_coefficients_fused(shape, rev):
    """Option logCoeffs: the kernels take log(c), apply exp while loading, and the backward kernels
    return d_c * c.  Checked for every loader (bulk copies, cp.async, plain loads, sequential) against
    the oracle run on c = exp(log c)."""
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data(shape, clo=0.3, chi=1.0)
    logc = torch.log(c)
    c_eff = torch.exp(logc)                      # what the kernels see, up to the rounding of exp
    y_ref = oracle.fwd_f32(x.numpy(), c_eff.numpy(), reverse=rev)
    dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c_eff.numpy(), y_ref, reverse=rev)
    dl_ref = dc_ref * c_eff.numpy()
    xd, ld, dyd, yd = x.to(dev), logc.to(dev), dy.to(dev), torch.from_numpy(y_ref).to(dev)
    fams = [("pipe", {}), ("ref", {}), ("pipe", {"memcode": 0})]
    if shape[1] % 4 == 0:
        fams.append(("pipe", {"memcode": 2}))
    for fam, kw in fams:
        y = getattr(lb._C, f"linrec_{fam}_fwd")(inputs=xd, coeffs=ld, reverse=rev, logCoeffs=1, **kw)
        np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=RTOL, atol=ATOL)
        dx, dl = getattr(lb._C, f"linrec_{fam}_bwd")(d_outputs=dyd, coeffs=ld, outputs=yd, reverse=rev, logCoeffs=1, **kw)
        np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(dl.cpu().numpy(), dl_ref, rtol=RTOL, atol=2 * ATOL)
    lb.check_status()


def test_log_coefficients_two_byte_and_first_element():
    lb = _ops()
    dev = torch.device("cuda:0")
    for dtype in (torch.bfloat16, torch.float16):
        for shape in [(6, 256), (3, 4104), (2, 40000)]:
            x, c, dy = _data(shape, clo=0.5, chi=1.0)
            xd, ld = x.to(dev, dtype), torch.log(c).to(dev, dtype)
            c_eff = torch.exp(ld.float()).cpu()
            for rev in (False, True):
                y = lb._C.linrec_pipe_fwd(inputs=xd, coeffs=ld, reverse=rev, logCoeffs=1)
                ref = oracle.fwd_f32(xd.float().cpu().numpy(), c_eff.numpy(), reverse=rev)
                np.testing.assert_allclose(y.float().cpu().numpy(), ref, rtol=2e-2, atol=2e-2)
    # a non-finite logarithm at the first element of a row has no effect
    x, c, dy = _data((4, 1000))
    l2 = torch.log(c)
    l2[:, 0] = float("inf")
    y = lb._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=l2.to(dev), reverse=False, logCoeffs=1)
    np.testing.assert_allclose(y.cpu().numpy(), oracle.fwd_f32(x.numpy(), c.numpy()), rtol=RTOL, atol=ATOL)
    lb.check_status()


def test_log_coefficients_not_offered_for_sequence_sharding():
    import ctypes
    from linrec_b200 import _capi
    dev = torch.device("cuda:0")
    x = torch.ones(2, 256, device=dev)
    rec = torch.zeros(2, 2, device=dev)
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device=dev)
    opts, keep = _capi.make_opts({"logCoeffs": 1})
    rc = _capi.lib.linrec_b200_fwd_carry(x.data_ptr(), x.data_ptr(), x.data_ptr(), rec.data_ptr(), 2, 256, 256, 0, 0, 0, 2,
                                         opts, ws.data_ptr(), ws.numel(), None)
    assert rc == _capi.ERR_NOT_IMPLEMENTED


try:
    from hypothesis import given, settings, strategies as st, HealthCheck
    _HAVE_HYPOTHESIS = True
except Exception:  # pragma: no cover
    _HAVE_HYPOTHESIS = False

if _HAVE_HYPOTHESIS:
    @settings(max_examples=60, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
    @given(rows=st.integers(1, 40), length=st.integers(1, 5000), pad=st.integers(0, 9), off=st.integers(0, 5),
           rev=st.booleans(), seed=st.integers(0, 1000))
    def test_fuzz_small_shapes(rows, length, pad, off, rev, seed):
        """Random small shapes, row strides and base offsets, both directions, forward and backward."""
        lb = _ops()
        dev = torch.device("cuda:0")
        g = torch.Generator(device="cpu").manual_seed(seed)
        stride = length + pad
        n = rows * stride + off
        bx, bc, bd = torch.randn(n, generator=g), 0.3 + 0.7 * torch.rand(n, generator=g), torch.randn(n, generator=g)
        view = lambda t: torch.as_strided(t, (rows, length), (stride, 1), off)
        xh, ch, dh = (view(t).contiguous() for t in (bx, bc, bd))
        xd, cd, dd = (view(t.to(dev)) for t in (bx, bc, bd))
        y = lb.linrec(xd, cd, reverse=rev)
        y_ref = oracle.fwd_f32(xh.numpy(), ch.numpy(), reverse=rev)
        np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=RTOL, atol=ATOL)
        yv = view(torch.zeros(n).to(dev))
        yv.copy_(torch.from_numpy(y_ref))
        dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dd, coeffs=cd, outputs=yv, reverse=rev)
        dx_ref, dc_ref = oracle.bwd_f32(dh.numpy(), ch.numpy(), y_ref, reverse=rev)
        np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(dc.cpu().numpy(), dc_ref, rtol=RTOL, atol=2 * ATOL)


@pytest.mark.parametrize("rev", [False, True])
def test_handful_of_very_long_rows(rev):
    """Few rows, many tiles each: the selector's one-ticket-at-a-time mode (every tile looks back at
    tiles that are in flight at the same moment)."""
    x, c, dy = _data((3, 40 * 8192 + 4096), clo=0.9)
    _check_fwd_bwd(x, c, dy, rev)                      # default: super-chunks (see test_super_chunks)
    _check_fwd_bwd(x, c, dy, rev, superChunks=0)       # the rows as they are: one ticket at a time
    _check_fwd_bwd(x, c, dy, rev, superChunks=0, kElemsPerThread=16, kThreadsPerBlock=128, kStages=1, lazyTickets=1)
    _check_fwd_bwd(x, c, dy, rev, superChunks=0, kElemsPerThread=16, kThreadsPerBlock=256, kStages=1, lazyTickets=0)
    # the same regime for rows that are not whole 128-byte lines (cp.async kernel)
    x, c, dy = _data((3, 40 * 8192 + 4100), clo=0.9)
    _check_fwd_bwd(x, c, dy, rev)
    _check_fwd_bwd(x, c, dy, rev, memcode=2, kThreadsPerBlock=128, kStages=2, lazyTickets=1)
    _check_fwd_bwd(x, c, dy, rev, memcode=2, kThreadsPerBlock=512, lazyTickets=0)
    x, c, dy = _data((150, 3 * 8192 + 8), clo=0.9)   # few rows: the 4096-element tile
    _check_fwd_bwd(x, c, dy, rev)


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("rev", [False, True])
def test_super_chunks_backward_with_fewer_rows_than_four_per_sm(rev, dtype):
    """Between 128 rows and four per SM only the backward operator cuts its rows (two launches); the
    forward operator scans them as they are (one launch).  (130, 2^17): four super-chunks per row."""
    lb = _ops()
    dev = torch.device("cuda:0")
    rows, L = 130, 1 << 17
    x, c, dy = _data((rows, L), clo=0.9, seed=SEED + 77)
    if dtype == "bf16":
        x, c, dy = x.bfloat16(), c.bfloat16(), dy.bfloat16()
    xf, cf, dyf = x.float().numpy(), c.float().numpy(), dy.float().numpy()
    rtol = RTOL if dtype == "f32" else 2.0 ** -7
    before = lb._C.launch_count()
    y = lb._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=rev)
    assert lb._C.launch_count() - before == 1
    y_ref = oracle.fwd_f32(xf, cf, reverse=rev)
    np.testing.assert_allclose(y.float().cpu().numpy(), y_ref, rtol=rtol, atol=ATOL)
    yd = torch.from_numpy(y_ref).to(dev).to(x.dtype)
    before = lb._C.launch_count()
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy.to(dev), coeffs=c.to(dev), outputs=yd, reverse=rev)
    assert lb._C.launch_count() - before == 2, "expected the super-chunk path (scan + fix-up)"
    dx_ref, dc_ref = oracle.bwd_f32(dyf, cf, yd.float().cpu().numpy(), reverse=rev)
    np.testing.assert_allclose(dx.float().cpu().numpy(), dx_ref, rtol=rtol, atol=ATOL)
    np.testing.assert_allclose(dc.float().cpu().numpy(), dc_ref, rtol=rtol, atol=2 * ATOL * max(1.0, float(np.abs(y_ref).max())))
    dx1, dc1 = lb._C.linrec_pipe_bwd(d_outputs=dy.to(dev), coeffs=c.to(dev), outputs=yd, reverse=rev, superChunks=0)
    np.testing.assert_allclose(dx.float().cpu().numpy(), dx1.float().cpu().numpy(), rtol=rtol, atol=ATOL)
    lb.check_status()


@pytest.mark.parametrize("rev", [False, True])
@pytest.mark.parametrize("rows,L,clo,chi", [(3, 1 << 18, 0.0, 1.0), (1, 1 << 20, 0.9, 1.0), (5, 3 << 17, 0.999, 1.0),
                                            (2, 1 << 18, 1.0, 1.0), (7, 1 << 17, 0.5, 1.5)],
                         ids=["fast_decay", "one_row", "slow_decay", "no_decay", "growing_stretches"])
def test_super_chunks(rows, L, clo, chi, rev):
    """Few very long rows are cut into super-chunks that are scanned independently and then corrected
    by a fix-up kernel (two launches).  Checked against the oracle for coefficients that decay fast,
    slowly (the correction crosses whole super-chunks), not at all (c = 1: a plain prefix sum, the
    fix-up is a full second pass) and for c in (0.5, 1.5), where stretches of |c| > 1 let a
    carry grow back; the result must also agree with the single-launch scan of the same rows."""
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data((rows, L), clo=clo, chi=chi, seed=SEED + rows)
    if clo == chi:
        c = torch.full_like(c, clo)
        x, dy = x * 1e-2, dy * 1e-2
    before = lb._C.launch_count()
    y = lb._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=rev)
    assert lb._C.launch_count() - before == 2, "expected the super-chunk path (scan + fix-up)"
    y1 = lb._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=rev, superChunks=0)
    y_ref = oracle.fwd_f32(x.numpy(), c.numpy(), reverse=rev)
    y64 = oracle.fwd_f64(x.numpy(), c.numpy(), reverse=rev)
    scale = max(1.0, float(np.abs(y64).max()))
    # judged like every slowly decaying case: against the fp64 evaluation, relative to the sequential
    # fp32 oracle's own error (two valid fp32 orders differ by more than the nominal tolerance there)
    err_seq = float(np.abs(y_ref - y64).max())
    for got in (y, y1):
        assert float(np.abs(got.cpu().numpy() - y64).max()) <= 2 * err_seq + ATOL * scale
    yd = torch.from_numpy(y_ref).to(dev)
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy.to(dev), coeffs=c.to(dev), outputs=yd, reverse=rev)
    dx1, dc1 = lb._C.linrec_pipe_bwd(d_outputs=dy.to(dev), coeffs=c.to(dev), outputs=yd, reverse=rev, superChunks=0)
    dx64, dc64 = oracle.bwd_f64(dy.numpy(), c.numpy(), y_ref.astype(np.float64), reverse=rev)
    dx32, dc32 = oracle.bwd_f32(dy.numpy(), c.numpy(), y_ref, reverse=rev)
    gscale = max(1.0, float(np.abs(dx64).max()))
    for gx, gc in ((dx, dc), (dx1, dc1)):
        assert float(np.abs(gx.cpu().numpy() - dx64).max()) <= 2 * float(np.abs(dx32 - dx64).max()) + ATOL * gscale
        assert float(np.abs(gc.cpu().numpy() - dc64).max()) <= 2 * float(np.abs(dc32 - dc64).max()) + 2 * ATOL * gscale * scale
    if chi <= 1.0 and clo < 1.0:
        np.testing.assert_allclose(y.cpu().numpy(), y1.cpu().numpy(), rtol=RTOL, atol=ATOL * scale)
    # explicit cut counts, bf16 storage
    for V in (2, 8):
        yv = lb._C.linrec_pipe_fwd(inputs=x.to(dev), coeffs=c.to(dev), reverse=rev, superChunks=V)
        assert float(np.abs(yv.cpu().numpy() - y64).max()) <= 2 * err_seq + ATOL * scale
    # 2-byte storage: the fix-up computes the head of every super-chunk again from its operands (it does
    # not add a correction to an already rounded value), so the element-wise tolerance holds
    before = lb._C.launch_count()
    xb, cb, dyb = x.bfloat16(), c.bfloat16(), dy.bfloat16()
    yb = lb._C.linrec_pipe_fwd(inputs=xb.to(dev), coeffs=cb.to(dev), reverse=rev)
    assert lb._C.launch_count() - before == 2
    if clo < 0.99 and chi <= 1.0:      # (growing stretches are too ill-conditioned for an element-wise 2^-7)
        yb_ref = oracle.fwd_f32(xb.float().numpy(), cb.float().numpy(), reverse=rev)
        np.testing.assert_allclose(yb.float().cpu().numpy(), yb_ref, rtol=2.0 ** -7, atol=ATOL)
        ybd = torch.from_numpy(yb_ref).bfloat16().to(dev)
        dxb, dcb = lb._C.linrec_pipe_bwd(d_outputs=dyb.to(dev), coeffs=cb.to(dev), outputs=ybd, reverse=rev)
        dxb_ref, dcb_ref = oracle.bwd_f32(dyb.float().numpy(), cb.float().numpy(), ybd.float().cpu().numpy(), reverse=rev)
        np.testing.assert_allclose(dxb.float().cpu().numpy(), dxb_ref, rtol=2.0 ** -7, atol=ATOL)
        np.testing.assert_allclose(dcb.float().cpu().numpy(), dcb_ref, rtol=2.0 ** -7, atol=2 * ATOL)
    lb.check_status()


def test_cuda_graph_capture_and_replay():
    """An operator is one kernel launch on a self-cleaning workspace, so a forward + backward step can
    be captured into a CUDA graph once and replayed on new data."""
    lb = _ops()
    dev = torch.device("cuda:0")
    shape = (64, 3 * 8192)
    x, c, dy = (t.to(dev) for t in _data(shape, clo=0.8))
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):          # warm-up on the capture stream: attributes, workspace
        for _ in range(2):
            y = lb._C.linrec_pipe_fwd(inputs=x, coeffs=c)
            lb._C.linrec_pipe_bwd(d_outputs=dy, coeffs=c, outputs=y)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        y = lb._C.linrec_pipe_fwd(inputs=x, coeffs=c)
        dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy, coeffs=c, outputs=y)
    for seed in (1, 2, 3):
        x2, c2, dy2 = _data(shape, clo=0.8, seed=seed)
        x.copy_(x2); c.copy_(c2); dy.copy_(dy2)
        graph.replay()
        torch.cuda.synchronize()
        y_ref = oracle.fwd_f32(x2.numpy(), c2.numpy())
        dx_ref, dc_ref = oracle.bwd_f32(dy2.numpy(), c2.numpy(), y.cpu().numpy())
        np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(dc.cpu().numpy(), dc_ref, rtol=RTOL, atol=4 * ATOL)
    lb.check_status()


def test_host_streamed_path():
    """Tensors in host memory, streamed through the device in row slabs (ragged last slab)."""
    from linrec_b200 import host
    for shape, slab in [((37, 1024), 8), ((5, 3 * 8192), 2), ((3, 7, 100), 4), ((9, 4096), None)]:
        x, c, dy = _data(shape, clo=0.5)
        pinned = [t.pin_memory() for t in (x, c, dy)]
        for rev in (False, True):
            y, dx, dc = host.linrec_fwd_bwd_host(*pinned, reverse=rev, slab_rows=slab)
            yf = host.linrec_fwd_host(pinned[0], pinned[1], reverse=rev, slab_rows=slab)
            torch.cuda.synchronize()
            y_ref = oracle.fwd_f32(x.numpy(), c.numpy(), reverse=rev)
            dx_ref, dc_ref = oracle.bwd_f32(dy.numpy(), c.numpy(), y.numpy(), reverse=rev)
            np.testing.assert_allclose(y.numpy(), y_ref, rtol=RTOL, atol=ATOL)
            np.testing.assert_allclose(yf.numpy(), y_ref, rtol=RTOL, atol=ATOL)
            np.testing.assert_allclose(dx.numpy(), dx_ref, rtol=RTOL, atol=ATOL)
            np.testing.assert_allclose(dc.numpy(), dc_ref, rtol=RTOL, atol=2 * ATOL)
    _ops().check_status()


# ---- the three operator families and their error behaviour ------------------------------------------
def test_tile_family_refuses_long_rows():
    lb = _ops()
    dev = torch.device("cuda:0")
    x = torch.zeros(2, 1 << 16, device=dev)
    with pytest.raises(RuntimeError):
        lb._C.linrec_tile_fwd(inputs=x, coeffs=x)
    y = lb._C.linrec_tile_fwd(inputs=x[:, :1024].contiguous(), coeffs=x[:, :1024].contiguous())
    assert y.shape == (2, 1024)


def test_unknown_option_is_not_implemented():
    lb = _ops()
    dev = torch.device("cuda:0")
    x = torch.zeros(2, 64, device=dev)
    with pytest.raises(NotImplementedError):
        lb._C.linrec_pipe_fwd(inputs=x, coeffs=x, kElemsPerThread=5)
    with pytest.raises(NotImplementedError):
        lb._C.linrec_pipe_fwd(inputs=x, coeffs=x, noSuchOption=1)


def test_precondition_errors():
    lb = _ops()
    dev = torch.device("cuda:0")
    a = torch.zeros(2, 64, device=dev)
    with pytest.raises(RuntimeError):
        lb._C.linrec_pipe_fwd(inputs=a, coeffs=torch.zeros(2, 32, device=dev))
    with pytest.raises(RuntimeError):
        lb._C.linrec_pipe_fwd(inputs=a, coeffs=a.double())
    with pytest.raises(RuntimeError):
        lb._C.linrec_pipe_fwd(inputs=a.t(), coeffs=a.t())
    with pytest.raises(RuntimeError):
        lb._C.linrec_pipe_fwd(inputs=a.cpu(), coeffs=a.cpu())


def test_empty_inputs():
    lb = _ops()
    dev = torch.device("cuda:0")
    for shape in [(0, 5), (3, 0)]:
        z = torch.zeros(shape, device=dev)
        assert lb.linrec(z, z).shape == shape


def test_attrs_and_configs():
    lb = _ops()
    names, configs = _variants()
    assert names[0] == "kElemsPerThread" and len(set(configs)) == len(configs)
    a = lb._C.linrec_pipe_attrs(True)
    assert a["numRegs"] > 0 and a["binaryVersion"] >= 100 and a["localSizeBytes"] == 0
    b = lb._C.linrec_pipe_attrs(False, **dict(zip(names, configs[0])))
    assert b["numRegs"] > 0 and b["residentBlocksPerSM"] >= 1


@pytest.mark.parametrize("bad", [float("inf"), float("nan")], ids=["inf", "nan"])
@pytest.mark.parametrize("L", [8192 + 32, 3 * 8192 + 64, 2 * 2048 + 64, 5000, 5001, 512, 100], ids=lambda v: f"L{v}")
@pytest.mark.parametrize("rev", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_nonfinite_first_coefficient_is_ignored(dtype, rev, L, bad):
    """c at the scan start has no effect, even when it is not finite (linrec_ref.cuh:63): the first
    output is x itself.  Lengths cover the bulk-copy kernel with a ragged last piece (the scan start
    of a reversed scan then lies inside the tile, not at its end), the 16-byte cp.async kernel
    (5000), the plain-load kernel (5001) and rows that share a tile (512, 100)."""
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data((3, L), clo=0.5)
    x, c, dy = x.to(dtype), c.to(dtype), dy.to(dtype)
    first = L - 1 if rev else 0
    c[:, first] = bad
    rtol = RTOL if dtype == torch.float32 else 2.0 ** -7
    y = lb.linrec(x.to(dev), c.to(dev), reverse=rev)
    c2 = c.clone()
    c2[:, first] = 0.0
    y_ref = oracle.fwd_f32(x.float().numpy(), c2.float().numpy(), reverse=rev)
    np.testing.assert_allclose(y.float().cpu().numpy(), y_ref, rtol=rtol, atol=ATOL)
    # the backward pass never reads that coefficient either (its shifted coefficients start one later)
    yd = torch.from_numpy(y_ref).to(dtype).to(dev)
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy.to(dev), coeffs=c.to(dev), outputs=yd, reverse=rev)
    dx_ref, dc_ref = oracle.bwd_f32(dy.float().numpy(), c2.float().numpy(), yd.float().cpu().numpy(), reverse=rev)
    np.testing.assert_allclose(dx.float().cpu().numpy(), dx_ref, rtol=rtol, atol=ATOL)
    np.testing.assert_allclose(dc.float().cpu().numpy(), dc_ref, rtol=rtol, atol=2 * ATOL)
    lb.check_status()


@pytest.mark.parametrize("L", [3 * 8192 + 64, 5000, 5001], ids=lambda v: f"L{v}")
@pytest.mark.parametrize("rev", [False, True])
def test_nonfinite_first_coefficient_on_the_shard_that_holds_the_scan_start(rev, L):
    """The carry-emitting forward of sequence sharding: on the shard that holds the scan start the
    first coefficient is ignored as in the unsharded operator (the other shards use theirs)."""
    from linrec_b200.sharded import CudaShardKernels
    dev = torch.device("cuda:0")
    x, c, _ = _data((4, L), clo=0.5)
    first = L - 1 if rev else 0
    c[:, first] = float("inf")
    nshards = 3
    shard = nshards - 1 if rev else 0
    y, rec = CudaShardKernels().fwd_carry(x.to(dev), c.to(dev), rev, shard, nshards)
    c2 = c.clone()
    c2[:, first] = 0.0
    y_ref = oracle.fwd_f32(x.numpy(), c2.numpy(), reverse=rev)
    np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=RTOL, atol=ATOL)
    last = 0 if rev else L - 1
    np.testing.assert_allclose(rec[:, 1].cpu().numpy(), y_ref[:, last], rtol=RTOL, atol=ATOL)
    assert float(rec[:, 0].abs().max()) == 0.0     # the product over the shard contains the ignored factor as 0
    _ops().check_status()


def test_call_from_a_fresh_host_thread():
    """The first call a host thread makes finds the caches warm and makes no CUDA runtime call that
    would bind a device context before the tensor maps are encoded (autograd workers are such
    threads); the library has to bind it."""
    import threading
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data((64, 4096))
    xd, cd, dyd = x.to(dev), c.to(dev), dy.to(dev)
    y0 = lb._C.linrec_pipe_fwd(inputs=xd, coeffs=cd, reverse=False)      # warms every cache
    dx0, dc0 = lb._C.linrec_pipe_bwd(d_outputs=dyd, coeffs=cd, outputs=y0, reverse=False)
    torch.cuda.synchronize()
    out = {}

    def work():
        try:
            y = lb._C.linrec_pipe_fwd(inputs=xd, coeffs=cd, reverse=False)
            dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dyd, coeffs=cd, outputs=y0, reverse=False)
            torch.cuda.synchronize()
            out["ok"] = torch.equal(y, y0) and torch.equal(dx, dx0) and torch.equal(dc, dc0)
        except Exception as exc:   # reported in the main thread
            out["exc"] = exc

    t = threading.Thread(target=work)
    t.start()
    t.join()
    assert "exc" not in out, out.get("exc")
    assert out["ok"]


# ---- rows of any alignment: one CTA per row ------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["f32", "bf16", "f16"])
@pytest.mark.parametrize("rev", [False, True])
@pytest.mark.parametrize("shape,skew", [((700, 1001), 0), ((600, 10001), 0), ((1000, 77), 0), ((650, 2049), 0),
                                        ((640, 4099), 1), ((5, 1001), 0), ((3, 20003), 3), ((2, 7), 1)],
                         ids=lambda v: str(v).replace(" ", ""))
def test_row_kernel_any_alignment(shape, skew, rev, dtype):
    """`memcode` 4: one CTA walks one row with aligned 16-byte accesses, whatever the row's length and
    wherever it starts (here also rows that start `skew` elements into a wider tensor, so that for
    2-byte storage not even 4-byte alignment holds).  Forward and backward against the oracle, the
    columns around the rows untouched, one launch; with several rows per SM it is chosen by itself."""
    lb = _ops()
    dev = torch.device("cuda:0")
    rows, L = shape
    x, c, dy = _data(shape, clo=0.5, seed=SEED + L)
    tt = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[dtype]
    rtol = {"f32": RTOL, "bf16": 2.0 ** -7, "f16": 2.0 ** -9}[dtype]
    FILL = 123.0

    def embed(t):
        """The rows inside a wider tensor of guard columns."""
        full = torch.full((rows, L + skew + 5), FILL, dtype=tt, device=dev)
        full[:, skew:skew + L] = t.to(tt).to(dev)
        return full, full[:, skew:skew + L]

    (xf, xv), (cf, cv), (dyf, dyv) = embed(x), embed(c), embed(dy)
    xr, cr, dyr = (t.float().cpu().numpy() for t in (xv, cv, dyv))
    opts = {} if rows >= 600 else {"memcode": 4}
    before = lb._C.launch_count()
    y = lb._C.linrec_pipe_fwd(inputs=xv, coeffs=cv, reverse=rev, **opts)
    assert lb._C.launch_count() - before == 1
    y_ref = oracle.fwd_f32(xr, cr, reverse=rev)
    np.testing.assert_allclose(y.float().cpu().numpy(), y_ref, rtol=rtol, atol=ATOL)
    assert y.stride() == xv.stride()     # results keep the layout of the inputs
    yfull, yv = embed(torch.from_numpy(y_ref))
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dyv, coeffs=cv, outputs=yv, reverse=rev, **opts)
    dx_ref, dc_ref = oracle.bwd_f32(dyr, cr, yv.float().cpu().numpy(), reverse=rev)
    np.testing.assert_allclose(dx.float().cpu().numpy(), dx_ref, rtol=rtol, atol=ATOL)
    np.testing.assert_allclose(dc.float().cpu().numpy(), dc_ref, rtol=rtol, atol=2 * ATOL * max(1.0, float(np.abs(y_ref).max())))
    for full in (xf, cf, dyf, yfull):
        guard = torch.cat([full[:, :skew], full[:, skew + L:]], dim=1)
        assert bool((guard == FILL).all()), "guard columns changed"
    if rows >= 600:
        # the loaders these rows used to take still give the same answer when pinned
        y0 = lb._C.linrec_pipe_fwd(inputs=xv, coeffs=cv, reverse=rev, memcode=0)
        np.testing.assert_allclose(y0.float().cpu().numpy(), y_ref, rtol=rtol, atol=ATOL)
    lb.check_status()


def test_row_kernel_first_coefficient_and_nonfinite_values():
    """The coefficient of a row's first element in scan order is never used (linrec_ref.cuh:63), also
    when it is inf or nan; a non-finite input travels along its own row and does not leak into the
    neighbouring rows that share its 16-byte chunks."""
    lb = _ops()
    dev = torch.device("cuda:0")
    rows, L = 700, 1001
    x, c, _ = _data((rows, L), clo=0.5)
    for rev in (False, True):
        cc = c.clone()
        cc[:, -1 if rev else 0] = float("inf")
        cc[3, -1 if rev else 0] = float("nan")
        xx = x.clone()
        xx[10, L - 1] = float("inf")      # last element of row 10: shares a chunk with row 11's first
        y = lb._C.linrec_pipe_fwd(inputs=xx.to(dev), coeffs=cc.to(dev), reverse=rev).cpu().numpy()
        c0 = cc.clone()
        c0[:, -1 if rev else 0] = 0.0
        y_ref = oracle.fwd_f32(xx.numpy(), c0.numpy(), reverse=rev)
        ok = np.isfinite(y_ref)
        np.testing.assert_array_equal(np.isfinite(y), ok)
        assert ok[9].all() and ok[11].all()
        np.testing.assert_allclose(y[ok], y_ref[ok], rtol=RTOL, atol=ATOL)
    lb.check_status()


# ---- double precision: the sequential family ----------------------------------------------------------
@pytest.mark.parametrize("shape", [(1, 1), (5, 17), (64, 512), (3, 20000)], ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
def test_float64_sequential_operator(shape, rev):
    """fp64 storage and arithmetic through `linrec_ref` (the dtype dispatch the reference leaves as a
    TODO, linrec_pipe.cu:22), against the fp64 oracle at rtol 1e-10."""
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data(shape, clo=0.9)
    y = lb._C.linrec_ref_fwd(inputs=x.double().to(dev), coeffs=c.double().to(dev), reverse=rev)
    assert y.dtype == torch.float64
    y_ref = oracle.fwd_f64(x.numpy(), c.numpy(), reverse=rev)
    np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=1e-10, atol=1e-12)
    dx, dc = lb._C.linrec_ref_bwd(d_outputs=dy.double().to(dev), coeffs=c.double().to(dev), outputs=y, reverse=rev)
    dx_ref, dc_ref = oracle.bwd_f64(dy.numpy(), c.numpy(), y.cpu().numpy(), reverse=rev)
    np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(dc.cpu().numpy(), dc_ref, rtol=1e-10, atol=1e-12)
    # autograd through the sequential family
    xd = x.double().to(dev).requires_grad_(True)
    cd = c.double().to(dev).requires_grad_(True)
    gx, gc = torch.autograd.grad(lb.linrec_ref(xd, cd, reverse=rev), (xd, cd), dy.double().to(dev))
    np.testing.assert_allclose(gx.cpu().numpy(), dx_ref, rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(gc.cpu().numpy(), dc_ref, rtol=1e-10, atol=1e-12)


@pytest.mark.parametrize("shape", [(1, 1), (5, 17), (64, 1024), (3, 20000), (300, 5001), (2, 1025), (700, 4096)],
                         ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
def test_float64_tiled_families(shape, rev):
    """fp64 through `linrec_pipe` / `linrec_tile` / `linrec` (one CTA per row, the carry kept by the CTA),
    forward, backward and autograd, against the fp64 oracle at rtol 1e-10; padded rows; coefficients
    given as logarithms; a pinned variant is refused (there are none to pin for this type)."""
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data(shape, clo=0.9)
    xd, cd, dyd = x.double().to(dev), c.double().to(dev), dy.double().to(dev)
    y_ref = oracle.fwd_f64(x.numpy(), c.numpy(), reverse=rev)
    for op in (lb._C.linrec_pipe_fwd, lb._C.linrec_tile_fwd):
        y = op(inputs=xd, coeffs=cd, reverse=rev)
        assert y.dtype == torch.float64
        np.testing.assert_allclose(y.cpu().numpy(), y_ref, rtol=1e-10, atol=1e-12)
    dx_ref, dc_ref = oracle.bwd_f64(dy.numpy(), c.numpy(), y_ref, reverse=rev)
    yd = torch.from_numpy(y_ref).to(dev)
    for op in (lb._C.linrec_pipe_bwd, lb._C.linrec_tile_bwd):
        dx, dc = op(d_outputs=dyd, coeffs=cd, outputs=yd, reverse=rev)
        np.testing.assert_allclose(dx.cpu().numpy(), dx_ref, rtol=1e-10, atol=1e-12)
        np.testing.assert_allclose(dc.cpu().numpy(), dc_ref, rtol=1e-10, atol=1e-12)
    xg, cg = xd.clone().requires_grad_(True), cd.clone().requires_grad_(True)
    gx, gc = torch.autograd.grad(lb.linrec(xg, cg, reverse=rev), (xg, cg), dyd)
    np.testing.assert_allclose(gx.cpu().numpy(), dx_ref, rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(gc.cpu().numpy(), dc_ref, rtol=1e-10, atol=1e-12)
    # rows with a stride larger than their length, guard columns untouched
    rows, L = shape
    pad = 3
    def padded(t, fill):
        full = torch.full((rows, L + pad), fill, dtype=torch.float64, device=dev)
        full[:, :L] = t
        return full[:, :L]
    yp = lb._C.linrec_pipe_fwd(inputs=padded(xd, 7.0), coeffs=padded(cd, 7.0), reverse=rev)
    np.testing.assert_allclose(yp.cpu().numpy(), y_ref, rtol=1e-10, atol=1e-12)
    # logarithmic coefficients: exp inside the kernel
    from linrec_b200.general import linrec_general
    yl = linrec_general(xd, cd.log(), logc=True, reverse=rev)
    np.testing.assert_allclose(yl.cpu().numpy(), y_ref, rtol=1e-9, atol=1e-11)
    with pytest.raises(NotImplementedError):
        lb._C.linrec_pipe_fwd(inputs=xd, coeffs=cd, reverse=rev, kThreadsPerBlock=256)
    lb.check_status()


# ---- bounded waits -----------------------------------------------------------------------------------
def test_lookback_wait_gives_up_with_status():
    """Tickets are started past the first piece of every row, so the pieces that run wait for a
    predecessor that never publishes.  The wait must end by itself and leave a status code; the
    context must stay usable."""
    lb = _ops()
    dev = torch.device("cuda:0")
    x = torch.ones(2, 4096 * 4, device=dev)
    lb._C.linrec_pipe_fwd(inputs=x, coeffs=x, firstTicket=2, waitBudgetMs=20)
    with pytest.raises(RuntimeError, match="wait gave up"):
        lb.check_status()
    # the next call resets the status word and works
    y = lb.linrec(x, x * 0.5)
    lb.check_status()
    assert torch.isfinite(y).all()


# ---- against the reference's own CUDA kernels, where the checker library was built -------------------
def _refcuda():
    import ctypes
    import os
    path = os.path.join(os.path.dirname(oracle.__file__), "_ref", "liblinrec_refcuda.so")
    if not os.path.exists(path):
        pytest.skip("reference CUDA checker not built on this machine")
    L = ctypes.CDLL(path)
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    L.refcuda_fwd_f32.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    L.refcuda_bwd_f32.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, vp]
    return L


@pytest.mark.parametrize("shape", [(64, 512), (16, 65536)], ids=lambda s: f"{s[0]}x{s[1]}")
@pytest.mark.parametrize("rev", [False, True])
def test_against_reference_cuda_kernels(shape, rev):
    R = _refcuda()
    lb = _ops()
    dev = torch.device("cuda:0")
    x, c, dy = _data(shape, clo=0.9, chi=1.0)
    xd, cd, dyd = x.to(dev), c.to(dev), dy.to(dev)
    stream = torch.cuda.current_stream().cuda_stream
    y_ref = torch.empty_like(xd)
    assert R.refcuda_fwd_f32(xd.data_ptr(), cd.data_ptr(), y_ref.data_ptr(), shape[0], shape[1], int(rev), stream) == 0
    y = lb.linrec(xd, cd, reverse=rev)
    torch.testing.assert_close(y, y_ref, rtol=RTOL, atol=ATOL)
    dx_ref, dc_ref = torch.empty_like(xd), torch.empty_like(xd)
    assert R.refcuda_bwd_f32(dyd.data_ptr(), cd.data_ptr(), y_ref.data_ptr(), dx_ref.data_ptr(), dc_ref.data_ptr(),
                             shape[0], shape[1], int(rev), stream) == 0
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dyd, coeffs=cd, outputs=y_ref, reverse=rev)
    torch.testing.assert_close(dx, dx_ref, rtol=RTOL, atol=ATOL)
    if rev:
        # the reference's reverse backward lets two blocks race on column 0 of rows >= 1
        torch.testing.assert_close(dc[:, 1:], dc_ref[:, 1:], rtol=RTOL, atol=2 * ATOL)
        torch.testing.assert_close(dc[0], dc_ref[0], rtol=RTOL, atol=2 * ATOL)
    else:
        torch.testing.assert_close(dc, dc_ref, rtol=RTOL, atol=2 * ATOL)
    # our own sequential operator against the reference's, same algorithm: tight agreement
    y_seq = lb._C.linrec_ref_fwd(inputs=xd, coeffs=cd, reverse=rev)
    torch.testing.assert_close(y_seq, y_ref, rtol=1e-6, atol=1e-6)
