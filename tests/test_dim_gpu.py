"""Scan along a dimension other than the last (GPU only; every call goes through the C ABI:
linrec_b200_fwd_dim / linrec_b200_bwd_dim).  The checker is the CPU oracle run on the transposed
tensors, i.e. the definition of the reference's `dim` argument (linrec/impl/python/ops.py:8-14).

Tolerances as for the last-dimension operators: fp32 rtol 1e-4 / atol 1e-5 (2e-5 for dc);
2-byte storage rtol 2^-7 / atol 1e-5 against fp32 on the rounded inputs.
"""
import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5
SEED = 12334567890


def _lb():
    import linrec_b200
    import linrec_b200.ops as ops
    from linrec_b200.general import linrec_general
    return linrec_b200, ops, linrec_general


def _data(shape, clo=0.5, chi=1.0, seed=SEED):
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(shape, generator=g)
    c = clo + (chi - clo) * torch.rand(shape, generator=g)
    dy = torch.randn(shape, generator=g)
    return x, c, dy


def _oracle_dim(x, c, dy, dim, rev):
    """Oracle along `dim`: move the axis last, scan rows, move it back."""
    last = x.dim() - 1
    xt, ct, dyt = (t.transpose(dim, last).contiguous().numpy() for t in (x, c, dy))
    y = oracle.fwd_f32(xt, ct, reverse=rev)
    dx, dc = oracle.bwd_f32(dyt, ct, y, reverse=rev)
    back = lambda a: torch.from_numpy(a).transpose(dim, last).contiguous()
    return back(y), back(dx), back(dc)


def _check(shape, dim, rev, dtype=torch.float32, rtol=RTOL, atol=ATOL, **kw):
    lb, ops, _ = _lb()
    dev = torch.device("cuda:0")
    x, c, dy = _data(shape)
    if dtype != torch.float32:
        x, c, dy = (t.to(dtype).float() for t in (x, c, dy))
    y_ref, dx_ref, dc_ref = _oracle_dim(x, c, dy, dim, rev)
    xd, cd, dyd = (t.to(dev, dtype) for t in (x, c, dy))
    y = ops.linrec_dim_fwd(xd, cd, dim, rev, **kw)
    np.testing.assert_allclose(y.float().cpu().numpy(), y_ref.numpy(), rtol=rtol, atol=atol)
    yd = y_ref.to(dev, dtype)
    if dtype != torch.float32:
        # backward from the rounded forward outputs, as autograd would hand them over
        _, dx_ref, dc_ref = _oracle_bwd_from(yd.float().cpu(), c, dy, dim, rev)
    dx, dc = ops.linrec_dim_bwd(dyd, cd, yd, dim, rev, **kw)
    np.testing.assert_allclose(dx.float().cpu().numpy(), dx_ref.numpy(), rtol=rtol, atol=atol)
    np.testing.assert_allclose(dc.float().cpu().numpy(), dc_ref.numpy(), rtol=rtol, atol=2 * atol)
    lb.check_status()


def _oracle_bwd_from(y, c, dy, dim, rev):
    last = y.dim() - 1
    yt, ct, dyt = (t.transpose(dim, last).contiguous().numpy() for t in (y, c, dy))
    dx, dc = oracle.bwd_f32(dyt, ct, yt, reverse=rev)
    back = lambda a: torch.from_numpy(a).transpose(dim, last).contiguous()
    return None, back(dx), back(dc)


SHAPES = [(3, 100, 36), (2, 1000, 4), (1, 5000, 128), (5, 33, 260), (2, 4099, 512), (4, 300, 1024), (1, 1, 8), (7, 2, 4)]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("rev", [False, True])
def test_middle_axis_fp32(shape, rev):
    for kw in ({}, {"kChunksPerJob": 0}, {"kChunksPerJob": 1}, {"kChunksPerJob": 3}):
        _check(shape, 1, rev, **kw)


@pytest.mark.parametrize("variant", [(128, 32, 3), (128, 32, 2), (128, 32, 4), (64, 64, 3), (64, 64, 2), (32, 64, 3),
                                     (32, 64, 2), (32, 128, 2), (256, 32, 2)], ids=lambda v: "x".join(map(str, v)))
def test_every_compiled_variant(variant):
    nt, lc, s = variant
    for shape in [(3, 700, 264), (40, 129, 132)]:
        for rev in (False, True):
            for k in (1, 2, 0):
                _check(shape, 1, rev, kThreadsPerBlock=nt, kRowsPerChunk=lc, kStages=s, kChunksPerJob=k)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16], ids=["bf16", "f16"])
@pytest.mark.parametrize("shape", [(3, 100, 40), (2, 1000, 8), (1, 3000, 256), (3, 515, 1032)], ids=lambda s: "x".join(map(str, s)))
def test_middle_axis_two_byte(dtype, shape):
    for rev in (False, True):
        for kw in ({}, {"kChunksPerJob": 1}, {"kChunksPerJob": 0}):
            _check(shape, 1, rev, dtype=dtype, rtol=2 ** -7 if dtype == torch.bfloat16 else 2 ** -9,
                   atol=1e-5 if dtype == torch.bfloat16 else 1e-4, **kw)


def test_256_wide_variant_is_fp32_only():
    lb, ops, _ = _lb()
    dev = torch.device("cuda:0")
    x = torch.ones(2, 64, 512, device=dev, dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        ops.linrec_dim_fwd(x, x, 1, False, kThreadsPerBlock=256, kRowsPerChunk=32, kStages=2)


def test_many_columns_and_long_sequences():
    """Enough columns for jobs of several chunks that wait on their predecessor, and few columns with
    long sequences (decoupled look-back over many chunks)."""
    _check((600, 2100, 128), 1, False)
    _check((600, 2100, 128), 1, True)
    _check((2, 70000, 64), 1, False)
    _check((1, 50001, 256), 1, True)


def test_general_signature_uses_the_axis_kernel_and_matches_the_transposed_path():
    lb, ops, linrec_general = _lb()
    dev = torch.device("cuda:0")
    for shape, dim in [((64, 200, 64), 1), ((8, 16, 150, 32), 2), ((130, 90, 4, 8), 1), ((300, 4096), 0)]:
        x, c, dy = _data(shape)
        for rev in (False, True):
            xd = x.to(dev).requires_grad_(True)
            cd = c.to(dev).requires_grad_(True)
            n0 = lb._C.launch_count()
            y = linrec_general(xd, cd, dim=dim, reverse=rev)
            gx, gc = torch.autograd.grad(y, (xd, cd), dy.to(dev))
            assert lb._C.launch_count() - n0 == 2        # one kernel forward, one backward, no copies of ours
            y_ref, dx_ref, dc_ref = _oracle_dim(x, c, dy, dim, rev)
            np.testing.assert_allclose(y.detach().cpu().numpy(), y_ref.numpy(), rtol=RTOL, atol=ATOL)
            np.testing.assert_allclose(gx.cpu().numpy(), dx_ref.numpy(), rtol=RTOL, atol=ATOL)
            np.testing.assert_allclose(gc.cpu().numpy(), dc_ref.numpy(), rtol=RTOL, atol=2 * ATOL)
    lb.check_status()


def test_general_signature_takes_the_transposed_path_for_a_handful_of_columns():
    lb, ops, linrec_general = _lb()
    dev = torch.device("cuda:0")
    x, c, dy = _data((2, 300, 64))
    assert ops.dim_eligible(x.to(dev), 1) and not ops.dim_worthwhile(x.to(dev), 1)
    y = linrec_general(x.to(dev), c.to(dev), dim=1, reverse=True)
    y_ref, _, _ = _oracle_dim(x, c, dy, 1, True)
    np.testing.assert_allclose(y.cpu().numpy(), y_ref.numpy(), rtol=RTOL, atol=ATOL)


def test_general_signature_falls_back_for_unaligned_channels():
    lb, ops, linrec_general = _lb()
    dev = torch.device("cuda:0")
    x, c, dy = _data((3, 50, 7))          # 7 channels of 4 bytes: not whole 16-byte chunks
    assert not ops.dim_eligible(x.to(dev), 1)
    y = linrec_general(x.to(dev), c.to(dev), dim=1)
    y_ref, _, _ = _oracle_dim(x, c, dy, 1, False)
    np.testing.assert_allclose(y.cpu().numpy(), y_ref.numpy(), rtol=RTOL, atol=ATOL)
    with pytest.raises(RuntimeError):
        ops.linrec_dim_fwd(x.to(dev), c.to(dev), 1, False)


def test_first_coefficient_is_ignored():
    """A non-finite coefficient at the first element of a sequence has no effect, as in the
    reference kernels that start with y[s] = x[s] (linrec/impl/cuda/linrec_ref.cuh:63)."""
    lb, ops, _ = _lb()
    dev = torch.device("cuda:0")
    x, c, dy = _data((2, 77, 16))
    for rev in (False, True):
        c2 = c.clone()
        c2[:, -1 if rev else 0, :] = float("inf")
        y = ops.linrec_dim_fwd(x.to(dev), c2.to(dev), 1, rev)
        y_ref, _, _ = _oracle_dim(x, c, dy, 1, rev)
        np.testing.assert_allclose(y.cpu().numpy(), y_ref.numpy(), rtol=RTOL, atol=ATOL)


def test_guard_bands_untouched():
    """Outputs written through the C ABI into the middle of sentinel-filled allocations."""
    import ctypes
    from linrec_b200 import _capi
    lb, ops, _ = _lb()
    dev = torch.device("cuda:0")
    for (nb, L, D) in [(3, 45, 12), (2, 130, 260), (1, 33, 516)]:
        for bwd in (False, True):
            x, c, dy = _data((nb, L, D))
            n, pad = nb * L * D, 1024
            outs = [torch.full((n + 2 * pad,), -777.0, device=dev) for _ in range(2)]
            xd, cd, yd = x.to(dev), c.to(dev), dy.to(dev)
            need = _capi.lib.linrec_b200_dim_workspace_size(int(bwd), nb, L, D, 0, None)
            ws = torch.zeros(need, dtype=torch.uint8, device=dev)
            st = torch.cuda.current_stream().cuda_stream
            o0 = outs[0].data_ptr() + pad * 4
            o1 = outs[1].data_ptr() + pad * 4
            if not bwd:
                rc = _capi.lib.linrec_b200_fwd_dim(xd.data_ptr(), cd.data_ptr(), o0, nb, L, D, 0, 0, None, ws.data_ptr(), need, st)
            else:
                rc = _capi.lib.linrec_b200_bwd_dim(xd.data_ptr(), cd.data_ptr(), yd.data_ptr(), o0, o1, nb, L, D, 0, 0, None,
                                                   ws.data_ptr(), need, st)
            assert rc == 0
            torch.cuda.synchronize()
            for o in outs[: 2 if bwd else 1]:
                assert (o[:pad] == -777.0).all() and (o[pad + n:] == -777.0).all()
                assert (o[pad:pad + n] != -777.0).all()


def test_lookback_wait_gives_up_with_status():
    """Tickets are started past the first job of every column, so the jobs that run wait for a
    predecessor that never publishes.  The wait ends by itself and leaves a status code; the context
    stays usable."""
    lb, ops, _ = _lb()
    dev = torch.device("cuda:0")
    x = torch.ones(1, 4096, 128, device=dev)
    ops.linrec_dim_fwd(x, x, 1, False, kChunksPerJob=1, firstTicket=3, waitBudgetMs=20)
    with pytest.raises(RuntimeError, match="wait gave up"):
        lb.check_status()
    y = ops.linrec_dim_fwd(x, x * 0.5, 1, False)
    lb.check_status()
    assert torch.isfinite(y).all()


try:
    from hypothesis import given, settings, strategies as st, HealthCheck
    _HAVE_HYPOTHESIS = True
except Exception:  # pragma: no cover
    _HAVE_HYPOTHESIS = False

if _HAVE_HYPOTHESIS:
    @settings(max_examples=50, deadline=None, suppress_health_check=list(HealthCheck), derandomize=True)
    @given(nb=st.integers(1, 6), length=st.integers(1, 700), chan4=st.integers(1, 150), rev=st.booleans(),
           k=st.sampled_from([None, 0, 1, 2, 5]), seed=st.integers(0, 1000))
    def test_fuzz_small_shapes(nb, length, chan4, rev, k, seed):
        """Random small (batch, sequence, channel) shapes, both directions, forward and backward, every
        way of cutting a column into jobs."""
        lb, ops, _ = _lb()
        dev = torch.device("cuda:0")
        shape = (nb, length, 4 * chan4)
        x, c, dy = _data(shape, clo=0.3, seed=seed)
        kw = {} if k is None else {"kChunksPerJob": k}
        y_ref, dx_ref, dc_ref = _oracle_dim(x, c, dy, 1, rev)
        y = ops.linrec_dim_fwd(x.to(dev), c.to(dev), 1, rev, **kw)
        np.testing.assert_allclose(y.cpu().numpy(), y_ref.numpy(), rtol=RTOL, atol=ATOL)
        dx, dc = ops.linrec_dim_bwd(dy.to(dev), c.to(dev), y_ref.to(dev), 1, rev, **kw)
        np.testing.assert_allclose(dx.cpu().numpy(), dx_ref.numpy(), rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(dc.cpu().numpy(), dc_ref.numpy(), rtol=RTOL, atol=2 * ATOL)
        lb.check_status()


def test_cuda_graph_capture_and_replay():
    """Like the last-axis operators, a middle-axis operator is one kernel launch on a self-cleaning
    workspace: a forward + backward step is captured once and replayed on new data."""
    lb, ops, _ = _lb()
    dev = torch.device("cuda:0")
    shape = (6, 900, 256)
    x, c, dy = (t.to(dev) for t in _data(shape, clo=0.8))
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):          # warm-up on the capture stream: attributes, workspace
        for _ in range(2):
            y = ops.linrec_dim_fwd(x, c, 1, False)
            ops.linrec_dim_bwd(dy, c, y, 1, False)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        y = ops.linrec_dim_fwd(x, c, 1, False)
        dx, dc = ops.linrec_dim_bwd(dy, c, y, 1, False)
    for seed in (1, 2, 3):
        x2, c2, dy2 = _data(shape, clo=0.8, seed=seed)
        x.copy_(x2); c.copy_(c2); dy.copy_(dy2)
        graph.replay()
        torch.cuda.synchronize()
        y_ref, dx_ref, dc_ref = _oracle_dim(x2, c2, dy2, 1, False)
        np.testing.assert_allclose(y.cpu().numpy(), y_ref.numpy(), rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(dx.cpu().numpy(), dx_ref.numpy(), rtol=RTOL, atol=4 * ATOL)
        np.testing.assert_allclose(dc.cpu().numpy(), dc_ref.numpy(), rtol=RTOL, atol=4 * ATOL)
    lb.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_full_size_against_the_last_axis_kernels(dtype):
    """The autograd configuration's 2^28 elements laid out (16, 8192, 2048): the scan along the
    middle axis must agree with the last-axis kernels run on transposed copies (two independent
    kernels, tile algebra against a sequential walk), forward and backward, and with linearity:
    scan(a*x) = a*scan(x)."""
    lb, ops, _ = _lb()
    dev = torch.device("cuda:0")
    shape = (16, 8192, 2048)
    g = torch.Generator(device=dev).manual_seed(SEED)
    x = torch.randn(shape, device=dev, generator=g).to(dtype)
    c = (0.9 + 0.1 * torch.rand(shape, device=dev, generator=g)).to(dtype)
    dy = torch.randn(shape, device=dev, generator=g).to(dtype)
    rtol, atol = (RTOL, 1e-4) if dtype == torch.float32 else (2 ** -6, 2e-2)

    def close(a, b, what):
        a, b = a.float(), b.float()
        bad = ((a - b).abs() > atol + rtol * b.abs()).sum().item()
        assert bad <= a.numel() * 1e-6, f"{what}: {bad} of {a.numel()} outside tolerance"

    for rev in (False, True):
        y = ops.linrec_dim_fwd(x, c, 1, rev)
        xt, ct = x.transpose(1, 2).contiguous(), c.transpose(1, 2).contiguous()
        yt = lb._C.linrec_pipe_fwd(inputs=xt, coeffs=ct, reverse=rev)
        close(y, yt.transpose(1, 2), "forward")
        del xt
        dx, dc = ops.linrec_dim_bwd(dy, c, y, 1, rev)
        dyt, y_t = dy.transpose(1, 2).contiguous(), y.transpose(1, 2).contiguous()
        dxt, dct = lb._C.linrec_pipe_bwd(d_outputs=dyt, coeffs=ct, outputs=y_t, reverse=rev)
        close(dx, dxt.transpose(1, 2), "d_inputs")
        close(dc, dct.transpose(1, 2), "d_coeffs")
        del dyt, y_t, dxt, dct, ct, yt, dx, dc
        if dtype == torch.float32:
            y2 = ops.linrec_dim_fwd(x * 2.0, c, 1, rev)
            assert torch.equal(y2, y * 2.0)       # scaling by a power of two is exact
            del y2
        del y
    lb.check_status()


@pytest.mark.parametrize("shape", [(3, 100, 36), (2, 1000, 4), (5, 33, 260), (2, 4099, 512), (300, 130, 128)],
                         ids=lambda s: "x".join(map(str, s)))
def test_log_coefficients_fused(shape):
    """Option logCoeffs along the middle axis: exp while loading, d_c * c out of the backward kernel
    (the element's own coefficient comes from the neighbouring row of the shifted box, or from global
    memory at the chunk edge)."""
    lb, ops, linrec_general = _lb()
    dev = torch.device("cuda:0")
    x, c, dy = _data(shape, clo=0.3)
    logc = torch.log(c)
    c_eff = torch.exp(logc)
    for rev in (False, True):
        y_ref, dx_ref, dc_ref = _oracle_dim(x, c_eff, dy, 1, rev)
        dl_ref = dc_ref * c_eff
        for kw in ({}, {"kChunksPerJob": 1}, {"kChunksPerJob": 0}, {"kThreadsPerBlock": 128}):
            y = ops.linrec_dim_fwd(x.to(dev), logc.to(dev), 1, rev, logCoeffs=1, **kw)
            np.testing.assert_allclose(y.cpu().numpy(), y_ref.numpy(), rtol=RTOL, atol=ATOL)
            dx, dl = ops.linrec_dim_bwd(dy.to(dev), logc.to(dev), y_ref.to(dev), 1, rev, logCoeffs=1, **kw)
            np.testing.assert_allclose(dx.cpu().numpy(), dx_ref.numpy(), rtol=RTOL, atol=ATOL)
            np.testing.assert_allclose(dl.cpu().numpy(), dl_ref.numpy(), rtol=RTOL, atol=2 * ATOL)
    # through the Python signature with autograd
    xd, ld = x.to(dev).requires_grad_(True), logc.to(dev).requires_grad_(True)
    y = linrec_general(xd, ld, logc=True, dim=1)
    gx, gl = torch.autograd.grad(y, (xd, ld), dy.to(dev))
    y_ref, dx_ref, dc_ref = _oracle_dim(x, c_eff, dy, 1, False)
    np.testing.assert_allclose(gx.cpu().numpy(), dx_ref.numpy(), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(gl.cpu().numpy(), (dc_ref * c_eff).numpy(), rtol=RTOL, atol=2 * ATOL)
    lb.check_status()
