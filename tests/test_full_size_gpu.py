"""The task's configurations at their full sizes (GPU only).

At these sizes the CPU oracle is run on a sample of rows (it is a sequential loop); the whole tensor
is covered by size-independent properties instead:
  * agreement with the sequential one-thread-per-row operator of the library over ALL elements
    (an independent code path: no tiles, no look-back, no bulk copies),
  * agreement with the reference's own CUDA kernels where the checker library was built,
  * reverse == flip(forward(flip)),
  * linearity in x:  scan(a*x1 + x2, c) == a*scan(x1, c) + scan(x2, c).
Inputs are seeded synthetic tensors with the distributions the configurations name.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-4, 1e-5
SEED = 12334567890


def _lb():
    import linrec_b200
    return linrec_b200


def _gen(shape, clo, chi, seed, dev):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(shape, device=dev, generator=g)
    c = clo + (chi - clo) * torch.rand(shape, device=dev, generator=g)
    dy = torch.randn(shape, device=dev, generator=g)
    return x, c, dy


def _sample_rows(n, k=6):
    rs = np.random.RandomState(0)
    rows = sorted(set([0, n - 1] + list(rs.randint(0, n, size=k))))
    return torch.tensor(rows)


def _judge(ours, seq32, truth64, what):
    """ours vs the fp64 evaluation: at most twice the sequential fp32 oracle's own error, and at most
    twice its share of elements outside rtol 1e-4 / atol 1e-5 (or 1e-4 of the elements)."""
    err, err_seq = float(np.abs(ours - truth64).max()), float(np.abs(seq32 - truth64).max())
    assert err <= 2 * err_seq + ATOL, f"{what}: {err:.3g} vs sequential {err_seq:.3g}"
    tol = ATOL + RTOL * np.abs(truth64)
    miss, miss_seq = (np.abs(ours - truth64) > tol).mean(), (np.abs(seq32 - truth64) > tol).mean()
    assert miss <= max(1e-4, 2 * miss_seq), f"{what}: miss share {miss:.2e} vs sequential {miss_seq:.2e}"


def _refcuda():
    path = os.path.join(os.path.dirname(oracle.__file__), "_ref", "liblinrec_refcuda.so")
    if not os.path.exists(path):
        return None
    L = ctypes.CDLL(path)
    vp, i32 = ctypes.c_void_p, ctypes.c_int
    L.refcuda_fwd_f32.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    L.refcuda_bwd_f32.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, vp]
    return L


@pytest.mark.parametrize("rev", [False, True])
def test_config2_readme_shape_against_reference_kernel(rev):
    """(512, 65536) fp32, x~N(0,1), c~U[0,1): forward in both directions against linrec_ref."""
    lb, dev = _lb(), torch.device("cuda:0")
    x, c, _ = _gen((512, 65536), 0.0, 1.0, SEED + 2, dev)
    y = lb.linrec(x, c, reverse=rev)
    R = _refcuda()
    y_ref = torch.empty_like(x)
    if R is not None:
        assert R.refcuda_fwd_f32(x.data_ptr(), c.data_ptr(), y_ref.data_ptr(), 512, 65536, int(rev),
                                 torch.cuda.current_stream().cuda_stream) == 0
    else:
        y_ref = lb._C.linrec_ref_fwd(inputs=x, coeffs=c, reverse=rev)
    torch.testing.assert_close(y, y_ref, rtol=RTOL, atol=ATOL)
    rows = _sample_rows(512)
    np.testing.assert_allclose(y[rows].cpu().numpy(), oracle.fwd_f32(x[rows].cpu().numpy(), c[rows].cpu().numpy(), reverse=rev),
                               rtol=RTOL, atol=ATOL)
    # reverse == flip o forward o flip
    y2 = lb.linrec(x.flip(-1).contiguous(), c.flip(-1).contiguous(), reverse=not rev).flip(-1)
    torch.testing.assert_close(y, y2, rtol=RTOL, atol=ATOL)
    lb.check_status()


def test_config3_autograd_mamba_layout():
    """(16, 2048, 8192) fp32, c~U(0.9,1), dy~N(0,1): y, dx, dc through autograd."""
    lb, dev = _lb(), torch.device("cuda:0")
    x, c, dy = _gen((16, 2048, 8192), 0.9, 1.0, SEED + 3, dev)
    x.requires_grad_(True); c.requires_grad_(True)
    y = lb.linrec(x, c)
    gx, gc = torch.autograd.grad(y, (x, c), dy)
    # all elements against the sequential operator of the library (independent code path)
    y_seq = lb._C.linrec_ref_fwd(inputs=x.detach(), coeffs=c.detach())
    torch.testing.assert_close(y.detach(), y_seq, rtol=RTOL, atol=ATOL)
    dx_seq, dc_seq = lb._C.linrec_ref_bwd(d_outputs=dy, coeffs=c.detach(), outputs=y_seq)
    torch.testing.assert_close(gx, dx_seq, rtol=RTOL, atol=ATOL)
    torch.testing.assert_close(gc, dc_seq, rtol=RTOL, atol=1e-4)   # |y| reaches ~10 here: dc = dx*y
    del y_seq, dx_seq, dc_seq
    # sampled rows against the CPU oracle, with autograd semantics of the reference
    x2, c2, dy2 = (t.detach().reshape(-1, 8192) for t in (x, c, dy))
    rows = _sample_rows(x2.shape[0])
    xs, cs, dys = (t[rows].cpu().numpy() for t in (x2, c2, dy2))
    y_o = oracle.fwd_f32(xs, cs)
    dx_o, dc_o = oracle.bwd_f32(dys, cs, y_o)
    np.testing.assert_allclose(y.detach().reshape(-1, 8192)[rows].cpu().numpy(), y_o, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(gx.reshape(-1, 8192)[rows].cpu().numpy(), dx_o, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(gc.reshape(-1, 8192)[rows].cpu().numpy(), dc_o, rtol=RTOL, atol=1e-4)
    # linearity in x
    a = 0.37
    x1 = torch.randn_like(x2)
    lhs = lb.linrec(a * x1 + x2, c2)
    rhs = a * lb.linrec(x1, c2) + y.detach().reshape(-1, 8192)
    torch.testing.assert_close(lhs, rhs, rtol=1e-3, atol=1e-4)
    lb.check_status()


@pytest.mark.parametrize("log2L", [8, 10, 12, 14, 16, 18, 20])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_config4_length_sweep(log2L, dtype):
    """2^28 elements, L = 2^8 ... 2^20, x~N(0,1), c~U[0,1): forward and backward."""
    lb, dev = _lb(), torch.device("cuda:0")
    L = 1 << log2L
    n = (1 << 28) // L
    x, c, dy = (t.to(dtype) for t in _gen((n, L), 0.0, 1.0, SEED + 4 + log2L, dev))
    rtol = RTOL if dtype == torch.float32 else 2.0 ** -7
    rev = bool(log2L % 4 == 0)
    y = lb.linrec(x, c, reverse=rev)
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy, coeffs=c, outputs=y, reverse=rev)
    rows = _sample_rows(n, 4 if L >= (1 << 18) else 16)
    xs, cs, dys, ys = (t[rows].float().cpu().numpy() for t in (x, c, dy, y))
    y_o = oracle.fwd_f32(xs, cs, reverse=rev)
    np.testing.assert_allclose(ys, y_o, rtol=rtol, atol=ATOL)
    dx_o, dc_o = oracle.bwd_f32(dys, cs, ys, reverse=rev)
    np.testing.assert_allclose(dx[rows].float().cpu().numpy(), dx_o, rtol=rtol, atol=ATOL)
    np.testing.assert_allclose(dc[rows].float().cpu().numpy(), dc_o, rtol=rtol, atol=2 * ATOL)
    # every element: against the library's sequential operator
    y_seq = lb._C.linrec_ref_fwd(inputs=x, coeffs=c, reverse=rev)
    torch.testing.assert_close(y.float(), y_seq.float(), rtol=rtol, atol=ATOL)
    lb.check_status()


@pytest.mark.parametrize("rev", [False, True])
def test_config5_slab_slow_decay(rev):
    """A row slab of the (8192, 2^20) configuration, c~U(0.99,1): 512 rows x 2^20, forward and
    backward, judged against the fp64 evaluation on sampled rows (two valid fp32 orders already
    differ by more than the nominal tolerance for these coefficients)."""
    lb, dev = _lb(), torch.device("cuda:0")
    n, L = 512, 1 << 20
    x, c, dy = _gen((n, L), 0.99, 1.0, SEED + 5, dev)
    y = lb.linrec(x, c, reverse=rev)
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=dy, coeffs=c, outputs=y, reverse=rev)
    rows = _sample_rows(n, 3)
    xs, cs, dys, ys = (t[rows].cpu().numpy() for t in (x, c, dy, y))
    y32, y64 = oracle.fwd_f32(xs, cs, reverse=rev), oracle.fwd_f64(xs, cs, reverse=rev)
    _judge(ys, y32, y64, "y")
    dx32, dc32 = oracle.bwd_f32(dys, cs, ys, reverse=rev)
    dx64, dc64 = oracle.bwd_f64(dys, cs, ys.astype(np.float64), reverse=rev)
    _judge(dx[rows].cpu().numpy(), dx32, dx64, "dx")
    scale = max(1.0, float(np.abs(ys).max()))
    _judge(dc[rows].cpu().numpy() / scale, dc32 / scale, dc64 / scale, "dc")
    lb.check_status()


def test_more_than_2_to_31_elements():
    """64-bit element offsets: (4100, 2^19) = 2.15e9 elements per tensor (the reference's kernels
    index with int and stop below 2^31, linrec_pipe.cuh:14, linrec_tile.cu:61).  Rows at the far end
    of the tensor are checked against the CPU oracle, forward and backward."""
    lb, dev = _lb(), torch.device("cuda:0")
    n, L = 4100, 1 << 19
    assert n * L > 2 ** 31
    g = torch.Generator(device=dev).manual_seed(SEED + 6)
    x = torch.randn((n, L), device=dev, generator=g)
    c = torch.rand((n, L), device=dev, generator=g)
    y = lb.linrec(x, c)
    rows = torch.tensor([0, 1, 2047, 4095, 4096, 4099])
    np.testing.assert_allclose(y[rows].cpu().numpy(), oracle.fwd_f32(x[rows].cpu().numpy(), c[rows].cpu().numpy()),
                               rtol=RTOL, atol=ATOL)
    # backward writes two tensors: reuse x as the upstream gradient to stay within memory
    dx, dc = lb._C.linrec_pipe_bwd(d_outputs=x, coeffs=c, outputs=y)
    dx_o, dc_o = oracle.bwd_f32(x[rows].cpu().numpy(), c[rows].cpu().numpy(), y[rows].cpu().numpy())
    np.testing.assert_allclose(dx[rows].cpu().numpy(), dx_o, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(dc[rows].cpu().numpy(), dc_o, rtol=RTOL, atol=2 * ATOL)
    lb.check_status()
