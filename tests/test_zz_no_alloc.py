"""The forward entry point that works on the library's built-in scratch buffer
(`linrec_b200_fwd_static`, for hosts that cannot allocate device memory for a workspace).

Collected last on purpose: it touches library-wide state (the one static buffer), so every other
test has already run if this one fails under `-x`.  It must pass in a fresh process as well as after
the rest of the suite; it therefore assumes nothing about what earlier calls left in the buffer.

Checked here, through the C ABI only: the same numbers as `linrec_b200_fwd` with a caller workspace
(fp32 tolerance of the suite, rtol 1e-4 / atol 1e-5), on two calls in a row and with a dirty buffer in
between; rejection of problems whose scratch need exceeds the built-in 1 MiB.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


def _lib():
    from linrec_b200 import _capi
    L = _capi.lib
    i32, i64, vp = ctypes.c_int, ctypes.c_int64, ctypes.c_void_p
    L.linrec_b200_fwd_static.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, vp]
    L.linrec_b200_fwd_static.restype = i32
    return _capi, L


def _with_workspace(_capi, L, x, c, rev):
    rows, n = x.shape
    y = torch.empty_like(x)
    nbytes = L.linrec_b200_workspace_size(rows, n, _capi.DTYPE_F32)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device=x.device)
    stream = torch.cuda.current_stream().cuda_stream
    rc = L.linrec_b200_fwd(_capi.KIND_PIPE, x.data_ptr(), c.data_ptr(), y.data_ptr(), rows, n, n, int(rev),
                           _capi.DTYPE_F32, None, ws.data_ptr(), nbytes, stream)
    assert rc == 0, _capi.strerror(rc)
    torch.cuda.synchronize()
    return y


def _static(_capi, L, x, c, rev):
    rows, n = x.shape
    y = torch.full_like(x, float("nan"))
    stream = torch.cuda.current_stream().cuda_stream
    rc = L.linrec_b200_fwd_static(x.data_ptr(), c.data_ptr(), y.data_ptr(), rows, n, n, int(rev), _capi.DTYPE_F32, stream)
    assert rc == 0, _capi.strerror(rc)
    torch.cuda.synchronize()
    return y


@pytest.mark.parametrize("shape", [(48, 65536), (7, 3 * 8192 + 96), (300, 512), (5, 1001)],
                         ids=lambda s: f"{s[0]}x{s[1]}")
def test_static_scratch_matches_workspace_entry_point(shape):
    _capi, L = _lib()
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(4242)
    x = torch.randn(shape, generator=g).to(dev)
    c = (0.5 + 0.5 * torch.rand(shape, generator=g)).to(dev)
    for rev in (False, True):
        want = _with_workspace(_capi, L, x, c, rev)
        first = _static(_capi, L, x, c, rev)
        # a different problem in between leaves other tickets and descriptors in the shared buffer
        _static(_capi, L, x[:3, :4096 * 3].contiguous(), c[:3, :4096 * 3].contiguous(), not rev) if shape[1] >= 12288 else None
        second = _static(_capi, L, x, c, rev)
        torch.testing.assert_close(first, want, rtol=RTOL, atol=ATOL)
        torch.testing.assert_close(second, want, rtol=RTOL, atol=ATOL)


def test_static_scratch_rejects_what_does_not_fit():
    _capi, L = _lib()
    dev = torch.device("cuda:0")
    # 70,000 rows of two tiles each would need 140,000 descriptors; no memory of that size is touched
    # because the call has to refuse before it launches anything
    small = torch.zeros(16, device=dev)
    before = _capi.launch_count()
    rc = L.linrec_b200_fwd_static(small.data_ptr(), small.data_ptr(), small.data_ptr(), 70000, 16384, 16384, 0,
                                  _capi.DTYPE_F32, torch.cuda.current_stream().cuda_stream)
    assert rc == -8 and "scratch" in _capi.strerror(rc)
    assert _capi.launch_count() == before
    assert L.linrec_b200_fwd_static(None, None, None, 4, 64, 64, 0, _capi.DTYPE_F32, None) == _capi.ERR_INVALID_ARG
