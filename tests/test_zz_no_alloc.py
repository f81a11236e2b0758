"""The forward entry point that works on the library's built-in scratch buffer
(`linrec_b200_fwd_static`, for hosts that cannot allocate device memory for a workspace).

Collected last on purpose: it touches library-wide state (the one static buffer), so every other
test has already run if this one fails under `-x`.  It must pass in a fresh process as well as after
the rest of the suite; it therefore assumes nothing about what earlier calls left in the buffer.

Checked here, through the C ABI only: the same numbers as `linrec_b200_fwd` with a caller workspace
and as the CPU oracle (fp32 tolerance of the suite, rtol 1e-4 / atol 1e-5), on two calls in a row and
with a dirty buffer in between; that the calls leave the amount of free device memory unchanged;
that the status word of the built-in buffer can be read (and reports a wait that gave up); recovery
from counters left non-zero; rejection of problems whose scratch need exceeds the built-in 1 MiB.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-4, 1e-5


def _lib():
    from linrec_b200 import _capi
    return _capi, _capi.lib


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


def _static(_capi, L, x, c, rev, y=None):
    rows, n = x.shape
    if y is None:
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
    xh = torch.randn(shape, generator=g)
    ch = 0.5 + 0.5 * torch.rand(shape, generator=g)
    x, c = xh.to(dev), ch.to(dev)
    small = (x[:3, :4096 * 3].contiguous(), c[:3, :4096 * 3].contiguous()) if shape[1] >= 12288 else None
    for rev in (False, True):
        want = _with_workspace(_capi, L, x, c, rev)
        y1, y2 = torch.full_like(x, float("nan")), torch.full_like(x, float("nan"))
        y3 = torch.empty_like(small[0]) if small else None
        _static(_capi, L, x, c, rev)          # the first call on a device resolves the buffer's address
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(dev)
        first = _static(_capi, L, x, c, rev, y1)
        if small:   # a different problem in between leaves other tickets and descriptors in the shared buffer
            _static(_capi, L, small[0], small[1], not rev, y3)
        second = _static(_capi, L, x, c, rev, y2)
        free_after, _ = torch.cuda.mem_get_info(dev)
        assert free_after == free_before, "the static entry point changed the amount of free device memory"
        assert L.linrec_b200_status(None, torch.cuda.current_stream().cuda_stream) == 0
        torch.testing.assert_close(first, want, rtol=RTOL, atol=ATOL)
        torch.testing.assert_close(second, want, rtol=RTOL, atol=ATOL)
        ref = oracle.fwd_f32(xh.numpy(), ch.numpy(), reverse=rev)
        np.testing.assert_allclose(first.cpu().numpy(), ref, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(second.cpu().numpy(), ref, rtol=RTOL, atol=ATOL)


def test_static_scratch_status_word_and_recovery():
    """The built-in buffer is an ordinary workspace for the other entry points
    (`linrec_b200_static_workspace`).  A scan whose tickets start past the first piece of every row
    waits for predecessors that never publish: the wait ends by itself after its 20 ms budget and must
    show in `linrec_b200_status(NULL, stream)` exactly once.  Counters left non-zero in the buffer (as a
    failed or racing launch would leave them) must not spoil the next static call."""
    _capi, L = _lib()
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    ptr, nbytes = ctypes.c_void_p(), ctypes.c_size_t()
    assert L.linrec_b200_static_workspace(ctypes.byref(ptr), ctypes.byref(nbytes)) == 0
    assert ptr.value and ptr.value % 256 == 0 and nbytes.value == 1 << 20
    assert L.linrec_b200_status(None, stream) in (0, _capi.ERR_TIMEOUT)      # whatever earlier tests left: cleared now
    x = torch.ones(2, 4096 * 4, device=dev)
    y = torch.empty_like(x)
    o, keep = _capi.make_opts({"firstTicket": 2, "waitBudgetMs": 20})
    rc = L.linrec_b200_fwd(_capi.KIND_PIPE, x.data_ptr(), x.data_ptr(), y.data_ptr(), 2, 16384, 16384, 0, _capi.DTYPE_F32,
                           o, ptr, nbytes, stream)
    assert rc == 0, _capi.strerror(rc)
    assert L.linrec_b200_status(None, stream) == _capi.ERR_TIMEOUT
    assert L.linrec_b200_status(None, stream) == 0
    # counters as a failed launch would leave them: ticket counter and finished-CTA count not zero
    # (words 0 and 3 of the header; the status, word 1, and the epoch, word 2, keep their values)
    torch.cuda.synchronize()
    hdr = torch.empty(4, dtype=torch.int32, device=dev)
    _raw_copy(hdr.data_ptr(), ptr.value, 16)
    hdr[0], hdr[3] = 12345, 7
    _raw_copy(ptr.value, hdr.data_ptr(), 16)
    torch.cuda.synchronize()
    g = torch.Generator(device="cpu").manual_seed(7)
    xh, ch = torch.randn((6, 3 * 8192), generator=g), torch.rand((6, 3 * 8192), generator=g)
    got = _static(_capi, L, xh.to(dev), ch.to(dev), False)
    np.testing.assert_allclose(got.cpu().numpy(), oracle.fwd_f32(xh.numpy(), ch.numpy()), rtol=RTOL, atol=ATOL)
    assert L.linrec_b200_status(None, stream) == 0


def _raw_copy(dst: int, src: int, nbytes: int) -> None:
    """Device-to-device copy between raw addresses, through tensors that alias them."""
    n = nbytes // 4

    class _Alias:
        def __init__(self, ptr):
            self.__cuda_array_interface__ = {"shape": (n,), "typestr": "<i4", "data": (ptr, False), "version": 3}

    torch.as_tensor(_Alias(dst), device="cuda:0").copy_(torch.as_tensor(_Alias(src), device="cuda:0"))


def test_static_scratch_rejects_what_does_not_fit():
    _capi, L = _lib()
    dev = torch.device("cuda:0")
    # 70,000 rows of two tiles each would need 140,000 descriptors; no memory of that size is touched
    # because the call has to refuse before it launches anything
    small = torch.zeros(16, device=dev)
    before = _capi.launch_count()
    rc = L.linrec_b200_fwd_static(small.data_ptr(), small.data_ptr(), small.data_ptr(), 70000, 16384, 16384, 0,
                                  _capi.DTYPE_F32, torch.cuda.current_stream().cuda_stream)
    assert rc == _capi.ERR_SCRATCH_LIMIT and "scratch" in _capi.strerror(rc)
    assert _capi.launch_count() == before
    assert L.linrec_b200_fwd_static(None, None, None, 4, 64, 64, 0, _capi.DTYPE_F32, None) == _capi.ERR_INVALID_ARG
