"""CPU-only checks of the drop-in boundary: the shared library loads, exports every symbol that
include/linrec_b200.h declares, answers its introspection calls and rejects bad arguments before
touching a device.  No compute call is made here."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "linrec_b200.h")).read()
    return sorted(set(re.findall(r"LINREC_API\s+[\w\s\*]+?\b(linrec_b200_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = _declared_symbols()
    for must in ("linrec_b200_fwd", "linrec_b200_bwd", "linrec_b200_workspace_size", "linrec_b200_status",
                 "linrec_b200_attrs", "linrec_b200_config_names", "linrec_b200_config_list"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    from linrec_b200 import _capi
    for name in _declared_symbols():
        assert hasattr(_capi.lib, name), f"{name} is declared in the header but not exported"


def test_introspection_without_a_device():
    from linrec_b200 import _capi
    names = _capi.config_names()
    assert names == ["kElemsPerThread", "kThreadsPerBlock", "kStages", "kOutBuffers", "memcode"]
    configs = _capi.config_list()
    assert len(configs) >= 4 and all(len(c) == len(names) for c in configs)
    assert any(c[-1] == 0 for c in configs) and any(c[-1] == 1 for c in configs)
    assert _capi.lib.linrec_b200_version() >= 100
    assert _capi.strerror(0) == "ok" and "variant" in _capi.strerror(_capi.ERR_NOT_IMPLEMENTED)


def test_workspace_size_rules():
    from linrec_b200 import _capi
    ws = _capi.lib.linrec_b200_workspace_size
    assert ws(0, 0, 0) == 256 and ws(10, 100, 0) == 256        # short rows: header only
    big = ws(8, 1 << 20, 0)
    assert big % 256 == 0 and big >= 256 + 8 * ((1 << 20) // 2048) * 16
    # a handful of very long rows may be cut into super-chunks: room for their records on top of the
    # descriptors (about 1024 records of 16 bytes), but only in that regime
    many = ws(4096, 1 << 20, 0)
    assert many == 256 + 4096 * ((1 << 20) // 1024) * 16          # the smallest tile any variant uses: 1024
    assert big >= 256 + 8 * ((1 << 20) // 1024) * 16 + 1024 * 16
    assert ws(8, 1 << 16, 0) == 256 + 8 * ((1 << 16) // 1024) * 16          # rows too short to be cut
    # (the backward operator cuts long rows while there are fewer than four per SM)
    assert ws(256, 1 << 20, 0) >= 256 + 256 * ((1 << 20) // 1024) * 16 + 1024 * 16
    # the entry points of version 0.2.0 (the fix-up calls take the operands) are there
    assert _capi.lib.linrec_b200_version() >= 200


def test_bad_arguments_are_refused_before_any_launch():
    from linrec_b200 import _capi
    L = _capi.lib
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    assert L.linrec_b200_fwd(_capi.KIND_PIPE, None, p, p, 2, 8, 8, 0, 0, None, None, 0, None) == _capi.ERR_INVALID_ARG
    assert L.linrec_b200_fwd(_capi.KIND_PIPE, p, p, p, 2, 8, 4, 0, 0, None, None, 0, None) == _capi.ERR_INVALID_ARG
    assert L.linrec_b200_fwd(_capi.KIND_PIPE, p, p, p, -1, 8, 8, 0, 0, None, None, 0, None) == _capi.ERR_INVALID_ARG
    assert L.linrec_b200_fwd(_capi.KIND_PIPE, p, p, p, 2, 8, 8, 0, 7, None, None, 0, None) == _capi.ERR_NOT_IMPLEMENTED
    assert L.linrec_b200_fwd(99, p, p, p, 2, 8, 8, 0, 0, None, None, 0, None) == _capi.ERR_INVALID_ARG
    assert L.linrec_b200_fwd(_capi.KIND_PIPE, p + 2, p, p, 2, 8, 8, 0, 0, None, None, 0, None) == _capi.ERR_INVALID_ARG
    # empty problems succeed without a device
    assert L.linrec_b200_fwd(_capi.KIND_PIPE, None, None, None, 0, 8, 8, 0, 0, None, None, 0, None) == _capi.OK
    opts, keep = _capi.make_opts({"noSuchOption": 1})
    assert L.linrec_b200_fwd(_capi.KIND_PIPE, p, p, p, 2, 8, 8, 0, 0, opts, None, 0, None) == _capi.ERR_NOT_IMPLEMENTED
    # a NULL workspace stands for the built-in buffer of the current device: without a device the look-up fails
    assert L.linrec_b200_status(None, None) == _capi.ERR_CUDA


def test_error_translation():
    from linrec_b200 import _capi
    with pytest.raises(NotImplementedError):
        _capi.raise_for(_capi.ERR_NOT_IMPLEMENTED, "x")
    with pytest.raises(RuntimeError):
        _capi.raise_for(_capi.ERR_TOO_LONG, "x")
    _capi.raise_for(_capi.OK, "x")


def test_row_layout_host_logic():
    from linrec_b200.ops import _row_layout
    assert _row_layout(torch.empty(7)) == (1, 7, 7)
    assert _row_layout(torch.empty(3, 7)) == (3, 7, 7)
    assert _row_layout(torch.empty(2, 3, 7)) == (6, 7, 7)
    assert _row_layout(torch.empty(3, 10)[:, :7]) == (3, 7, 10)
    assert _row_layout(torch.empty(2, 3, 10)[:, :, :7]) == (6, 7, 10)
    assert _row_layout(torch.empty(3, 2, 7).permute(1, 0, 2)) is None
    assert _row_layout(torch.empty(1, 7).expand(3, 7)) is None
    assert _row_layout(torch.empty(1, 3, 1, 7)) == (3, 7, 7)


def test_operator_surface_and_fake_kernels():
    import linrec
    import linrec_b200
    from linrec.impl.cuda import ops as cuops
    assert linrec.linrec is linrec_b200.linrec_pipe
    for fam in ("ref", "tile", "pipe"):
        assert hasattr(torch.ops.linreccuda, f"linrec_{fam}_fwd") and hasattr(torch.ops.linreccuda, f"linrec_{fam}_bwd")
        assert hasattr(cuops, f"linrec_{fam}") and hasattr(cuops._C, f"linrec_{fam}_fwd")
    x = torch.empty(4, 5, 6, device="meta")
    y = torch.ops.linreccuda.linrec_pipe_fwd(x, x, False)
    assert y.shape == x.shape and y.device.type == "meta"
    dx, dc = torch.ops.linreccuda.linrec_pipe_bwd(x, x, x, True)
    assert dx.shape == x.shape and dc.shape == x.shape


def test_cpu_tensors_are_rejected():
    """There is no CPU implementation behind the operators."""
    import linrec_b200
    a = torch.zeros(2, 8)
    with pytest.raises(Exception):
        linrec_b200.linrec(a, a)
    with pytest.raises(RuntimeError):
        linrec_b200._C.linrec_pipe_fwd(inputs=a, coeffs=a)


def test_dim_entry_points_host_logic():
    """Scan along the middle axis: sizing and refusals that need no device."""
    from linrec_b200 import _capi
    L = _capi.lib
    ws = L.linrec_b200_dim_workspace_size
    assert ws(0, 0, 10, 10, 0, None) == 256
    # many columns, short sequences: one job per column or few generations -> small workspace
    assert ws(0, 4096, 64, 128, 0, None) == 256
    # enough columns for chained jobs: one 16-byte descriptor per channel and job
    n = ws(0, 256, 1024, 1024, 0, None)
    assert n % 256 == 0 and 256 < n < 256 * 1024 * 1024 * 4 // 8
    # a handful of columns: every chunk is a job
    few = ws(1, 1, 1 << 16, 64, 0, None)
    assert few >= 256 + (1 << 16) // 64 * 2 * 32 * 16
    # options that match no compiled variant
    opts, keep = _capi.make_opts({"kThreadsPerBlock": 96})
    assert ws(0, 4, 100, 64, 0, opts) == 0
    buf = (ctypes.c_float * 64)()
    p = ctypes.addressof(buf)
    p16 = (p + 15) & ~15
    assert L.linrec_b200_fwd_dim(None, None, None, 0, 8, 8, 0, 0, None, None, 0, None) == _capi.OK
    assert L.linrec_b200_fwd_dim(p16, p16, p16, -1, 8, 8, 0, 0, None, None, 0, None) == _capi.ERR_INVALID_ARG
    assert L.linrec_b200_fwd_dim(p16, p16, p16, 1, 2, 4, 0, 9, None, None, 0, None) == _capi.ERR_NOT_IMPLEMENTED
    assert L.linrec_b200_fwd_dim(None, p16, p16, 1, 2, 4, 0, 0, None, None, 0, None) == _capi.ERR_INVALID_ARG
    # 3 channels of 4 bytes are not whole 16-byte chunks; a pointer 4 bytes off is not aligned
    assert L.linrec_b200_fwd_dim(p16, p16, p16, 1, 2, 3, 0, 0, None, None, 0, None) == _capi.ERR_UNALIGNED
    assert L.linrec_b200_fwd_dim(p16 + 4, p16, p16, 1, 2, 4, 0, 0, None, None, 0, None) == _capi.ERR_UNALIGNED
    assert L.linrec_b200_last_cuda_error() is not None


def test_dim_eligibility_helpers():
    from linrec_b200.ops import dim_eligible, dim_worthwhile
    t = torch.empty(4, 10, 8)
    assert not dim_eligible(t, 1)                       # not a CUDA tensor
    m = torch.empty(4, 10, 8, device="meta")
    assert not dim_eligible(m, 1)
    assert not dim_worthwhile(t, 1)
