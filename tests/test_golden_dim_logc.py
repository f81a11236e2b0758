"""Golden vectors for the `dim` and `logc` arguments, recorded from the unmodified reference's Python
operator (tests/golden/make_golden_dim_logc.py): the CPU oracle against them without a GPU, the CUDA
kernels against them with one."""
import os

import numpy as np
import pytest
import torch

import oracle

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = ["dim1_3x40x8", "dim2_2x3x40x4", "dim0_70x16", "dim1_2x130x12", "logc_last_4x100", "logc_last_1x2100",
         "logc_dim1_3x60x8"]
RTOL, ATOL = 1e-4, 1e-5


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(HERE, "golden", "linrec_golden_dim_logc.npz"))


def _last(a, dim):
    return np.ascontiguousarray(np.moveaxis(a, dim, -1))


def _back(a, dim):
    return np.ascontiguousarray(np.moveaxis(a, -1, dim))


@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("rev", [False, True])
def test_oracle_reproduces_the_reference(gold, name, rev):
    x, c, dy = gold[f"{name}/x"], gold[f"{name}/c"], gold[f"{name}/dy"]
    dim, logc = int(gold[f"{name}/dim"]) % x.ndim, bool(gold[f"{name}/logc"])
    tag = f"{name}/rev{int(rev)}"
    ce = torch.exp(torch.from_numpy(c)).numpy() if logc else c      # the reference's own exp
    y = oracle.fwd_f32(_last(x, dim), _last(ce, dim), reverse=rev)
    np.testing.assert_array_equal(_back(y, dim), gold[f"{tag}/y"])
    dx, dc = oracle.bwd_f32(_last(dy, dim), _last(ce, dim), y, reverse=rev)
    np.testing.assert_array_equal(_back(dx, dim), gold[f"{tag}/dx"])
    if not logc:
        np.testing.assert_array_equal(_back(dc, dim), gold[f"{tag}/dc"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
@pytest.mark.parametrize("rev", [False, True])
def test_kernels_against_the_reference(gold, name, rev):
    import linrec_b200
    from linrec_b200 import ops
    dev = torch.device("cuda:0")
    x, c, dy = (torch.from_numpy(gold[f"{name}/{k}"]).to(dev) for k in ("x", "c", "dy"))
    dim, logc = int(gold[f"{name}/dim"]) % x.dim(), bool(gold[f"{name}/logc"])
    tag = f"{name}/rev{int(rev)}"
    kw = {"logCoeffs": 1} if logc else {}
    yg = torch.from_numpy(gold[f"{tag}/y"]).to(dev)
    # through the Python signature (whatever path it picks), forward only
    y = linrec_b200.linrec_general(x, c, logc=logc, dim=dim, reverse=rev)
    np.testing.assert_allclose(y.cpu().numpy(), gold[f"{tag}/y"], rtol=RTOL, atol=ATOL)
    if dim != x.dim() - 1:
        # straight through the middle-axis entry points of the C ABI
        y = ops.linrec_dim_fwd(x, c, dim, rev, **kw)
        dx, dc = ops.linrec_dim_bwd(dy, c, yg, dim, rev, **kw)
    else:
        y = linrec_b200._C.linrec_pipe_fwd(inputs=x, coeffs=c, reverse=rev, **kw)
        dx, dc = linrec_b200._C.linrec_pipe_bwd(d_outputs=dy, coeffs=c, outputs=yg, reverse=rev, **kw)
    np.testing.assert_allclose(y.cpu().numpy(), gold[f"{tag}/y"], rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(dx.cpu().numpy(), gold[f"{tag}/dx"], rtol=RTOL, atol=ATOL)
    if not logc:
        np.testing.assert_allclose(dc.cpu().numpy(), gold[f"{tag}/dc"], rtol=RTOL, atol=2 * ATOL)
    linrec_b200.check_status()
