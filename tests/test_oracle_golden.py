"""The CPU oracle against the fixtures recorded from the unmodified reference (CPU only).

Bar: the fp32 C restatement and the torch loop restatement are BIT-EXACT against the reference's
Python implementation; the fp64 evaluation agrees within fp32 rounding noise.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import GOLDEN_CASES


@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("rev", [False, True])
def test_c_oracle_bit_exact(golden, name, rev):
    x, c, dy = golden[f"{name}/x"], golden[f"{name}/c"], golden[f"{name}/dy"]
    tag = f"{name}/rev{int(rev)}"
    y = oracle.fwd_f32(x, c, reverse=rev)
    assert y.shape == x.shape
    np.testing.assert_array_equal(y, golden[f"{tag}/y"])
    dx, dc = oracle.bwd_f32(dy, c, y, reverse=rev)
    np.testing.assert_array_equal(dx, golden[f"{tag}/dx"])
    np.testing.assert_array_equal(dc, golden[f"{tag}/dc"])


@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("rev", [False, True])
def test_torch_loop_bit_exact(golden, name, rev):
    x, c, dy = (torch.from_numpy(golden[f"{name}/{k}"]) for k in ("x", "c", "dy"))
    tag = f"{name}/rev{int(rev)}"
    y = oracle.pyloop_fwd(x, c, reverse=rev)
    assert torch.equal(y, torch.from_numpy(golden[f"{tag}/y"]))
    dx, dc = oracle.pyloop_bwd(dy, c, y, reverse=rev)
    assert torch.equal(dx, torch.from_numpy(golden[f"{tag}/dx"]))
    assert torch.equal(dc, torch.from_numpy(golden[f"{tag}/dc"]))


@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("rev", [False, True])
def test_f64_oracle_close(golden, name, rev):
    x, c, dy = golden[f"{name}/x"], golden[f"{name}/c"], golden[f"{name}/dy"]
    tag = f"{name}/rev{int(rev)}"
    y64 = oracle.fwd_f64(x, c, reverse=rev)
    np.testing.assert_allclose(y64, golden[f"{tag}/y"], rtol=1e-4, atol=1e-5)
    dx64, dc64 = oracle.bwd_f64(dy, c, y64, reverse=rev)
    np.testing.assert_allclose(dx64, golden[f"{tag}/dx"], rtol=1e-4, atol=1e-5)
    np.testing.assert_allclose(dc64, golden[f"{tag}/dc"], rtol=2e-4, atol=2e-5)


def test_definition_by_hand():
    """The recurrence written out by hand on a tiny case (y_0 = x_0, c_0 has no effect)."""
    x = np.array([[1.0, 2.0, 3.0]], np.float32)
    c = np.array([[9.0, 0.5, 2.0]], np.float32)
    np.testing.assert_array_equal(oracle.fwd_f32(x, c), [[1.0, 2.5, 8.0]])
    np.testing.assert_array_equal(oracle.fwd_f32(x, c, reverse=True), [[1.0 + 9.0 * 3.5, 3.5, 3.0]])
    dy = np.ones_like(x)
    y = oracle.fwd_f32(x, c)
    dx, dc = oracle.bwd_f32(dy, c, y)
    # dx_2 = 1, dx_1 = 1 + 2*1 = 3, dx_0 = 1 + 0.5*3 = 2.5 ; dc_i = dx_i * y_{i-1}
    np.testing.assert_array_equal(dx, [[2.5, 3.0, 1.0]])
    np.testing.assert_array_equal(dc, [[0.0, 3.0 * 1.0, 1.0 * 2.5]])


def test_empty_and_threads():
    assert oracle.fwd_f32(np.zeros((0, 5), np.float32), np.zeros((0, 5), np.float32)).shape == (0, 5)
    assert oracle.fwd_f32(np.zeros((3, 0), np.float32), np.zeros((3, 0), np.float32)).shape == (3, 0)
    assert oracle.threads() >= 1
