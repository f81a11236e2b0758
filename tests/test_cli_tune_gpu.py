"""The standalone harness (`linrec_cli`, counterpart of the reference's linrec/impl/cuda/executable.cpp:16-68)
and the sweep module (`linrec_b200.tune`, counterpart of eval/tune.py:58-134), on the GPU.

The harness verifies itself against the library's sequential operator; here its `--dump` output is
judged against the CPU oracle as well, so that the check does not rest on the library alone.
"""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-4, 1e-5


def _exe():
    from linrec_b200 import build
    return build.build_executable()


def _run(args):
    out = subprocess.run([_exe(), *map(str, args)], capture_output=True, text=True, timeout=300)
    rows = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    return out.returncode, rows, out.stderr


CASES = [
    dict(numseq=64, seqlen=4096, dtype="f32", bwd=False, rev=False),
    dict(numseq=5, seqlen=3 * 8192 + 64, dtype="f32", bwd=False, rev=True),
    dict(numseq=40, seqlen=1000, dtype="f32", bwd=True, rev=False),
    dict(numseq=7, seqlen=10001, dtype="f32", bwd=True, rev=True),
    dict(numseq=3, seqlen=1 << 18, dtype="f32", bwd=False, rev=False),      # super-chunks
    dict(numseq=16, seqlen=65536, dtype="bf16", bwd=False, rev=True),
    dict(numseq=16, seqlen=65536, dtype="bf16", bwd=True, rev=False),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"{c['numseq']}x{c['seqlen']}-{c['dtype']}-{'bwd' if c['bwd'] else 'fwd'}{'-rev' if c['rev'] else ''}")
def test_cli_verifies_and_its_dump_matches_the_oracle(case, tmp_path):
    args = ["--numseq", case["numseq"], "--seqlen", case["seqlen"], "--dtype", case["dtype"], "--iters", 2, "--warmup", 1,
            "--clo", 0.5, "--chi", 1.0, "--dump", tmp_path / "d"]
    if case["bwd"]:
        args.append("--bwd")
    if case["rev"]:
        args.append("--reverse")
    rc, rows, err = _run(args)
    assert rc == 0 and len(rows) == 1, err[-400:]
    r = rows[0]
    assert r["rc"] == 0 and r["status"] == 0 and r["out_of_tol"] == [0, 0] and r["gbps_median"] > 0
    shape = (case["numseq"], case["seqlen"])

    def load(what):
        raw = np.fromfile(tmp_path / f"d.{what}.bin", dtype=np.float32 if case["dtype"] == "f32" else np.uint16)
        if case["dtype"] == "f32":
            return raw.reshape(shape)
        return torch.from_numpy(raw.astype(np.int16)).view(torch.bfloat16).float().numpy().reshape(shape)

    rtol = RTOL if case["dtype"] == "f32" else 2.0 ** -7
    in0, c, out0 = load("in0"), load("c"), load("out0")
    assert 0.5 <= c.min() and c.max() <= 1.0
    if not case["bwd"]:
        np.testing.assert_allclose(out0, oracle.fwd_f32(in0, c, reverse=case["rev"]), rtol=rtol, atol=ATOL)
    else:
        y, out1 = load("y"), load("out1")
        dx, dc = oracle.bwd_f32(in0, c, y, reverse=case["rev"])
        np.testing.assert_allclose(out0, dx, rtol=rtol, atol=ATOL)
        np.testing.assert_allclose(out1, dc, rtol=rtol, atol=2 * ATOL * max(1.0, float(np.abs(y).max())))


def test_cli_middle_axis_mode():
    rc, rows, err = _run(["--numseq", 8, "--seqlen", 512, "--chan", 256, "--iters", 2, "--warmup", 1, "--bwd"])
    assert rc == 0 and rows and rows[0]["rc"] == 0 and rows[0]["out_of_tol"] == [0, 0], err[-400:]


def test_cli_reports_a_bad_option():
    rc, rows, err = _run(["--numseq", 4, "--seqlen", 4096, "--iters", 1, "--opt", "noSuchOption=1"])
    assert rc != 0 and rows and rows[0]["rc"] != 0 and "error" in rows[0]


def test_tune_sweep_lists_every_variant_and_picks_a_winner():
    """One row per compiled variant that can take the shape (the reference's tune prints one row per
    entry of `_C.config_list`, eval/tune.py:98-115), each verified, best first."""
    from linrec_b200 import _capi, tune
    rows = tune.sweep(64, 20004, iters=2, verify=True)
    offered = {cfg for cfg in _capi.config_list()}
    names = tune.NAMES
    seen = {tuple(r["opts"][n] for n in names) for r in rows}
    assert seen and seen <= offered
    # 20004 fp32 elements: rows of whole 16-byte chunks but not whole 128-byte lines -> every loader but the bulk copy
    assert {cfg for cfg in offered if cfg[4] in (0, 2, 3)} <= seen
    assert all(cfg[4] != 1 for cfg in seen)
    assert all(r["out_of_tol"] == [0, 0] for r in rows)
    assert rows == sorted(rows, key=lambda r: -r["gbps_median"])
    bwd = tune.sweep(64, 20004, bwd=True, iters=2, verify=True)
    assert bwd and all(r["bwd"] == 1 and r["out_of_tol"] == [0, 0] for r in bwd)


def test_tune_regimes_table():
    """The length/regime table: fixed element count, L = 2^8 ... 2^20, fp32 and bf16, forward and backward."""
    from linrec_b200 import tune
    table = tune.regimes(total_log2=22, iters=2)
    assert len(table) == 7 * 2 * 2
    assert {r["seqlen"] for r in table} == {1 << k for k in range(8, 21, 2)}
    assert all(r["rc"] == 0 and r["status"] == 0 and r["numseq"] * r["seqlen"] == 1 << 22 and r["gbps_median"] > 0 for r in table)
    assert tune.main(["--numseq", "32", "--seqlen", "8192", "--iters", "2"]) == 0
