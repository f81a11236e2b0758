"""Sweep of the compiled kernel variants -- what the reference does with eval/tune.py:58-134, which
times every entry of `_C.config_list` per sequence length and prints the best one.  Here the
standalone harness does the timing (`linrec_cli --sweep`, CUDA events, no Python in the loop) and
this module formats its JSON lines.

    python -m linrec_b200.tune --numseq 4096 --seqlen 65536 [--bwd] [--dtype bf16]
    python -m linrec_b200.tune --regimes          # 2^28 elements, L = 2^8 ... 2^20, selector defaults

The selector defaults in csrc/capi.cu (`make_plan`) are the winners of these sweeps on B200.
"""
from __future__ import annotations

import argparse
import json
import subprocess
import sys

from . import build as _build

NAMES = ("kElemsPerThread", "kThreadsPerBlock", "kStages", "kOutBuffers", "memcode")


def run_cli(args):
    exe = _build.build_executable()
    out = subprocess.run([exe, *map(str, args)], check=False, capture_output=True, text=True)
    rows = [json.loads(line) for line in out.stdout.splitlines() if line.startswith("{")]
    if not rows:
        raise RuntimeError(f"linrec_cli produced no result: {out.stderr.strip()[-400:]}")
    return rows


def sweep(numseq, seqlen, bwd=False, dtype="f32", iters=10, verify=False):
    a = ["--numseq", numseq, "--seqlen", seqlen, "--dtype", dtype, "--iters", iters, "--sweep"]
    if bwd:
        a.append("--bwd")
    if not verify:
        a.append("--no-verify")
    rows = [r for r in run_cli(a) if r["rc"] == 0]
    rows.sort(key=lambda r: -r["gbps_median"])
    return rows


def regimes(total_log2=28, iters=5):
    table = []
    for log2l in range(8, 21, 2):
        L = 1 << log2l
        n = (1 << total_log2) // L
        for dtype in ("f32", "bf16"):
            for bwd in (False, True):
                a = ["--numseq", n, "--seqlen", L, "--dtype", dtype, "--iters", iters, "--no-verify"]
                if bwd:
                    a.append("--bwd")
                table.append(run_cli(a)[0])
    return table


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--numseq", type=int, default=4096)
    ap.add_argument("--seqlen", type=int, default=65536)
    ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--dtype", default="f32", choices=["f32", "bf16"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--verify", action="store_true")
    ap.add_argument("--regimes", action="store_true")
    ns = ap.parse_args(argv)
    if ns.regimes:
        print(f"{'seqlen':>9} {'rows':>9} {'dtype':>5} {'pass':>4} {'ms':>8} {'GB/s':>8} {'Gelem/s':>8}")
        for r in regimes(iters=ns.iters):
            print(f"{r['seqlen']:>9} {r['numseq']:>9} {r['dtype']:>5} {'bwd' if r['bwd'] else 'fwd':>4} "
                  f"{r['ms_median']:>8.3f} {r['gbps_median']:>8.0f} {r['gelem_s']:>8.1f}")
        return 0
    print(" ".join(f"{n:>17}" for n in NAMES) + f" {'ms':>8} {'GB/s':>8}")
    for r in sweep(ns.numseq, ns.seqlen, ns.bwd, ns.dtype, ns.iters, ns.verify):
        print(" ".join(f"{r['opts'].get(n, -1):>17}" for n in NAMES) + f" {r['ms_median']:>8.3f} {r['gbps_median']:>8.0f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
