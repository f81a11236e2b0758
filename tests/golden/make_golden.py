"""Generate tests/golden/linrec_golden.npz from the UNMODIFIED reference implementation.

The reference ships no golden vectors or known-answer tests, so the fixtures are made here by
importing its Python implementation (linrec/impl/python/ops.py: `linrec_ref_fwd`,
`linrec_ref_bwd`, and autograd through `linrec_ref`) on CPU and recording inputs and outputs.
Run on a machine that has the reference checked out:

    python tests/golden/make_golden.py --reference <path to the safelix/linrec checkout>

The inputs are stored with the outputs, so the fixtures do not depend on a torch RNG stream.
"""
from __future__ import annotations

import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, shape, coefficient range)
CASES = [
    ("len1", (3, 1), (0.0, 1.0)),
    ("len2", (4, 2), (0.0, 1.0)),
    ("odd17", (3, 17), (0.0, 1.0)),
    ("pow64", (5, 64), (0.0, 1.0)),
    ("batch3d", (2, 3, 33), (0.0, 1.0)),
    ("ragged300", (2, 300), (0.0, 1.0)),
    ("slow1000", (1, 1000), (0.9, 1.0)),
    ("slower2100", (1, 2100), (0.99, 1.0)),
]
SEED = 12334567890  # the reference's own evaluation seed (eval/test.py:45)


def load_reference_ops(reference: str):
    path = os.path.join(reference, "linrec", "impl", "python", "ops.py")
    spec = importlib.util.spec_from_file_location("reference_python_ops", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get(
        "LINREC_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")))
    ap.add_argument("--out", default=os.path.join(HERE, "linrec_golden.npz"))
    args = ap.parse_args()
    ref = load_reference_ops(args.reference)

    gen = torch.Generator(device="cpu").manual_seed(SEED)
    out = {}
    for name, shape, (lo, hi) in CASES:
        x = torch.randn(shape, generator=gen, dtype=torch.float32)
        c = lo + (hi - lo) * torch.rand(shape, generator=gen, dtype=torch.float32)
        dy = torch.randn(shape, generator=gen, dtype=torch.float32)
        out[f"{name}/x"], out[f"{name}/c"], out[f"{name}/dy"] = x.numpy(), c.numpy(), dy.numpy()
        for rev in (False, True):
            tag = f"{name}/rev{int(rev)}"
            y = ref.linrec_ref_fwd(x, c, reverse=rev)
            dx, dc = ref.linrec_ref_bwd(dy, c, y, reverse=rev)
            # the analytic backward must agree with autograd through the sequential loop
            xg, cg = x.clone().requires_grad_(True), c.clone().requires_grad_(True)
            ya = ref.linrec_ref_fwd(xg, cg, reverse=rev)
            gx, gc = torch.autograd.grad(ya, (xg, cg), dy)
            assert torch.allclose(gx, dx, rtol=1e-5, atol=1e-6), (name, rev)
            assert torch.allclose(gc, dc, rtol=1e-5, atol=1e-6), (name, rev)
            # and the autograd.Function wrapper must return the same numbers
            xf, cf = x.clone().requires_grad_(True), c.clone().requires_grad_(True)
            yf = ref.linrec_ref(xf, cf, reverse=rev)
            fx, fc = torch.autograd.grad(yf, (xf, cf), dy)
            assert torch.equal(yf.detach(), y) and torch.equal(fx, dx) and torch.equal(fc, dc)
            out[f"{tag}/y"] = y.contiguous().numpy()
            out[f"{tag}/dx"] = dx.contiguous().numpy()
            out[f"{tag}/dc"] = dc.contiguous().numpy()
    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes", file=sys.stderr)


if __name__ == "__main__":
    main()
