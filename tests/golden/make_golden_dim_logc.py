"""Generate tests/golden/linrec_golden_dim_logc.npz from the UNMODIFIED reference implementation.

Golden vectors for the two wider arguments of the reference's Python operator
(linrec/impl/python/ops.py:8-61): `dim` (scan along a dimension other than the last) and `logc`
(coefficients given as logarithms).  Recorded by importing that file on CPU:

    python tests/golden/make_golden_dim_logc.py --reference <path to the safelix/linrec checkout>

For `dim` the forward outputs and both gradients are recorded.  For `logc` the forward outputs and
d_inputs are recorded; the reference's d_coeffs under `logc` multiplies by the SHIFTED coefficients
(ops.py:33-38), which is not the derivative of its own forward, so it is left out.
"""
from __future__ import annotations

import argparse
import os

import numpy as np
import torch

from make_golden import SEED, load_reference_ops

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, shape, dim, logc)
CASES = [
    ("dim1_3x40x8", (3, 40, 8), 1, False),
    ("dim2_2x3x40x4", (2, 3, 40, 4), 2, False),
    ("dim0_70x16", (70, 16), 0, False),
    ("dim1_2x130x12", (2, 130, 12), 1, False),
    ("logc_last_4x100", (4, 100), -1, True),
    ("logc_last_1x2100", (1, 2100), -1, True),
    ("logc_dim1_3x60x8", (3, 60, 8), 1, True),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get(
        "LINREC_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(HERE))), "reference")))
    ap.add_argument("--out", default=os.path.join(HERE, "linrec_golden_dim_logc.npz"))
    args = ap.parse_args()
    ref = load_reference_ops(args.reference)
    gen = torch.Generator(device="cpu").manual_seed(SEED + 1)
    out = {}
    for name, shape, dim, logc in CASES:
        x = torch.randn(shape, generator=gen, dtype=torch.float32)
        c = 0.3 + 0.7 * torch.rand(shape, generator=gen, dtype=torch.float32)
        if logc:
            c = torch.log(c)
        dy = torch.randn(shape, generator=gen, dtype=torch.float32)
        out[f"{name}/x"], out[f"{name}/c"], out[f"{name}/dy"] = x.numpy(), c.numpy(), dy.numpy()
        out[f"{name}/dim"], out[f"{name}/logc"] = np.int64(dim), np.int64(logc)
        for rev in (False, True):
            tag = f"{name}/rev{int(rev)}"
            y = ref.linrec_ref_fwd(x, c, logc=logc, dim=dim, reverse=rev).contiguous()
            dx, dc = ref.linrec_ref_bwd(dy, c, y, logc=logc, dim=dim, reverse=rev)
            out[f"{tag}/y"], out[f"{tag}/dx"] = y.numpy(), dx.contiguous().numpy()
            if not logc:
                out[f"{tag}/dc"] = dc.contiguous().numpy()
                # cross-check against autograd through the reference's own loop
                xa, ca = x.clone().requires_grad_(True), c.clone().requires_grad_(True)
                ya = ref.linrec_ref_fwd(xa, ca, logc=False, dim=dim, reverse=rev)
                gx, gc = torch.autograd.grad(ya, (xa, ca), dy)
                assert torch.allclose(gx, dx, rtol=1e-5, atol=1e-6) and torch.allclose(gc, dc, rtol=1e-5, atol=1e-6)
    np.savez_compressed(args.out, **out)
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
