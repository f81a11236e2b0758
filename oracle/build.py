"""Build recipe for the CPU oracle (TEST INFRASTRUCTURE ONLY).

`build_oracle()` compiles oracle/linrec_oracle.c into oracle/liblinrec_oracle.so with gcc.
`build_ref()` compiles, when the reference tree is present on this machine, the reference's own
sequential CUDA kernels (linrec/impl/cuda/linrec_ref.cuh, included from where it lies -- no
reference source is copied into this repository) behind a small C shim into
oracle/_ref/liblinrec_refcuda.so.  That second library is a GPU-side checker: it can only run
where a GPU is visible, and it is used by tests only.

Run as a script to build both:  python oracle/build.py [--reference /path/to/reference]
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liblinrec_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "liblinrec_refcuda.so")
# the reference checkout: $LINREC_REFERENCE_DIR, else a directory "reference" next to this repository
DEFAULT_REFERENCE = os.environ.get("LINREC_REFERENCE_DIR",
                                   os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def _newer(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "linrec_oracle.c")
    if not force and _newer(ORACLE_SO, src, __file__):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-fPIC", "-shared", "-std=c11", "-ffp-contract=off", "-fno-fast-math",
           "-fopenmp", "-fvisibility=hidden", "-o", ORACLE_SO, src]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_ref(reference: str = DEFAULT_REFERENCE, force: bool = False) -> str | None:
    """Compile the reference's linrec_ref kernels from the reference tree, if it is there."""
    hdr_dir = os.path.join(reference, "linrec", "impl", "cuda")
    hdr = os.path.join(hdr_dir, "linrec_ref.cuh")
    shim = os.path.join(HERE, "refcuda_shim.cu")
    if not os.path.exists(hdr):
        return REF_SO if os.path.exists(REF_SO) else None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, hdr, shim, __file__):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    # Same code-generation switches as the reference's build (linrec/impl/cuda/build.py:15-47):
    # -O3 and --use_fast_math (FMA contraction, flush-to-zero); the architecture is pinned here.
    cmd = [nvcc, "-O3", "--use_fast_math", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           "-gencode", "arch=compute_100a,code=sm_100a", "-I", hdr_dir, "-o", REF_SO, shim]
    subprocess.run(cmd, check=True)
    return REF_SO


if __name__ == "__main__":
    ref = DEFAULT_REFERENCE
    if "--reference" in sys.argv:
        ref = sys.argv[sys.argv.index("--reference") + 1]
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(ref, force="--force" in sys.argv))
