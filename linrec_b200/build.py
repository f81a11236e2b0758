"""In-tree build of the CUDA library (and of the standalone harness) for sm_100a.

    python -m linrec_b200.build [--force] [--exe]

The library is a plain C-ABI shared object built by nvcc alone: no torch headers, no Python
headers.  The reference builds its extension just-in-time with torch's cpp_extension and no
architecture flag (linrec/impl/cuda/build.py:15-80); here the architecture is pinned and the
result lives next to the sources so that it travels with the tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(ROOT, "include")
LIB_PATH = os.path.join(PKG, "liblinrec_b200.so")
EXE_PATH = os.path.join(PKG, "_build", "linrec_cli")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xfatbin=-compress-all", "-Xcompiler", "-fPIC,-fvisibility=hidden"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA library of linrec_b200 cannot be built")
    return exe


def _sources(*names):
    return [os.path.join(CSRC, n) for n in names]


def _digest(deps) -> str:
    import hashlib
    h = hashlib.sha256()
    for d in sorted(deps):
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target: str, deps) -> bool:
    """Content based (a digest of the sources is stored next to the target): file times do not
    survive every way of copying a tree."""
    stamp = target + ".srchash"
    if not (os.path.exists(target) and os.path.exists(stamp)):
        return True
    with open(stamp) as f:
        return f.read().strip() != _digest(deps)


def _stamp(target: str, deps) -> None:
    with open(target + ".srchash", "w") as f:
        f.write(_digest(deps))


def _all_deps():
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(INCLUDE, "linrec_b200.h"))
    deps.append(os.path.abspath(__file__))
    return deps


def _translation_units():
    """capi.cu (host logic, the small kernels) and the variants_*.cu files the kernel variants are spread
    over so that they compile side by side."""
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC)
                  if f.endswith(".cu") and (f == "capi.cu" or f.startswith("variants_")))


class _BuildLock:
    """One builder at a time per tree: the ranks of a multi-process job import the package together, and
    if the library is stale every one of them would compile into the same object files."""

    def __enter__(self):
        import fcntl
        os.makedirs(os.path.join(PKG, "_build"), exist_ok=True)
        self.f = open(os.path.join(PKG, "_build", ".lock"), "w")
        fcntl.flock(self.f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl
        fcntl.flock(self.f, fcntl.LOCK_UN)
        self.f.close()
        return False


def build_library(force: bool = False, verbose: bool = False, jobs: int | None = None) -> str:
    if not force and not _stale(LIB_PATH, _all_deps()):
        return LIB_PATH
    with _BuildLock():
        if not force and not _stale(LIB_PATH, _all_deps()):   # another process built it while this one waited
            return LIB_PATH
        return _build_library_locked(verbose, jobs)


def _build_library_locked(verbose: bool, jobs: int | None) -> str:
    nvcc = _nvcc()
    objdir = os.path.join(PKG, "_build", "obj")
    os.makedirs(objdir, exist_ok=True)
    units = _translation_units()
    jobs = jobs or max(1, min(len(units), os.cpu_count() or 1))
    objs, running, failed = [], [], []

    def reap(block_until_below: int):
        while len(running) > block_until_below:
            proc, src, log = running.pop(0)
            rc = proc.wait()
            log.close()
            if verbose or rc != 0:
                with open(log.name) as f:
                    sys.stderr.write(f.read())
            if rc != 0:
                failed.append(src)

    for src in units:
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", INCLUDE, "-c", "-o", obj, src]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        log = open(obj + ".log", "w")
        running.append((subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT), src, log))
        reap(jobs - 1)
    reap(0)
    if failed:
        raise RuntimeError("nvcc failed on " + ", ".join(os.path.basename(f) for f in failed))
    subprocess.run([nvcc, *ARCH_FLAGS, "-shared", "-Xcompiler", "-fPIC", "-o", LIB_PATH, *objs], check=True)
    for obj in objs:            # the objects are not reused (staleness is judged for the library as a whole)
        for f in (obj, obj + ".log"):
            if os.path.exists(f):
                os.remove(f)
    _stamp(LIB_PATH, _all_deps())
    return LIB_PATH


def build_executable(force: bool = False) -> str:
    """The standalone verify/bench harness (counterpart of linrec/impl/cuda/executable.cpp)."""
    lib = build_library(force=force)
    src = os.path.join(CSRC, "linrec_cli.cu")
    if not force and not _stale(EXE_PATH, _all_deps()):
        return EXE_PATH
    with _BuildLock():
        if not force and not _stale(EXE_PATH, _all_deps()):
            return EXE_PATH
        os.makedirs(os.path.dirname(EXE_PATH), exist_ok=True)
        cmd = [_nvcc(), *ARCH_FLAGS, "-O3", "-std=c++17", "-lineinfo", "-I", INCLUDE, "-o", EXE_PATH, src,
               lib, "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/.."]
        subprocess.run(cmd, check=True)
        _stamp(EXE_PATH, _all_deps())
    return EXE_PATH


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_library(force=force, verbose="--verbose" in sys.argv))
    if "--exe" in sys.argv:
        print(build_executable(force=force))
