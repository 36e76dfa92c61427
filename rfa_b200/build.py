"""Build the C-ABI shared library ``rfa_b200/csrc/librfa_b200.so`` with nvcc for sm_100a.

    python -m rfa_b200.build [--force] [--verbose]

Each ``csrc/*.cu`` is compiled to an object file (in parallel) and linked into
one shared library that exports the ``extern "C"`` entry points declared in
``include/rfa_b200.h``.  nvcc cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(CSRC, "librfa_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--extended-lambda", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the rfa_b200 library can only be built with the CUDA toolkit")
    return exe


def sources():
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "rfa_b200.h"))
    return hs


def stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def compile_one(src: str, verbose: bool) -> str:
    obj = src[:-3] + ".o"
    if stale(obj, [src] + headers()):
        cmd = [nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log = r.stdout + r.stderr
        with open(obj + ".log", "w") as f:
            f.write(" ".join(cmd) + "\n" + log)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {os.path.basename(src)}:\n{log}")
        if verbose:
            print(log)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = sources()
    if force:
        for s in srcs:
            if os.path.exists(s[:-3] + ".o"):
                os.remove(s[:-3] + ".o")
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: compile_one(s, verbose), srcs))
    if stale(LIB, objs):
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs, "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
