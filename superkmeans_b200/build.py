"""Builds libskm_b200.so in-tree with nvcc for sm_100a.  Run as `python superkmeans_b200/build.py` (by path: importing the package needs the library)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
SOURCES = ["kernels.cu", "kernels_pruned_dense.cu", "kernels_tc.cu", "kernels_walk.cu", "kernels_topk.cu", "engine.cu", "noalloc.cu", "abi.cu"]
HEADERS = ["common.cuh", "device_utils.cuh", "gemm_simt.cuh", "kernels_tc.cuh", "noalloc.h", "engine.h", "host_logic.h", os.path.join("..", "..", "include", "skm_b200.h")]
OUTPUT = os.path.join(HERE, "libskm_b200.so")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def needs_build() -> bool:
    if not os.path.exists(OUTPUT):
        return True
    t = os.path.getmtime(OUTPUT)
    deps = [os.path.join(CSRC, s) for s in SOURCES + HEADERS] + [os.path.abspath(__file__)]
    return any(os.path.exists(p) and os.path.getmtime(p) > t for p in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return OUTPUT
    cmd = [
        _nvcc(), "-std=c++17", "-O3", "-lineinfo", "-shared",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-ccbin", "/usr/bin/g++",
        "-Xcompiler", "-fPIC,-fopenmp,-O3,-Wall,-Wno-unknown-pragmas",
        "-cudart", "static",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, s) for s in SOURCES]
    cmd += ["-o", OUTPUT, "-lgomp"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("nvcc failed")
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
