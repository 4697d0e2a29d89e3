"""Builds libskm_b200.so in-tree with nvcc for sm_100a.  Run as `python superkmeans_b200/build.py` (by path: importing the package needs the library).

Every source file is compiled to an object of its own (in parallel, and only when it or a header changed), then the
objects are linked into the shared library.  `-v` prints what ptxas reports (registers, spills, shared memory)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJDIR = os.path.join(HERE, "build")
SOURCES = ["kernels.cu", "kernels_pruned_dense.cu", "kernels_tc.cu", "kernels_tc_sparse.cu", "kernels_tc_rotate.cu", "kernels_walk.cu", "kernels_topk.cu", "kernels_replay.cu", "engine.cu",
           "comm_nccl.cu", "noalloc.cu", "abi.cu"]
HEADERS = ["common.cuh", "device_utils.cuh", "gemm_simt.cuh", "tc_ptx.cuh", "kernels_tc.cuh", "noalloc.h", "engine.h", "host_logic.h", "comm_nccl.h",
           os.path.join("..", "..", "include", "skm_b200.h")]
OUTPUT = os.path.join(HERE, "libskm_b200.so")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _sources():
    return [s for s in SOURCES if os.path.exists(os.path.join(CSRC, s))]


def _newest_header() -> float:
    paths = [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    return max(os.path.getmtime(p) for p in paths if os.path.exists(p))


def needs_build() -> bool:
    if not os.path.exists(OUTPUT):
        return True
    t = os.path.getmtime(OUTPUT)
    if _newest_header() > t:
        return True
    return any(os.path.getmtime(os.path.join(CSRC, s)) > t for s in _sources())


def _compile_one(nvcc: str, src: str, verbose: bool):
    obj = os.path.join(OBJDIR, os.path.splitext(src)[0] + ".o")
    cmd = [
        nvcc, "-std=c++17", "-O3", "-lineinfo", "-c",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-ccbin", "/usr/bin/g++",
        "-Xcompiler", "-fPIC,-fopenmp,-O3,-Wall,-Wno-unknown-pragmas",
    ]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, src), "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    return src, obj, res


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not verbose and not needs_build():
        return OUTPUT
    nvcc = _nvcc()
    os.makedirs(OBJDIR, exist_ok=True)
    hdr_t = _newest_header()
    todo, objs = [], []
    for src in _sources():
        obj = os.path.join(OBJDIR, os.path.splitext(src)[0] + ".o")
        objs.append(obj)
        stale = force or verbose or not os.path.exists(obj) or os.path.getmtime(obj) < max(hdr_t, os.path.getmtime(os.path.join(CSRC, src)))
        if stale:
            todo.append(src)
    failed = False
    with ThreadPoolExecutor(max_workers=max(1, min(len(todo), os.cpu_count() or 1))) as pool:
        for src, _obj, res in pool.map(lambda s: _compile_one(nvcc, s, verbose), todo):
            if res.returncode != 0:
                sys.stderr.write(f"--- {src}\n" + res.stdout + res.stderr)
                failed = True
            elif verbose or res.stderr.strip():
                sys.stderr.write(f"--- {src}\n" + res.stdout + res.stderr)
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-ccbin", "/usr/bin/g++", "-cudart", "static", "-Xcompiler", "-fPIC"] + objs + ["-o", OUTPUT, "-lgomp", "-ldl"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
        raise RuntimeError("link failed")
    return OUTPUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
