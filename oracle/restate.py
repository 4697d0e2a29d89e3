"""TEST INFRASTRUCTURE ONLY: ctypes access to the independent CPU restatement (oracle/libskm_oracle.so,
built from oracle/skm_oracle.cpp by `make -C oracle oracle`)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Callable, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libskm_oracle.so")

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
u64p = np.ctypeslib.ndpointer(dtype=np.uint64, flags="C_CONTIGUOUS")
REDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_int)


class Stats(C.Structure):
    _fields_ = [("iteration", C.c_uint64), ("objective", C.c_float), ("shift", C.c_float), ("split", C.c_uint64), ("not_pruned_pct", C.c_float),
                ("partial_d", C.c_uint32), ("is_gemm_only", C.c_int32)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            subprocess.run(["make", "-C", _HERE, "oracle"], check=True, capture_output=True)
        L = C.CDLL(LIB_PATH)
        L.orc_dimension_split.argtypes = [C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
        L.orc_ratios.argtypes = [C.c_uint64, C.c_float, f32p]
        L.orc_rotate.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, f32p]
        L.orc_unrotate.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, f32p]
        L.orc_row_norms.argtypes = [f32p, C.c_uint64, C.c_uint64, C.c_uint64, f32p]
        L.orc_horizontal.argtypes = [f32p, f32p, C.c_uint64]
        L.orc_horizontal.restype = C.c_float
        L.orc_pdxify.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64]
        L.orc_find_nearest.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, f32p, f32p, u32p, f32p]
        L.orc_find_nearest_pruned.argtypes = [f32p, f32p, f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, f32p, f32p, f32p, C.c_uint32, u32p, f32p, u64p]
        L.orc_update.argtypes = [f32p, u32p, C.c_uint64, C.c_uint64, C.c_uint64, f32p, u32p]
        L.orc_mean_and_split.argtypes = [f32p, u32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint32]
        L.orc_mean_and_split.restype = C.c_uint64
        L.orc_tune_partial_d.argtypes = [u64p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_float, C.POINTER(C.c_float)]
        L.orc_tune_partial_d.restype = C.c_uint32
        L.orc_train_flat.argtypes = [f32p, C.c_uint64, C.c_uint64, C.c_uint64, f32p, C.c_uint32, C.c_uint32, C.c_int, C.c_float, C.c_uint64, C.c_uint64, REDUCE_FN,
                                     C.c_void_p, f32p, f32p, u32p, C.POINTER(Stats)]
        _lib = L
    return _lib


def dimension_split(d):
    h, v = C.c_uint64(), C.c_uint64()
    lib().orc_dimension_split(d, C.byref(h), C.byref(v))
    return int(h.value), int(v.value)


def ratios(d, eps0):
    out = np.empty(d + 1, dtype=np.float32)
    lib().orc_ratios(d, eps0, out)
    return out


def rotate(m, x):
    out = np.empty_like(x)
    lib().orc_rotate(m, x, x.shape[0], x.shape[1], out)
    return out


def unrotate(m, x):
    out = np.empty_like(x)
    lib().orc_unrotate(m, x, x.shape[0], x.shape[1], out)
    return out


def row_norms(x, upto=None):
    out = np.empty(x.shape[0], dtype=np.float32)
    lib().orc_row_norms(x, x.shape[0], x.shape[1], x.shape[1] if upto is None else upto, out)
    return out


def horizontal(a, b):
    return float(lib().orc_horizontal(a, b, a.shape[0]))


def pdxify(x):
    out = np.empty_like(x)
    lib().orc_pdxify(x, out, x.shape[0], x.shape[1])
    return out


def find_nearest(x, y):
    knn = np.zeros(x.shape[0], dtype=np.uint32)
    dist = np.empty(x.shape[0], dtype=np.float32)
    lib().orc_find_nearest(x, y, x.shape[0], y.shape[0], x.shape[1], row_norms(x), row_norms(y), knn, dist)
    return knn, dist


def find_nearest_pruned(x, y, prev_assign, partial_d, epsilon0=1.5):
    d = x.shape[1]
    _, vd = dimension_split(d)
    knn = np.ascontiguousarray(prev_assign, dtype=np.uint32).copy()
    dist = np.zeros(x.shape[0], dtype=np.float32)
    npc = np.zeros(x.shape[0], dtype=np.uint64)
    aux = np.ascontiguousarray(y[:, :vd])
    lib().orc_find_nearest_pruned(x, y, pdxify(y), aux, x.shape[0], y.shape[0], d, row_norms(x, partial_d), row_norms(y, partial_d), ratios(d, epsilon0), partial_d,
                                  knn, dist, npc)
    return knn, dist, npc


def update(x, assign, k):
    sums = np.empty((k, x.shape[1]), dtype=np.float32)
    sizes = np.empty(k, dtype=np.uint32)
    lib().orc_update(x, np.ascontiguousarray(assign, dtype=np.uint32), x.shape[0], k, x.shape[1], sums, sizes)
    return sums, sizes


def mean_and_split(sums, sizes, n_samples, seed):
    c = np.ascontiguousarray(sums, dtype=np.float32).copy()
    s = np.ascontiguousarray(sizes, dtype=np.uint32).copy()
    n_split = lib().orc_mean_and_split(c, s, n_samples, c.shape[0], c.shape[1], seed)
    return c, s, int(n_split)


def train_flat(data, k, m, iters=10, seed=42, use_blas_only=False, epsilon0=1.5, rows=None, reduce: Optional[Callable] = None):
    """Returns (centroids, rotated_centroids, assignments of the row range, list of Stats)."""
    n, d = data.shape
    lo, hi = (0, n) if rows is None else rows
    cent = np.empty((k, d), dtype=np.float32)
    rcent = np.empty((k, d), dtype=np.float32)
    assign = np.empty(hi - lo, dtype=np.uint32)
    stats = (Stats * iters)()

    def _cb(_user, buf, count, dtype):
        try:
            reduce(buf, count, dtype)
            return 0
        except Exception:
            import traceback

            traceback.print_exc()
            return 1

    cb = REDUCE_FN(_cb) if reduce is not None else C.cast(None, REDUCE_FN)
    st = lib().orc_train_flat(data, n, d, k, m, iters, seed, int(use_blas_only), epsilon0, lo, hi, cb, None, cent, rcent, assign, stats)
    if st != 0:
        raise RuntimeError(f"orc_train_flat failed with status {st}")
    return cent, rcent, assign, list(stats)
