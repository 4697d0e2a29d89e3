"""TEST INFRASTRUCTURE ONLY: ctypes access to the real reference (oracle/_ref/libskm_ref_*.so).

The shared object is the unmodified SuperKMeans reference compiled by oracle/Makefile.  Only tests/,
the smoke check and bench.py's CPU-baseline legs may import this module; the shipped package never
does.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import List, Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
u64p = np.ctypeslib.ndpointer(dtype=np.uint64, flags="C_CONTIGUOUS")


class RefConfig(C.Structure):
    """Mirror of SuperKMeansConfig + HierarchicalSuperKMeansConfig (superkmeans.h:23-55,
    hierarchical_superkmeans.h:11-17)."""

    _fields_ = [
        ("iters", C.c_uint32),
        ("sampling_fraction", C.c_float),
        ("max_points_per_cluster", C.c_uint32),
        ("n_threads", C.c_uint32),
        ("seed", C.c_uint32),
        ("use_blas_only", C.c_int32),
        ("tol", C.c_float),
        ("recall_tol", C.c_float),
        ("early_termination", C.c_int32),
        ("sample_queries", C.c_int32),
        ("objective_k", C.c_uint64),
        ("ann_explore_fraction", C.c_float),
        ("min_not_pruned_pct", C.c_float),
        ("max_not_pruned_pct", C.c_float),
        ("adjustment_factor_for_partial_d", C.c_float),
        ("unrotate_centroids", C.c_int32),
        ("verbose", C.c_int32),
        ("angular", C.c_int32),
        ("suppress_warnings", C.c_int32),
        ("data_already_rotated", C.c_int32),
        ("iters_mesoclustering", C.c_uint32),
        ("iters_fineclustering", C.c_uint32),
        ("iters_refinement", C.c_uint32),
    ]


class RefIterStats(C.Structure):
    _fields_ = [
        ("iteration", C.c_uint64),
        ("objective", C.c_float),
        ("shift", C.c_float),
        ("split", C.c_uint64),
        ("recall", C.c_float),
        ("not_pruned_pct", C.c_float),
        ("partial_d", C.c_uint32),
        ("is_gemm_only", C.c_int32),
    ]


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def library_path() -> Optional[str]:
    flags = _cpu_flags()
    need512 = {"avx512f", "avx512bw", "avx512dq", "avx512vl", "avx512cd"}
    names = []
    if need512 <= flags:
        names.append("libskm_ref_avx512.so")
    names.append("libskm_ref_avx2.so")
    for n in names:
        p = os.path.join(_HERE, "_ref", n)
        if os.path.exists(p):
            return p
    return None


_lib = None


def available() -> bool:
    return library_path() is not None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    p = library_path()
    if p is None:
        raise RuntimeError("oracle/_ref is not built (run `make -C oracle ref` where the reference sources exist)")
    L = C.CDLL(p)
    L.ref_default_config.argtypes = [C.POINTER(RefConfig), C.c_int]
    L.ref_default_config.restype = None
    L.ref_last_error.restype = C.c_char_p
    L.ref_create.argtypes = [C.c_uint64, C.c_uint64, C.POINTER(RefConfig), C.c_int, C.c_int, C.POINTER(C.c_void_p)]
    L.ref_destroy.argtypes = [C.c_void_p]
    L.ref_destroy.restype = None
    L.ref_train.argtypes = [C.c_void_p, f32p, C.c_uint64, C.c_void_p, C.c_uint64, f32p]
    L.ref_assign.argtypes = [C.c_void_p, f32p, f32p, C.c_uint64, C.c_uint64, u32p]
    L.ref_assign_training_points.argtypes = [C.c_void_p, f32p, f32p, C.c_uint64, C.c_uint64, u32p]
    L.ref_is_trained.argtypes = [C.c_void_p]
    L.ref_rotation_matrix.argtypes = [C.c_void_p, f32p]
    L.ref_rotation_matrix.restype = None
    L.ref_ratios.argtypes = [C.c_void_p, f32p]
    L.ref_ratios.restype = None
    L.ref_get_assignments.argtypes = [C.c_void_p, u32p, C.c_uint64]
    L.ref_get_assignments.restype = None
    L.ref_get_distances.argtypes = [C.c_void_p, f32p, C.c_uint64]
    L.ref_get_distances.restype = None
    L.ref_get_rotated_centroids.argtypes = [C.c_void_p, f32p]
    L.ref_get_rotated_centroids.restype = None
    L.ref_get_final_assignments.argtypes = [C.c_void_p, u32p, C.c_uint64]
    L.ref_get_final_assignments.restype = None
    L.ref_n_mesoclusters.argtypes = [C.c_void_p]
    L.ref_n_mesoclusters.restype = C.c_uint64
    L.ref_get_stats.argtypes = [C.c_void_p, C.c_int, C.POINTER(RefIterStats), C.c_uint64]
    L.ref_get_stats.restype = C.c_uint64
    L.ref_trace_count.argtypes = [C.c_void_p]
    L.ref_trace_count.restype = C.c_uint64
    L.ref_trace_get.argtypes = [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64),
                                C.POINTER(C.c_uint32), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    L.ref_trace_get.restype = None
    L.ref_dimension_split.argtypes = [C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]
    L.ref_dimension_split.restype = None
    L.ref_pdxify.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64]
    L.ref_pdxify.restype = None
    L.ref_horizontal.argtypes = [f32p, f32p, C.c_uint64]
    L.ref_horizontal.restype = C.c_float
    L.ref_find_nearest.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_int, u32p, f32p]
    L.ref_find_nearest.restype = None
    L.ref_find_nearest_pruned.argtypes = [f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float,
                                          C.c_uint32, C.c_int, u32p, f32p, u64p]
    L.ref_find_nearest_pruned.restype = None
    L.ref_make_blobs.argtypes = [C.c_uint64, C.c_uint64, C.c_uint64, C.c_int, C.c_float, C.c_float, C.c_uint32, f32p]
    L.ref_make_blobs.restype = None
    L.ref_set_blas_threads.argtypes = [C.c_int]
    L.ref_set_blas_threads.restype = None
    L.ref_get_blas_threads.restype = C.c_int
    L.ref_get_omp_threads.restype = C.c_int
    _lib = L
    return L


def default_config(hierarchical: bool = False, **kw) -> RefConfig:
    c = RefConfig()
    lib().ref_default_config(C.byref(c), int(hierarchical))
    for k, v in kw.items():
        if not hasattr(c, k):
            raise AttributeError(k)
        setattr(c, k, v)
    return c


class RefError(Exception):
    def __init__(self, status: int, msg: str):
        super().__init__(msg)
        self.status = status


def _check(st: int):
    if st != 0:
        msg = lib().ref_last_error().decode()
        if st == 1:
            raise ValueError(msg)
        if st == 2:
            raise RuntimeError(msg)
        raise RefError(st, msg)


@dataclass
class Snapshot:
    n_samples: int
    n_clusters: int
    partial_d_next: int
    centroids: np.ndarray
    assign: np.ndarray
    dist: np.ndarray
    sizes_pre: np.ndarray
    sizes_post: np.ndarray


class RefKMeans:
    """The reference's SuperKMeans / HierarchicalSuperKMeans object behind ctypes."""

    def __init__(self, k: int, d: int, cfg: Optional[RefConfig] = None, hierarchical: bool = False, trace: bool = False):
        self.k, self.d, self.hierarchical = k, d, hierarchical
        self.cfg = cfg if cfg is not None else default_config(hierarchical)
        h = C.c_void_p()
        _check(lib().ref_create(k, d, C.byref(self.cfg), int(hierarchical), int(trace), C.byref(h)))
        self._h = h
        self.n = 0

    def __del__(self):
        if getattr(self, "_h", None):
            lib().ref_destroy(self._h)
            self._h = None

    def train(self, data: np.ndarray, queries: Optional[np.ndarray] = None, n_queries: int = 0) -> np.ndarray:
        data = np.ascontiguousarray(data, dtype=np.float32)
        out = np.empty((self.k, self.d), dtype=np.float32)
        q, nq = None, int(n_queries)
        if queries is not None:
            queries = np.ascontiguousarray(queries, dtype=np.float32)
            q, nq = queries.ctypes.data_as(C.c_void_p), queries.shape[0]
        _check(lib().ref_train(self._h, data, data.shape[0], q, nq, out))
        self.n = data.shape[0]
        return out

    def assign(self, vectors: np.ndarray, centroids: np.ndarray) -> np.ndarray:
        out = np.empty(vectors.shape[0], dtype=np.uint32)
        _check(lib().ref_assign(self._h, vectors, centroids, vectors.shape[0], centroids.shape[0], out))
        return out

    def assign_training_points(self, vectors: np.ndarray, centroids: np.ndarray) -> np.ndarray:
        out = np.empty(vectors.shape[0], dtype=np.uint32)
        _check(lib().ref_assign_training_points(self._h, vectors, centroids, vectors.shape[0], centroids.shape[0], out))
        return out

    @property
    def is_trained(self) -> bool:
        return bool(lib().ref_is_trained(self._h))

    def rotation_matrix(self) -> np.ndarray:
        m = np.empty((self.d, self.d), dtype=np.float32)
        lib().ref_rotation_matrix(self._h, m)
        return m

    def ratios(self) -> np.ndarray:
        r = np.empty(self.d + 1, dtype=np.float32)
        lib().ref_ratios(self._h, r)
        return r

    def assignments(self, n: Optional[int] = None) -> np.ndarray:
        n = self.n if n is None else n
        a = np.empty(n, dtype=np.uint32)
        lib().ref_get_assignments(self._h, a, n)
        return a

    def distances(self, n: Optional[int] = None) -> np.ndarray:
        n = self.n if n is None else n
        a = np.empty(n, dtype=np.float32)
        lib().ref_get_distances(self._h, a, n)
        return a

    def rotated_centroids(self) -> np.ndarray:
        c = np.empty((self.k, self.d), dtype=np.float32)
        lib().ref_get_rotated_centroids(self._h, c)
        return c

    def final_assignments(self) -> np.ndarray:
        a = np.empty(self.n, dtype=np.uint32)
        lib().ref_get_final_assignments(self._h, a, self.n)
        return a

    def n_mesoclusters(self) -> int:
        return int(lib().ref_n_mesoclusters(self._h))

    def stats(self, phase: int = 0) -> List[dict]:
        cnt = lib().ref_get_stats(self._h, phase, None, 0)
        buf = (RefIterStats * max(int(cnt), 1))()
        lib().ref_get_stats(self._h, phase, buf, cnt)
        return [
            dict(iteration=int(s.iteration), objective=float(s.objective), shift=float(s.shift), split=int(s.split),
                 recall=float(s.recall), not_pruned_pct=float(s.not_pruned_pct), partial_d=int(s.partial_d),
                 is_gemm_only=bool(s.is_gemm_only))
            for s in buf[: int(cnt)]
        ]

    def trace(self) -> List[Snapshot]:
        out = []
        for i in range(int(lib().ref_trace_count(self._h))):
            ns, nc, pd = C.c_uint64(), C.c_uint64(), C.c_uint32()
            lib().ref_trace_get(self._h, i, C.byref(ns), C.byref(nc), C.byref(pd), None, None, None, None, None)
            cen = np.empty((nc.value, self.d), dtype=np.float32)
            asg = np.empty(ns.value, dtype=np.uint32)
            dst = np.empty(ns.value, dtype=np.float32)
            s0 = np.empty(nc.value, dtype=np.uint32)
            s1 = np.empty(nc.value, dtype=np.uint32)
            lib().ref_trace_get(self._h, i, None, None, None, cen.ctypes.data, asg.ctypes.data, dst.ctypes.data,
                                s0.ctypes.data, s1.ctypes.data)
            out.append(Snapshot(ns.value, nc.value, pd.value, cen, asg, dst, s0, s1))
        return out


def dimension_split(d: int):
    h, v = C.c_uint64(), C.c_uint64()
    lib().ref_dimension_split(d, C.byref(h), C.byref(v))
    return int(h.value), int(v.value)


def pdxify(x: np.ndarray) -> np.ndarray:
    out = np.empty_like(x)
    lib().ref_pdxify(x, out, x.shape[0], x.shape[1])
    return out


def horizontal(a: np.ndarray, b: np.ndarray) -> float:
    return float(lib().ref_horizontal(a, b, a.shape[0]))


def find_nearest(x: np.ndarray, y: np.ndarray, n_threads: int = 0):
    knn = np.empty(x.shape[0], dtype=np.uint32)
    dist = np.empty(x.shape[0], dtype=np.float32)
    lib().ref_find_nearest(x, y, x.shape[0], y.shape[0], x.shape[1], n_threads, knn, dist)
    return knn, dist


def find_nearest_pruned(x: np.ndarray, y: np.ndarray, prev_assign: np.ndarray, partial_d: int, epsilon0: float = 1.5,
                        n_threads: int = 0):
    knn = np.ascontiguousarray(prev_assign, dtype=np.uint32).copy()
    dist = np.zeros(x.shape[0], dtype=np.float32)
    npc = np.zeros(x.shape[0], dtype=np.uint64)
    lib().ref_find_nearest_pruned(x, y, x.shape[0], y.shape[0], x.shape[1], epsilon0, partial_d, n_threads, knn, dist, npc)
    return knn, dist, npc


def make_blobs(n: int, d: int, centers: int, normalize: bool, std: float, spread: float, seed: int) -> np.ndarray:
    out = np.empty((n, d), dtype=np.float32)
    lib().ref_make_blobs(n, d, centers, int(normalize), std, spread, seed, out)
    return out
