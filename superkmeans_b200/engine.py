"""Thin object wrappers over the C ABI: `Engine` (one skm_handle) and the stateless operators."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import numpy as np

from . import _lib
from ._lib import Config, IterStats, check, lib


def default_config(hierarchical: bool = False, **overrides) -> Config:
    cfg = Config()
    lib.skm_default_config(C.byref(cfg), int(hierarchical))
    for k, v in overrides.items():
        if not hasattr(cfg, k):
            raise AttributeError(f"unknown config field {k}")
        setattr(cfg, k, v)
    return cfg


def _f32(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a) -> C.c_void_p:
    """Host numpy array or an object with a CUDA array interface / data_ptr() -> raw pointer."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return C.c_void_p(a.ctypes.data)
    if hasattr(a, "data_ptr"):
        return C.c_void_p(a.data_ptr())
    raise TypeError(f"cannot take a pointer of {type(a)}")


class Engine:
    """One trained-or-trainable model (skm_handle)."""

    def __init__(self, n_clusters: int, dimensionality: int, config: Optional[Config] = None, hierarchical: bool = False, device: int = -1):
        self.k, self.d, self.hierarchical = int(n_clusters), int(dimensionality), bool(hierarchical)
        self.config = config if config is not None else default_config(hierarchical)
        h = C.c_void_p()
        if n_clusters < 0 or dimensionality < 0:
            raise ValueError("Value must be positive")
        st = lib.skm_create(C.byref(self.config), self.k, self.d, int(hierarchical), device, C.byref(h))
        check(st, None)
        self._h = h
        self._keepalive = None
        self.n_trained = 0

    def close(self):
        # `lib` may already be gone when the interpreter is shutting down
        if getattr(self, "_h", None) and lib is not None:
            lib.skm_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    # -- rotation -----------------------------------------------------------------------------
    def set_rotation(self, m: np.ndarray):
        m = _f32(m)
        if m.shape != (self.d, self.d):
            raise ValueError("rotation matrix must be d x d")
        check(lib.skm_set_rotation(self._h, m), self._h)

    def get_rotation(self) -> np.ndarray:
        m = np.empty((self.d, self.d), dtype=np.float32)
        check(lib.skm_get_rotation(self._h, m), self._h)
        return m

    # -- sharding -----------------------------------------------------------------------------
    def set_shard(self, n_global: int, row_offset: int, allreduce):
        """`allreduce(ptr:int, count:int, dtype:int) -> None` sums a device buffer across ranks."""

        def _cb(_user, buf, count, dtype):
            try:
                allreduce(buf, count, dtype)
                return 0
            except Exception:  # the C side turns this into SKM_RUNTIME_ERROR
                import traceback

                traceback.print_exc()
                return 1

        self._keepalive = _lib.ALLREDUCE_FN(_cb)
        check(lib.skm_set_shard(self._h, n_global, row_offset, self._keepalive, None), self._h)

    def set_shard_comm(self, n_global: int, row_offset: int, comm: "Comm"):
        """Sharded training with the sums done by NCCL inside the library (see skm_set_shard_comm)."""
        self._keepalive = comm
        check(lib.skm_set_shard_comm(self._h, n_global, row_offset, comm._c), self._h)

    # -- the three calls of the reference API -----------------------------------------------------
    def train(self, data, n: Optional[int] = None, on_device: bool = False, queries=None, n_queries: int = 0) -> np.ndarray:
        """queries: host array of query vectors for the recall figure; with config.sample_queries pass n_queries alone."""
        if not on_device:
            data = _f32(data)
            n = data.shape[0]
        out = np.empty((self.k, self.d), dtype=np.float32)
        nq = int(n_queries) if queries is None else int(queries.shape[0])
        q = None if queries is None else _ptr(_f32(queries))
        check(lib.skm_train(self._h, _ptr(data), int(n), int(on_device), q, nq, out), self._h)
        self.n_trained = int(n)
        return out

    def assign(self, vectors, centroids, n: Optional[int] = None, on_device: bool = False, out=None):
        if not on_device:
            vectors, centroids = _f32(vectors), _f32(centroids)
            n = vectors.shape[0]
            out = np.empty(n, dtype=np.uint32)
        k = centroids.shape[0]
        check(lib.skm_assign(self._h, _ptr(vectors), _ptr(centroids), int(n), int(k), int(on_device), _ptr(out)), self._h)
        return out

    def assign_training_points(self, vectors, centroids, n: Optional[int] = None, on_device: bool = False, out=None):
        if not on_device:
            vectors, centroids = _f32(vectors), _f32(centroids)
            n = vectors.shape[0]
            out = np.empty(n, dtype=np.uint32)
        k = centroids.shape[0]
        check(lib.skm_assign_training_points(self._h, _ptr(vectors), _ptr(centroids), int(n), int(k), int(on_device), _ptr(out)), self._h)
        return out

    # -- state --------------------------------------------------------------------------------
    @property
    def is_trained(self) -> bool:
        return bool(lib.skm_is_trained(self._h))

    @property
    def n_clusters(self) -> int:
        return int(lib.skm_n_clusters(self._h))

    @property
    def n_mesoclusters(self) -> int:
        return int(lib.skm_n_mesoclusters(self._h))

    @property
    def last_prune_path(self) -> int:
        return int(lib.skm_last_prune_path(self._h))

    def prune_counters(self) -> dict:
        """Work of the pruned passes so far: rows through a dense chain, pair-steps of the list walk, overflowed rows."""
        out = (C.c_uint64 * 3)()
        check(lib.skm_get_prune_counters(self._h, out), self._h)
        return {"dense_rows": int(out[0]), "walk_pair_steps": int(out[1]), "overflow_rows": int(out[2])}

    def chain_counters(self) -> dict:
        """Work of the chain over gathered centroids so far: rows of its tiles, centroid columns of its units (see skm_get_chain_counters)."""
        out = (C.c_uint64 * 4)()
        check(lib.skm_get_chain_counters(self._h, out), self._h)
        return {"rows": int(out[0]), "columns": int(out[1]), "redone_rows": int(out[2]), "fallback_rows": int(out[3])}

    @property
    def last_objective_f64(self) -> float:
        return float(lib.skm_last_objective_f64(self._h))

    def use_dct_rotation(self):
        """Rotate with sign flips + DCT-II (what the reference does when built with FFTW, d a power of two >= 512)."""
        check(lib.skm_use_dct_rotation(self._h), self._h)

    def set_trace(self, enabled: bool = True):
        check(lib.skm_set_trace(self._h, int(enabled)), self._h)

    def trace(self) -> list:
        """Per-iteration snapshots as dicts (see skm_trace_get)."""
        out = []
        for i in range(int(lib.skm_trace_count(self._h))):
            ns, nc, pd = C.c_uint64(), C.c_uint64(), C.c_uint32()
            check(lib.skm_trace_get(self._h, i, C.byref(ns), C.byref(nc), C.byref(pd), None, None, None, None, None), self._h)
            cen = np.empty((nc.value, self.d), dtype=np.float32)
            asg = np.empty(ns.value, dtype=np.uint32)
            dst = np.empty(ns.value, dtype=np.float32)
            s0 = np.empty(nc.value, dtype=np.uint32)
            s1 = np.empty(nc.value, dtype=np.uint32)
            check(lib.skm_trace_get(self._h, i, None, None, None, cen.ctypes.data, asg.ctypes.data, dst.ctypes.data, s0.ctypes.data, s1.ctypes.data), self._h)
            out.append(dict(n_samples=ns.value, n_clusters=nc.value, partial_d_next=pd.value, centroids=cen, assign=asg, dist=dst, sizes_pre=s0, sizes_post=s1))
        return out

    PHASES = ("rotator", "norms_calc", "search/1st_blas", "search", "update_centroids", "consolidate", "shift", "train", "search/first_test", "search/walk", "search/dense",
              "alloc_free", "init_centroids", "allreduce")

    def phase_times(self) -> dict:
        """{phase name: (device milliseconds, calls)} accumulated since creation / reset."""
        out = {}
        for i, name in enumerate(self.PHASES):
            ms, calls = C.c_double(), C.c_uint64()
            check(lib.skm_get_phase_time(self._h, i, C.byref(ms), C.byref(calls)), self._h)
            out[name] = (ms.value, int(calls.value))
        return out

    def reset_phase_times(self):
        check(lib.skm_reset_phase_times(self._h), self._h)

    def stats(self, phase: int = 0) -> List[IterStats]:
        cnt = C.c_uint64()
        check(lib.skm_get_iteration_stats(self._h, phase, None, 0, C.byref(cnt)), self._h)
        buf = (IterStats * max(int(cnt.value), 1))()
        check(lib.skm_get_iteration_stats(self._h, phase, buf, cnt.value, C.byref(cnt)), self._h)
        return list(buf[: int(cnt.value)])

    @property
    def n_samples(self) -> int:
        """Rows covered by assignments() / distances(): the sampled rows of Train, or all rows after assign_training_points."""
        return int(lib.skm_get_n_samples(self._h))

    def assignments(self, n: Optional[int] = None) -> np.ndarray:
        n = self.n_samples if n is None else n
        out = np.empty(n, dtype=np.uint32)
        check(lib.skm_get_assignments(self._h, out, n), self._h)
        return out

    def distances(self, n: Optional[int] = None) -> np.ndarray:
        n = self.n_samples if n is None else n
        out = np.empty(n, dtype=np.float32)
        check(lib.skm_get_distances(self._h, out, n), self._h)
        return out

    def rotated_centroids(self) -> np.ndarray:
        out = np.empty((self.k, self.d), dtype=np.float32)
        check(lib.skm_get_rotated_centroids(self._h, out), self._h)
        return out


class Comm:
    """An NCCL communicator owned by the library (skm_comm): `Comm.unique_id()` on one rank, the 128 bytes passed to all
    ranks, then `Comm(id, rank, world, device)` on every rank (a collective)."""

    def __init__(self, unique_id: bytes, rank: int, world: int, device: int):
        if len(unique_id) != 128:
            raise ValueError("the unique id has 128 bytes")
        c = C.c_void_p()
        buf = (C.c_uint8 * 128).from_buffer_copy(unique_id)
        check(lib.skm_comm_create(buf, rank, world, device, C.byref(c)))
        self._c = c
        self.rank, self.world = rank, world

    @staticmethod
    def unique_id() -> bytes:
        buf = (C.c_uint8 * 128)()
        check(lib.skm_comm_unique_id(buf))
        return bytes(buf)

    def close(self):
        if getattr(self, "_c", None) and lib is not None:
            lib.skm_comm_destroy(self._c)
            self._c = None

    def __del__(self):
        self.close()


def set_workspace_cache(enabled: bool) -> None:
    """Keep large device buffers between calls (see skm_set_workspace_cache); off by default."""
    lib.skm_set_workspace_cache(int(enabled))


def release_cached_memory() -> None:
    lib.skm_release_cached_memory()


def cached_memory_bytes() -> int:
    return int(lib.skm_cached_memory_bytes())


def set_tensor_cores(enabled: bool) -> None:
    """Route the dense products to the tcgen05 kernels (default) or to the fp32 SIMT kernels."""
    lib.skm_set_tensor_cores(int(enabled))


def tensor_cores_enabled() -> bool:
    return bool(lib.skm_get_tensor_cores())


def set_prune_split(mode: int) -> None:
    """0 = automatic (by the sampled survival of the first test: 9 below 2.5 %, under 32 points per cluster or under 262 144 points, else 10), 1 = SIMT candidate lists, 2 = dense SIMT chain, 3 = dense
    tensor-core chain, 4 = tensor-core first test + list walk, 5 = as 4 with small lists, 6 = ordered points + exact gathered chain, 7 = ordered points +
    lists, 8 = as 7 with small lists, 9 = unordered lists with the dense chain for expensive points, 10 = ordered points + optimistic chain pass with
    exact redo, 11 = ordered points, route chosen per tile (see skm_set_prune_split)."""
    lib.skm_set_prune_split(int(mode))


def kernel_launches() -> int:
    return int(lib.skm_kernel_launches())


_ROLE_NAMES = ("mma_wait_rows", "mma_wait_operands", "mma_total", "rows_wait_accumulator", "rows_norms", "rows_total", "rows_wait_partner", "gather_wait_stage",
               "gather_wait_copies", "gather_total", "splitter_wait_tile", "producer_wait_stage")


def chain_role_cycles() -> dict:
    """SM cycles the roles of the chain over gathered centroids spent, per (unit, segment) step and averaged over the CTAs of
    all launches since the last call (skm_debug_role_cycles; the counters are cleared by the call)."""
    buf = (C.c_uint64 * 16)()
    check(lib.skm_debug_role_cycles(buf))
    steps = max(int(buf[12]), 1)
    out = {name: round(int(buf[i]) / steps, 1) for i, name in enumerate(_ROLE_NAMES)}
    out["steps"] = int(buf[12])
    out["ctas"] = int(buf[13])
    return out


def device_allocations() -> int:
    """cudaMalloc / cudaMallocHost calls made by the library in this process so far."""
    return int(lib.skm_device_allocations())


# ---- stateless operators (host arrays in, host arrays out) ------------------------------------

def rotate(m: np.ndarray, x: np.ndarray, device: int = -1) -> np.ndarray:
    m, x = _f32(m), _f32(x)
    out = np.empty_like(x)
    check(lib.skm_op_rotate(device, m, x, x.shape[0], x.shape[1], out))
    return out


def unrotate(m: np.ndarray, x: np.ndarray, device: int = -1) -> np.ndarray:
    m, x = _f32(m), _f32(x)
    out = np.empty_like(x)
    check(lib.skm_op_unrotate(device, m, x, x.shape[0], x.shape[1], out))
    return out


def find_nearest(x: np.ndarray, y: np.ndarray, device: int = -1):
    x, y = _f32(x), _f32(y)
    knn = np.empty(x.shape[0], dtype=np.uint32)
    dist = np.empty(x.shape[0], dtype=np.float32)
    check(lib.skm_op_find_nearest(device, x, y, x.shape[0], y.shape[0], x.shape[1], knn, dist))
    return knn, dist


def find_nearest_noalloc(x_dev_ptr: int, y_dev_ptr: int, n: int, k: int, d: int, out_knn_dev_ptr: int, out_dist_dev_ptr: int, device: int = -1, stream: int = 0) -> None:
    """Exact assignment on DEVICE buffers given as raw addresses, with no allocation made on the way.

    For callers whose device memory belongs to someone else's pool, or who cannot afford the device-wide
    stall of an allocation.  x [n][d] and y [k][d] are fp32, the outputs uint32 [n] and fp32 [n].  Limited to
    n <= 262144 and k <= 65536 per call; calls share one scratch area on the GPU and must not overlap.
    """
    check(lib.skm_op_find_nearest_noalloc(device, x_dev_ptr, y_dev_ptr, n, k, d, out_knn_dev_ptr, out_dist_dev_ptr, stream or None))


def find_nearest_pruned(x: np.ndarray, y: np.ndarray, prev_assign: np.ndarray, partial_d: int, epsilon0: float = 1.5, device: int = -1):
    x, y = _f32(x), _f32(y)
    knn = np.ascontiguousarray(prev_assign, dtype=np.uint32).copy()
    dist = np.empty(x.shape[0], dtype=np.float32)
    npc = np.zeros(x.shape[0], dtype=np.uint64)
    check(lib.skm_op_find_nearest_pruned(device, x, y, x.shape[0], y.shape[0], x.shape[1], epsilon0, partial_d, knn, dist, npc))
    return knn, dist, npc


def update_centroids(x: np.ndarray, assign: np.ndarray, k: int, dist: Optional[np.ndarray] = None, device: int = -1):
    x = _f32(x)
    assign = np.ascontiguousarray(assign, dtype=np.uint32)
    sums = np.empty((k, x.shape[1]), dtype=np.float32)
    counts = np.empty(k, dtype=np.uint32)
    wcss = C.c_double()
    dptr = None if dist is None else _ptr(_f32(dist))
    check(lib.skm_op_update_centroids(device, x, assign, dptr, x.shape[0], k, x.shape[1], sums, counts, C.byref(wcss)))
    return sums, counts, wcss.value


def pdxify(x: np.ndarray, device: int = -1) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    check(lib.skm_op_pdxify(device, x, x.shape[0], x.shape[1], out))
    return out


# ---- host-side decisions -------------------------------------------------------------------------

def dimension_split(d: int):
    h, v = C.c_uint64(), C.c_uint64()
    lib.skm_host_dimension_split(d, C.byref(h), C.byref(v))
    return int(h.value), int(v.value)


def ratios(d: int, epsilon0: float) -> np.ndarray:
    out = np.empty(d + 1, dtype=np.float32)
    lib.skm_host_ratios(d, epsilon0, out)
    return out


def forgy_indices(n_points: int, k: int, seed: int) -> np.ndarray:
    out = np.empty(min(k, n_points), dtype=np.uint64)
    lib.skm_host_forgy_indices(n_points, k, seed, out)
    return out


def split_clusters(sizes: np.ndarray, n_samples: int, seed: int, hierarchical: bool = False):
    sizes = np.ascontiguousarray(sizes, dtype=np.uint32).copy()
    k = sizes.shape[0]
    cap = 4 * k + 16
    ops = np.zeros((cap, 3), dtype=np.uint32)
    n_ops, n_split = C.c_uint64(), C.c_uint64()
    st = lib.skm_host_split_clusters(sizes, n_samples, k, seed, int(hierarchical), ops.ctypes.data, cap, C.byref(n_ops), C.byref(n_split))
    if st != 0:
        raise RuntimeError("cannot repopulate empty clusters")
    return sizes, ops[: n_ops.value], int(n_split.value)


def tune_partial_d(not_pruned_total: float, n_samples: int, n_y: int, partial_d: int, vertical_d: int, min_pct=0.03, max_pct=0.05, adjustment=0.2):
    avg = C.c_float()
    nd = lib.skm_host_tune_partial_d(not_pruned_total, n_samples, n_y, partial_d, vertical_d, min_pct, max_pct, adjustment, C.byref(avg))
    return int(nd), float(avg.value)


def arrange_fine_clusters(n_clusters: int, n_samples: int, meso_sizes: np.ndarray) -> np.ndarray:
    meso_sizes = np.ascontiguousarray(meso_sizes, dtype=np.uint32)
    out = np.empty(meso_sizes.shape[0], dtype=np.uint64)
    lib.skm_host_arrange_fine_clusters(n_clusters, meso_sizes.shape[0], n_samples, meso_sizes, out)
    return out


def pdx_offset(row: int, dim: int, n: int, d: int) -> int:
    return int(lib.skm_host_pdx_offset(row, dim, n, d))


def rotation_matrix(d: int, seed: int) -> np.ndarray:
    out = np.empty((d, d), dtype=np.float32)
    lib.skm_host_rotation_matrix(d, seed, out)
    return out


def dct_rotation_matrix(d: int, seed: int) -> np.ndarray:
    """Random sign flips + orthonormal DCT-II as a d x d matrix (the reference's FFTW rotation branch)."""
    out = np.empty((d, d), dtype=np.float32)
    lib.skm_host_dct_rotation_matrix(d, seed, out)
    return out
