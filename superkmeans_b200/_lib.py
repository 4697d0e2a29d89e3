"""ctypes binding of libskm_b200.so (the C ABI declared in include/skm_b200.h).

There is no fallback: if the shared library is missing or cannot be loaded the import fails.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libskm_b200.so")

f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
u64p = np.ctypeslib.ndpointer(dtype=np.uint64, flags="C_CONTIGUOUS")

SKM_OK, SKM_INVALID_ARGUMENT, SKM_RUNTIME_ERROR, SKM_CUDA_ERROR, SKM_COMM_ERROR = range(5)


class Config(C.Structure):
    """skm_config: mirror of SuperKMeansConfig + the hierarchical iteration counts."""

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


class IterStats(C.Structure):
    """skm_iter_stats: mirror of SuperKMeansIterationStats."""

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


ALLREDUCE_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_int)

# name -> (restype, argtypes).  Every symbol include/skm_b200.h declares is listed here.
SIGNATURES = {
    "skm_default_config": (None, [C.POINTER(Config), C.c_int]),
    "skm_last_error": (C.c_char_p, [C.c_void_p]),
    "skm_create": (C.c_int, [C.POINTER(Config), C.c_uint64, C.c_uint64, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "skm_destroy": (None, [C.c_void_p]),
    "skm_set_rotation": (C.c_int, [C.c_void_p, f32p]),
    "skm_get_rotation": (C.c_int, [C.c_void_p, f32p]),
    "skm_train": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_int, C.c_void_p, C.c_uint64, f32p]),
    "skm_assign": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.c_void_p]),
    "skm_assign_training_points": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_int, C.c_void_p]),
    "skm_n_clusters": (C.c_uint64, [C.c_void_p]),
    "skm_is_trained": (C.c_int, [C.c_void_p]),
    "skm_sampling_fraction": (C.c_float, [C.c_void_p]),
    "skm_n_mesoclusters": (C.c_uint64, [C.c_void_p]),
    "skm_get_n_samples": (C.c_uint64, [C.c_void_p]),
    "skm_get_iteration_stats": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(IterStats), C.c_uint64, C.POINTER(C.c_uint64)]),
    "skm_get_assignments": (C.c_int, [C.c_void_p, u32p, C.c_uint64]),
    "skm_get_distances": (C.c_int, [C.c_void_p, f32p, C.c_uint64]),
    "skm_get_rotated_centroids": (C.c_int, [C.c_void_p, f32p]),
    "skm_last_objective_f64": (C.c_double, [C.c_void_p]),
    "skm_last_prune_path": (C.c_int, [C.c_void_p]),
    "skm_get_prune_counters": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "skm_get_chain_counters": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint64)]),
    "skm_set_trace": (C.c_int, [C.c_void_p, C.c_int]),
    "skm_trace_count": (C.c_uint64, [C.c_void_p]),
    "skm_trace_get": (C.c_int, [C.c_void_p, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64), C.POINTER(C.c_uint32), C.c_void_p, C.c_void_p, C.c_void_p,
                                C.c_void_p, C.c_void_p]),
    "skm_get_phase_time": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_uint64)]),
    "skm_reset_phase_times": (C.c_int, [C.c_void_p]),
    "skm_debug_wait_injection": (C.c_int, [C.c_uint64, C.c_uint32]),
    "skm_debug_role_cycles": (C.c_int, [C.POINTER(C.c_uint64)]),
    "skm_kernel_launches": (C.c_uint64, []),
    "skm_device_allocations": (C.c_uint64, []),
    "skm_set_prune_split": (None, [C.c_int]),
    "skm_get_prune_split": (C.c_int, []),
    "skm_set_tensor_cores": (None, [C.c_int]),
    "skm_get_tensor_cores": (C.c_int, []),
    "skm_set_shard": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, ALLREDUCE_FN, C.c_void_p]),
    "skm_comm_unique_id": (C.c_int, [C.c_void_p]),
    "skm_comm_create": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "skm_comm_wrap": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_void_p)]),
    "skm_comm_destroy": (None, [C.c_void_p]),
    "skm_set_shard_comm": (C.c_int, [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p]),
    "skm_set_workspace_cache": (None, [C.c_int]),
    "skm_get_workspace_cache": (C.c_int, []),
    "skm_release_cached_memory": (None, []),
    "skm_cached_memory_bytes": (C.c_uint64, []),
    "skm_op_rotate": (C.c_int, [C.c_int, f32p, f32p, C.c_uint64, C.c_uint64, f32p]),
    "skm_op_unrotate": (C.c_int, [C.c_int, f32p, f32p, C.c_uint64, C.c_uint64, f32p]),
    "skm_op_find_nearest": (C.c_int, [C.c_int, f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, u32p, f32p]),
    "skm_op_find_nearest_noalloc": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "skm_op_find_nearest_pruned": (C.c_int, [C.c_int, f32p, f32p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, C.c_uint32, u32p, f32p, u64p]),
    "skm_op_update_centroids": (C.c_int, [C.c_int, f32p, u32p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, f32p, u32p, C.POINTER(C.c_double)]),
    "skm_op_pdxify": (C.c_int, [C.c_int, f32p, C.c_uint64, C.c_uint64, f32p]),
    "skm_host_dimension_split": (None, [C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "skm_host_ratios": (None, [C.c_uint64, C.c_float, f32p]),
    "skm_host_forgy_indices": (None, [C.c_uint64, C.c_uint64, C.c_uint32, u64p]),
    "skm_host_split_clusters": (C.c_int, [u32p, C.c_uint64, C.c_uint64, C.c_uint32, C.c_int, C.c_void_p, C.c_uint64, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "skm_host_tune_partial_d": (C.c_uint32, [C.c_double, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_float, C.POINTER(C.c_float)]),
    "skm_host_arrange_fine_clusters": (None, [C.c_uint64, C.c_uint64, C.c_uint64, u32p, u64p]),
    "skm_host_pdx_offset": (C.c_uint64, [C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64]),
    "skm_host_rotation_matrix": (None, [C.c_uint64, C.c_uint32, f32p]),
    "skm_host_dct_rotation_matrix": (None, [C.c_uint64, C.c_uint32, f32p]),
    "skm_use_dct_rotation": (C.c_int, [C.c_void_p]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python superkmeans_b200/build.py` (needs nvcc). "
            "This package has no CPU implementation."
        )
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


lib = _load()


def check(status: int, handle=None):
    """Raises the exception class the reference would raise for this status."""
    if status == SKM_OK:
        return
    msg = lib.skm_last_error(handle)
    msg = msg.decode() if msg else "unknown error"
    if status == SKM_INVALID_ARGUMENT:
        raise ValueError(msg)
    raise RuntimeError(msg)
