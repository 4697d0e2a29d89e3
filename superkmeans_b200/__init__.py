"""B200-native k-means engine behind the SuperKMeans Python surface.

`SuperKMeans` has the constructor, methods, properties, validation and exception behaviour of
`superkmeans.SuperKMeans` (python/superkmeans/__init__.py in the SuperKMeans repository); all
computation happens in libskm_b200.so (hand-written CUDA for sm_100a).
"""
from __future__ import annotations

from typing import List, Optional

import numpy as np

from . import engine as _engine
from ._lib import IterStats as SuperKMeansIterationStats
from .engine import Engine, default_config

__version__ = "0.1.0"


class HierarchicalSuperKMeansIterationStats:
    """Counterpart of the reference's HierarchicalSuperKMeansIterationStats (three lists)."""

    def __init__(self, meso, fine, refine):
        self.mesoclustering_iteration_stats = meso
        self.fineclustering_iteration_stats = fine
        self.refinement_iteration_stats = refine


class SuperKMeans:
    """Same parameters and attributes as the reference's `superkmeans.SuperKMeans`
    (python/superkmeans/__init__.py:21-136); `device` is the only addition."""

    def __init__(
        self,
        n_clusters: int,
        dimensionality: int,
        hierarchical: Optional[bool] = None,
        iters: int = 10,
        iters_mesoclustering: int = 3,
        iters_fineclustering: int = 5,
        iters_refinement: int = 0,
        sampling_fraction: Optional[float] = None,
        max_points_per_cluster: int = 256,
        n_threads: int = 0,
        seed: int = 42,
        use_blas_only: bool = False,
        tol: float = 1e-4,
        recall_tol: float = 0.005,
        early_termination: bool = True,
        sample_queries: bool = False,
        objective_k: int = 100,
        verbose: bool = False,
        angular: bool = False,
        device: int = -1,
    ):
        if n_clusters <= 0:
            raise ValueError("n_clusters must be positive")
        if dimensionality <= 0:
            raise ValueError("dimensionality must be positive")
        if sampling_fraction is not None and not 0.0 < sampling_fraction <= 1.0:
            raise ValueError("sampling_fraction must be in (0.0, 1.0]")
        self._n_clusters = n_clusters
        self._dimensionality = dimensionality
        self._hierarchical_param = hierarchical
        self._hierarchical = None
        self._obj: Optional[Engine] = None
        self._device = device
        self._config_params = dict(
            iters=iters, iters_mesoclustering=iters_mesoclustering, iters_fineclustering=iters_fineclustering,
            iters_refinement=iters_refinement, sampling_fraction=sampling_fraction,
            max_points_per_cluster=max_points_per_cluster, n_threads=n_threads, seed=seed,
            use_blas_only=use_blas_only, tol=tol, recall_tol=recall_tol, early_termination=early_termination,
            sample_queries=sample_queries, objective_k=objective_k, verbose=verbose, angular=angular,
        )

    @staticmethod
    def validate_numpy_array(data, name: str, expected_dimensionality: Optional[int] = None) -> np.ndarray:
        if not isinstance(data, np.ndarray):
            data = np.asarray(data, dtype=np.float32)
        if data.dtype != np.float32:
            raise ValueError(f"{name} must have dtype float32, got {data.dtype}")
        if data.ndim != 2:
            raise ValueError(f"{name} must be 2-dimensional, got {data.ndim}")
        if expected_dimensionality is not None and data.shape[1] != expected_dimensionality:
            raise ValueError(f"{name} must have dimensionality {expected_dimensionality}, got {data.shape[1]}")
        if not data.flags["C_CONTIGUOUS"]:
            data = np.ascontiguousarray(data)
        return data

    def _make(self) -> Engine:
        p = self._config_params
        cfg = default_config(bool(self._hierarchical))
        if self._hierarchical:
            cfg.iters_mesoclustering = p["iters_mesoclustering"]
            cfg.iters_fineclustering = p["iters_fineclustering"]
            cfg.iters_refinement = p["iters_refinement"]
        else:
            cfg.iters = p["iters"]
        if p["sampling_fraction"] is not None:
            cfg.sampling_fraction = p["sampling_fraction"]
        for name in ("max_points_per_cluster", "n_threads", "seed", "tol", "recall_tol", "objective_k"):
            setattr(cfg, name, p[name])
        for name in ("use_blas_only", "early_termination", "sample_queries", "verbose", "angular"):
            setattr(cfg, name, int(bool(p[name])))
        return Engine(self._n_clusters, self._dimensionality, cfg, bool(self._hierarchical), self._device)

    def train(self, data, queries=None) -> np.ndarray:
        data = self.validate_numpy_array(data, "data", self._dimensionality)
        n_samples = data.shape[0]
        if self._hierarchical_param is None:
            self._hierarchical = n_samples > 100_000
        else:
            self._hierarchical = self._hierarchical_param
        if self._obj is None:
            self._obj = self._make()
        if queries is not None:
            queries = self.validate_numpy_array(queries, "queries", self._dimensionality)
        return self._obj.train(data, queries=queries)

    def _check_pair(self, vectors, centroids):
        vectors = self.validate_numpy_array(vectors, "vectors")
        centroids = self.validate_numpy_array(centroids, "centroids")
        if vectors.shape[1] != centroids.shape[1]:
            raise ValueError(
                f"vectors and centroids must have same dimensionality, got {vectors.shape[1]} and {centroids.shape[1]}"
            )
        return vectors, centroids

    def _need_obj(self) -> Engine:
        if self._obj is None:
            # The reference dereferences a null object here; an AttributeError is the Python analogue.
            raise AttributeError("'NoneType' object has no attribute 'assign'")
        return self._obj

    def assign(self, vectors, centroids) -> np.ndarray:
        vectors, centroids = self._check_pair(vectors, centroids)
        return self._need_obj().assign(vectors, centroids)

    add = assign

    def assign_training_points(self, vectors, centroids) -> np.ndarray:
        vectors, centroids = self._check_pair(vectors, centroids)
        return self._need_obj().assign_training_points(vectors, centroids)

    @property
    def n_clusters_(self) -> int:
        return self._n_clusters if self._obj is None else self._obj.n_clusters

    @property
    def is_trained_(self) -> bool:
        return False if self._obj is None else self._obj.is_trained

    @property
    def hierarchical_(self) -> Optional[bool]:
        return self._hierarchical

    @property
    def iteration_stats(self) -> List[SuperKMeansIterationStats]:
        return [] if self._obj is None else self._obj.stats(0)

    @property
    def hierarchical_iteration_stats(self):
        if self._obj is None or not self._hierarchical:
            return None
        return HierarchicalSuperKMeansIterationStats(self._obj.stats(1), self._obj.stats(2), self._obj.stats(3))

    def __repr__(self) -> str:
        h = f", hierarchical={self._hierarchical}" if self._hierarchical is not None else ""
        return f"SuperKMeans(n_clusters={self._n_clusters}, dimensionality={self._dimensionality}, trained={self.is_trained_}{h})"


__all__ = [
    "__version__",
    "SuperKMeans",
    "SuperKMeansIterationStats",
    "HierarchicalSuperKMeansIterationStats",
    "Engine",
    "default_config",
]
