"""Acceptance tests of the Python surface: what a user of `superkmeans.SuperKMeans` relies on must hold for
`superkmeans_b200.SuperKMeans`.  Each test names the reference test whose behaviour it re-checks
(python/tests/test_superkmeans.py in the SuperKMeans repository); data and assertions are written for this package."""
import numpy as np
import pytest

import superkmeans_b200 as skm
from superkmeans_b200 import HierarchicalSuperKMeansIterationStats, SuperKMeans, SuperKMeansIterationStats

pytestmark = pytest.mark.gpu


def _gauss(n, d, seed=0):
    return np.random.default_rng(seed).standard_normal((n, d), dtype=np.float32)


# ---- construction (test_init_default, test_init_with_params, test_init_invalid_params, test_repr)
def test_constructor_keeps_parameters_and_starts_untrained():
    km = SuperKMeans(n_clusters=10, dimensionality=50)
    assert km.n_clusters_ == 10 and not km.is_trained_
    km = SuperKMeans(n_clusters=20, dimensionality=64, iters=15, sampling_fraction=0.5, verbose=True, seed=123)
    assert km.n_clusters_ == 20 and not km.is_trained_
    text = repr(km)
    assert "SuperKMeans" in text and "n_clusters=20" in text and "dimensionality=64" in text and "trained=False" in text


@pytest.mark.parametrize("kwargs", [dict(n_clusters=0, dimensionality=50), dict(n_clusters=10, dimensionality=0),
                                    dict(n_clusters=10, dimensionality=50, sampling_fraction=1.5)])
def test_constructor_rejects_invalid_parameters(kwargs):
    with pytest.raises(ValueError):
        SuperKMeans(**kwargs)


# ---- flat training (test_train_simple, test_iteration_stats, test_assign, test_assign_different_data)
def test_train_returns_float32_centroids_and_iteration_records():
    n, d, k = 10_000, 512, 100
    data = _gauss(n, d, 1)
    km = SuperKMeans(n_clusters=k, dimensionality=d, iters=5, verbose=True)
    c = km.train(data)
    assert c.shape == (k, d) and c.dtype == np.float32 and km.is_trained_
    stats = km.iteration_stats
    assert len(stats) == 5
    for i, s in enumerate(stats):
        assert isinstance(s, SuperKMeansIterationStats)
        assert s.iteration == i + 1 and s.objective > 0 and s.shift >= 0
    a = km.assign(data, c)
    assert a.shape == (n,) and a.dtype == np.uint32 and a.max() < k
    other = km.assign(_gauss(500, d, 2), c)
    assert other.shape == (500,) and other.max() < k
    assert "trained=True" in repr(km)


def test_train_with_queries_records_recall():
    # test_train_with_queries
    n, d, k = 10_000, 512, 100
    km = SuperKMeans(n_clusters=k, dimensionality=d, iters=5, objective_k=10)
    c = km.train(_gauss(n, d, 3), queries=_gauss(50, d, 4))
    assert c.shape == (k, d) and km.is_trained_ and len(km.iteration_stats) > 0
    assert all(0.0 <= s.recall <= 1.0 for s in km.iteration_stats)


# ---- validation (test_train_dtype_validation, test_train_shape_validation, test_train_dimensionality_mismatch, test_assign_validation)
def test_train_and_assign_validate_their_arrays():
    km = SuperKMeans(n_clusters=10, dimensionality=32)
    with pytest.raises(ValueError, match="dtype float32"):
        km.train(_gauss(100, 32).astype(np.float64))
    with pytest.raises(ValueError, match="2-dimensional"):
        km.train(_gauss(100, 32).reshape(-1))
    with pytest.raises(ValueError, match="2-dimensional"):
        km.train(_gauss(100, 64).reshape(100, 32, 2))
    with pytest.raises(ValueError, match="dimensionality"):
        km.train(_gauss(100, 64))
    data = _gauss(100, 512, 5)
    km = SuperKMeans(n_clusters=10, dimensionality=512)
    c = km.train(data)
    with pytest.raises(ValueError, match="dtype float32"):
        km.assign(data.astype(np.float64), c)
    with pytest.raises(ValueError, match="same dimensionality"):
        km.assign(_gauss(100, 16), c)


def test_non_contiguous_input_is_accepted():
    # test_non_contiguous_arrays
    wide = _gauss(100, 512, 6)
    km = SuperKMeans(n_clusters=10, dimensionality=256)
    c = km.train(wide[:, ::2])
    assert c.shape == (10, 256)
    np.testing.assert_array_equal(c, SuperKMeans(n_clusters=10, dimensionality=256).train(np.ascontiguousarray(wide[:, ::2])))


# ---- reproducibility (test_reproducibility, test_hierarchical_reproducibility)
@pytest.mark.parametrize("hier", [False, True])
def test_same_seed_gives_the_same_bits(hier):
    data = _gauss(10_000, 512, 7)
    kw = dict(hierarchical=True, iters_mesoclustering=3, iters_fineclustering=3, iters_refinement=1) if hier else dict(iters=5)
    a = SuperKMeans(n_clusters=100, dimensionality=512, seed=123, **kw).train(data)
    b = SuperKMeans(n_clusters=100, dimensionality=512, seed=123, **kw).train(data)
    np.testing.assert_array_equal(a, b)


# ---- hierarchical mode (test_hierarchical_explicit_true / _false, _auto_small_dataset, _auto_large_dataset, _assign, _iteration_stats, _repr)
def test_hierarchical_when_asked_for():
    n, d, k = 10_000, 512, 100
    data = _gauss(n, d, 8)
    km = SuperKMeans(n_clusters=k, dimensionality=d, hierarchical=True, iters_mesoclustering=3, iters_fineclustering=3, iters_refinement=2, verbose=True)
    assert "trained=False" in repr(km)
    c = km.train(data)
    assert c.shape == (k, d) and c.dtype == np.float32 and km.is_trained_ and km.hierarchical_ is True
    hs = km.hierarchical_iteration_stats
    assert isinstance(hs, HierarchicalSuperKMeansIterationStats)
    assert len(hs.mesoclustering_iteration_stats) == 3
    assert 0 < len(hs.fineclustering_iteration_stats) <= 10 * 3   # ten mesoclusters, three iterations each at most
    assert len(hs.refinement_iteration_stats) == 2
    a = km.assign(data, c)
    assert a.shape == (n,) and a.dtype == np.uint32 and a.max() < k
    assert "hierarchical=True" in repr(km)


def test_flat_when_asked_for_and_for_small_inputs():
    data = _gauss(10_000, 512, 9)
    km = SuperKMeans(n_clusters=100, dimensionality=512, hierarchical=False, iters=5)
    assert km.train(data).shape == (100, 512)
    assert km.hierarchical_ is False and km.hierarchical_iteration_stats is None
    km = SuperKMeans(n_clusters=100, dimensionality=128, iters=3)     # n <= 100 000: flat by default
    km.train(_gauss(50_000, 128, 10))
    assert km.hierarchical_ is False


def test_hierarchical_by_default_above_100000_points():
    km = SuperKMeans(n_clusters=256, dimensionality=128, iters_mesoclustering=3, iters_fineclustering=3, iters_refinement=1)
    c = km.train(_gauss(150_000, 128, 11))
    assert c.shape == (256, 128) and km.hierarchical_ is True and km.hierarchical_iteration_stats is not None


# ---- fast assignment of the training points (test_assign_training_points)
def test_assign_training_points_agrees_with_brute_force():
    n, d, k = 50_000, 512, 500
    data = _gauss(n, d, 12)
    km = SuperKMeans(n_clusters=k, dimensionality=d, iters=5)
    c = km.train(data)
    brute = km.assign(data, c)
    fast = km.assign_training_points(data, c)
    assert fast.shape == (n,) and fast.dtype == np.uint32 and fast.max() < k
    assert float((brute == fast).mean()) >= 0.95


def test_package_exports():
    assert skm.__version__
    for name in ("SuperKMeans", "SuperKMeansIterationStats", "HierarchicalSuperKMeansIterationStats"):
        assert name in skm.__all__
