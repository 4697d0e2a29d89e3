"""Parity of the single CUDA operators with the compiled reference (oracle/_ref), through the C ABI.

Floating-point bars (fp32 arithmetic on both sides, different summation order):
  * distances / rotated values: 1e-5 relative to the row scale (stated per test);
  * assignments: identical except near-ties, where the reference-domain distance of the two answers
    differs by less than 1e-5 relative (the north-star bar);
  * integer outputs (counts, not-pruned counters, layouts): bit-exact.
"""
import numpy as np
import pytest

from tests import datagen, parity_util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", params=["tensor_cores", "simt"])
def eng(request):
    """Every operator test runs twice: dense products on the tcgen05 kernels and on the SIMT kernels."""
    from superkmeans_b200 import engine

    engine.set_tensor_cores(request.param == "tensor_cores")
    yield engine
    engine.set_tensor_cores(True)


def _near_tie_ok(x, y, a, b, rel=1e-5):
    """For rows where a != b: exact (float64) distances to both answers agree within rel."""
    idx = np.nonzero(a != b)[0]
    if len(idx) == 0:
        return True, 0
    xd = x[idx].astype(np.float64)
    da = ((xd - y[a[idx]].astype(np.float64)) ** 2).sum(1)
    db = ((xd - y[b[idx]].astype(np.float64)) ** 2).sum(1)
    ok = np.abs(da - db) <= rel * np.maximum(np.minimum(da, db), 1e-30)
    return bool(ok.all()), len(idx)


@pytest.mark.parametrize("n,d", [(1000, 64), (777, 130), (4096, 768), (129, 1024)])
def test_rotate_and_unrotate(eng, ref, n, d):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((n, d), dtype=np.float32)
    m = eng.rotation_matrix(d, 3)
    r = eng.rotate(m, x)
    want = x.astype(np.float64) @ m.astype(np.float64).T
    # fp32 accumulation level: rows have norm sqrt(d), outputs are O(1); a single long chain in tensor memory would be ~1e-5 * sqrt(d) off
    assert np.abs(r - want).max() < 1e-6 * np.sqrt(d)
    # tests/test_rotation.cpp: norms preserved, Unrotate(Rotate(x)) = x within 1e-4
    assert np.abs(np.linalg.norm(r, axis=1) - np.linalg.norm(x, axis=1)).max() < 1e-4 * np.sqrt(d)
    back = eng.unrotate(m, r)
    assert np.abs(back - x).max() < 1e-4


@pytest.mark.parametrize("n,k,d", [(5000, 1000, 64), (4097, 1025, 128), (333, 7, 33), (3000, 2500, 768), (1, 1, 4), (128, 128, 16)])
def test_find_nearest_matches_reference(eng, ref, n, k, d):
    # tests/test_distance_computers.cpp:83-152 (FindNearestNeighbor vs brute force, rel 1e-4)
    x = datagen.gaussian_mixture(n, d, max(k // 2, 1), 0.3, 5)
    y = datagen.gaussian_mixture(k, d, max(k // 2, 1), 0.3, 6)
    knn, dist = eng.find_nearest(x, y)
    rknn, rdist = ref.find_nearest(x, y)
    ok, n_diff = _near_tie_ok(x, y, knn.astype(np.int64), rknn.astype(np.int64))
    assert ok
    assert n_diff <= max(1, n // 1000)
    assert np.abs(dist - rdist).max() <= 1e-5 * max(1.0, float(np.abs(rdist).max()))
    assert (dist >= 0).all()


def test_find_nearest_exact_duplicates_pick_lowest_index(eng):
    # First minimum inside a batch, strict < across batches (batch_computers.h:163-164).
    rng = np.random.default_rng(2)
    d, k = 32, 2100
    y = rng.standard_normal((k, d), dtype=np.float32)
    y[1500] = y[3]
    y[2050] = y[3]
    y[1100] = y[1030]
    # queries slightly off the duplicated rows: the duplicates then tie at the same positive distance
    x = (np.stack([y[3], y[1030], y[7]]) + 0.01 * rng.standard_normal((3, d), dtype=np.float32)).astype(np.float32)
    knn, dist = eng.find_nearest(x, y)
    assert list(knn) == [3, 1030, 7]


@pytest.mark.parametrize("n,k,d", [(3000, 700, 128), (2500, 1500, 384), (1000, 2049, 130), (2000, 1024, 768)])
def test_pdxify_is_bit_exact(eng, ref, n, k, d):
    y = np.random.default_rng(3).standard_normal((k, d), dtype=np.float32)
    np.testing.assert_array_equal(eng.pdxify(y), ref.pdxify(y))


@pytest.mark.parametrize("n,k,d", [(20000, 300, 128), (5000, 4000, 64), (1025, 3, 33), (70000, 1000, 256), (10, 70000, 8)])
def test_update_centroids(eng, n, k, d):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((n, d), dtype=np.float32)
    # Zipf-like sizes, so that some clusters span many tiles and many are empty
    w = np.arange(1, k + 1, dtype=np.float64) ** -1.1
    a = rng.choice(k, size=n, p=w / w.sum()).astype(np.uint32)
    dist = rng.random(n, dtype=np.float32)
    sums, counts, wcss = eng.update_centroids(x, a, k, dist)
    np.testing.assert_array_equal(counts, np.bincount(a, minlength=k).astype(np.uint32))
    want = np.zeros((k, d), dtype=np.float64)
    np.add.at(want, a, x.astype(np.float64))
    scale = np.sqrt(np.maximum(counts, 1))[:, None]
    assert np.abs(sums - want).max() <= 2e-6 * float(np.abs(want).max() + scale.max())
    assert abs(wcss - float(dist.astype(np.float64).sum())) <= 1e-9 * n
    # deterministic: a second run gives the same bits
    sums2, counts2, _ = eng.update_centroids(x, a, k, dist)
    np.testing.assert_array_equal(sums, sums2)


_TRACES = {}


def _trace(ref, n, d, k, iters, seed, hier=False, centers=None, **kw):
    """A traced reference run; kept for the other routes of the same shape (the run is deterministic)."""
    key = (n, d, k, iters, seed, hier, centers, tuple(sorted(kw.items())))
    if key not in _TRACES:
        x = datagen.gaussian_mixture(n, d, centers or k, 0.3, seed)
        cfg = ref.default_config(hier, iters=iters, sampling_fraction=1.0, early_termination=0, seed=seed, **kw)
        km = ref.RefKMeans(k, d, cfg, hierarchical=hier, trace=True)
        cent = km.train(x)
        _TRACES[key] = (x, km, cent)
    return _TRACES[key]


@pytest.mark.parametrize("split_mode", [0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11],
                         ids=["auto", "lists_only", "dense_simt_only", "tensor_core_chain", "tensor_core_lists", "tensor_core_lists_overflowing", "ordered_gathered_chain",
                              "ordered_lists", "ordered_lists_overflowing", "unordered_lists_and_chain", "ordered_optimistic_chain", "ordered_route_per_tile"])
@pytest.mark.parametrize("n,d,k", [(20000, 256, 512), (12000, 768, 1500), (6000, 130, 1030), (9000, 1024, 2100)])
def test_pruned_step_matches_reference_teacher_forced(eng, ref, n, d, k, split_mode):
    """Every pruned iteration of a reference run, replayed from the reference's own inputs, with the
    points routed through the candidate-list kernel, the dense-chain kernel, or split between them."""
    if split_mode >= 3 and (d % 4 != 0 or not eng.tensor_cores_enabled()):
        pytest.skip("the tensor-core kernels need d % 4 == 0 and to be switched on")
    eng.set_prune_split(split_mode)
    try:
        # the tensor-memory accumulator truncates: partial distances sit ~1e-5 (relative to the dot product)
        # high, which moves a few more pairs across the thresholds than fp32 rounding does
        _pruned_step_check(eng, ref, n, d, k, count_tol=5e-3 if split_mode in (0, 3, 4, 5, 6, 7, 8, 9, 10, 11) else 1e-3)
    finally:
        eng.set_prune_split(0)


def _pruned_step_check(eng, ref, n, d, k, count_tol=1e-3):
    x, km, _ = _trace(ref, n, d, k, 5, 17)
    m = km.rotation_matrix()
    xr = eng.rotate(m, x)
    trace, stats = km.trace(), km.stats()
    checked = 0
    for t in range(1, len(trace)):
        prev, cur, st = trace[t - 1], trace[t], stats[t]
        assert not st["is_gemm_only"]
        pd = st["partial_d"]
        # the reference on the same rotated input (bitwise the same y, prev assignment and d')
        rknn, rdist, rnp = ref.find_nearest_pruned(xr, prev.centroids, prev.assign, pd)
        knn, dist, npc = eng.find_nearest_pruned(xr, prev.centroids, prev.assign, pd)
        agree = float((knn == rknn).mean())
        assert agree >= 0.999, (t, agree)
        # every disagreement is a near-tie (1e-5 relative) or an ADSampling false prune that rounding flipped at a
        # threshold (pdx/pdxearch.h:67-80); a float64 replay of the affected points must explain all of them
        hd, vd = eng.dimension_split(d)
        n_tie, n_flip, unexplained = parity_util.classify_disagreements(xr, prev.centroids, prev.assign.astype(np.int64), knn.astype(np.int64), rknn.astype(np.int64), pd, vd,
                                                                        eng.ratios(d, 1.5))
        assert not unexplained, (t, n_tie, n_flip, unexplained[:8])
        same = knn == rknn
        assert np.abs(dist[same] - rdist[same]).max() <= 2e-5 * max(1.0, float(rdist.max()))
        # not-pruned counters: integer, but each counts threshold tests on rounded partial distances
        tot, rtot = float(npc.sum()), float(rnp.sum())
        assert abs(tot - rtot) <= count_tol * rtot + 10, (tot, rtot)
        nd, _ = eng.tune_partial_d(tot, n, k, pd, eng.dimension_split(d)[1])
        assert nd == cur.partial_d_next
        checked += 1
    assert checked >= 3
