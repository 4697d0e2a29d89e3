"""The allocation-free exact-assignment entry point against the regular one.

Collected last on purpose (file name): the entry point keeps its intermediate data in a fixed array inside the
library's device image, and must work both as the first CUDA call of a fresh process and after every other
test has used the device.
"""
import numpy as np
import pytest

from tests import datagen

pytestmark = pytest.mark.gpu


def _device_copy(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run_noalloc(skm, torch, x, y):
    n, d = x.shape
    xd, yd = _device_copy(torch, x), _device_copy(torch, y)
    # filled with garbage so that stale contents cannot pass for results
    knn = torch.full((n,), 0x7FFFFFFF, dtype=torch.int32, device="cuda")
    dist = torch.full((n,), -1.0, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    # The reason the entry point exists: the library itself must not allocate on this call, neither on the first one
    # for a device nor on any later one (the counter covers every cudaMalloc / cudaMallocHost the library makes).
    before = skm.engine.device_allocations()
    skm.engine.find_nearest_noalloc(xd.data_ptr(), yd.data_ptr(), n, y.shape[0], d, knn.data_ptr(), dist.data_ptr(), device=torch.cuda.current_device())
    assert skm.engine.device_allocations() == before
    return knn.cpu().numpy().view(np.uint32), dist.cpu().numpy()


def _reference_answer(x, y):
    """FindNearestNeighbor of the compiled reference, or None where it was not built."""
    from oracle import ref

    if not ref.available():
        return None
    return ref.find_nearest(x, y)


def _compare(x, y, knn, dist, knn0, dist0):
    # the bar of the exact-assignment operator tests: same winners except fp32 near-ties (float64 distances of the
    # two answers within 1e-5 relative), distances within 1e-5 of the row scale
    idx = np.nonzero(knn != knn0)[0]
    assert len(idx) <= max(1, len(knn) // 1000)
    if len(idx):
        xd = x[idx].astype(np.float64)
        da = ((xd - y[knn[idx]].astype(np.float64)) ** 2).sum(1)
        db = ((xd - y[knn0[idx]].astype(np.float64)) ** 2).sum(1)
        assert (np.abs(da - db) <= 1e-5 * np.maximum(np.minimum(da, db), 1e-30)).all()
    assert np.abs(dist - dist0).max() <= 1e-5 * max(1.0, float(np.abs(dist0).max()))
    assert (dist >= 0).all()


@pytest.mark.parametrize("n,d,k", [(5000, 128, 300), (3001, 100, 77), (1000, 30, 17)])
def test_noalloc_matches_regular_entry_point_twice(n, d, k):
    import torch

    import superkmeans_b200 as skm

    # two calls in a row with different inputs and shapes of use: the second sees what the first left behind
    for seed in (41, 42):
        x = datagen.gaussian_mixture(n, d, k, 0.3, seed)
        y = x[np.random.default_rng(seed).choice(n, k, replace=False)].copy() + 1e-3
        knn0, dist0 = skm.engine.find_nearest(x, y)
        knn, dist = _run_noalloc(skm, torch, x, y)
        _compare(x, y, knn, dist, knn0, dist0)
        # ... and against the reference's own operator, at the bar of the regular operator's test
        r = _reference_answer(x, y)
        if r is not None:
            _compare(x, y, knn, dist, r[0], r[1])


def test_noalloc_large_then_small_call():
    import torch

    import superkmeans_b200 as skm

    xa = datagen.gaussian_mixture(40000, 256, 1200, 0.3, 43)
    ya = xa[:1200].copy() + 1e-3
    xb = datagen.gaussian_mixture(700, 256, 40, 0.3, 44)
    yb = xb[:40].copy() + 1e-3
    for x, y in ((xa, ya), (xb, yb)):
        knn0, dist0 = skm.engine.find_nearest(x, y)
        knn, dist = _run_noalloc(skm, torch, x, y)
        _compare(x, y, knn, dist, knn0, dist0)
        r = _reference_answer(x, y)
        if r is not None:
            _compare(x, y, knn, dist, r[0], r[1])


def test_noalloc_rejects_sizes_beyond_the_static_scratch():
    import torch

    import superkmeans_b200 as skm

    t = torch.zeros(16, dtype=torch.float32, device="cuda")
    # the size check comes before any access, so small buffers are enough here
    with pytest.raises(ValueError, match="at most 262144 rows"):
        skm.engine.find_nearest_noalloc(t.data_ptr(), t.data_ptr(), 262145, 4, 4, t.data_ptr(), t.data_ptr())
    with pytest.raises(ValueError, match="at most 65536 centroids"):
        skm.engine.find_nearest_noalloc(t.data_ptr(), t.data_ptr(), 4, 65537, 4, t.data_ptr(), t.data_ptr())
