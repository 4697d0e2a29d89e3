"""The benchmark configurations themselves.

* Config 1 (n = 100 000, d = 768, k = 1000, the reference's CPU-runnable case) at full size against the compiled
  reference, with the north-star gates: WCSS within 1e-4 relative, >= 99.9 % identical assignments, centroids of
  clusters with identical members within 1e-5 (any single near-tie that falls the other way moves two centroids by
  ~1/cluster size, which is why the plain centroid norm is gated at 5e-3 and not at 1e-4).
* Config 2's data law at a size the reference finishes in seconds.
* Configs 2, 3 and 5 at FULL size on device-generated data, through properties that do not need the reference:
  exact assignment is the float64 arg-min on sampled rows (up to near-ties of 1e-5), the pruned assignment of the
  training points agrees with the exact one on >= 98 % of the points (the reference's own bar,
  tests/test_assign.cpp:152-155), centroids are the means of their members, a second run gives the same bits.
* Config 4 (hierarchical) at a size the reference finishes in seconds, and its full-size run through properties.
"""
import numpy as np
import pytest

from tests import datagen

pytestmark = pytest.mark.gpu


def _wcss64(x, c, a):
    return float(((x.astype(np.float64) - c[a].astype(np.float64)) ** 2).sum())


def test_config1_full_size_matches_reference(ref):
    import superkmeans_b200 as skm

    n, d, k, seed = 100_000, 768, 1000, 42
    x = datagen.config1(n, d, k, seed)
    kw = dict(iters=10, sampling_fraction=1.0, early_termination=0, seed=seed)
    rk = ref.RefKMeans(k, d, ref.default_config(False, **kw))
    rc = rk.train(x)
    e = skm.Engine(k, d, skm.default_config(False, **kw))
    e.set_rotation(rk.rotation_matrix())
    c = e.train(x)
    rs, es = rk.stats(), e.stats(0)
    assert len(rs) == len(es) == 10
    assert [r["partial_d"] for r in rs] == [s.partial_d for s in es]
    ra, a = rk.assignments(), e.assignments()
    w, rw = _wcss64(x, c, a), _wcss64(x, rc, ra)
    assert abs(w - rw) <= 1e-4 * rw, (w, rw)
    assert (ra == a).mean() >= 0.999
    same = np.ones(k, dtype=bool)
    diff = a != ra
    same[a[diff]] = False
    same[ra[diff]] = False
    cr, rcr = e.rotated_centroids(), rk.rotated_centroids()
    rel = np.linalg.norm(cr[same].astype(np.float64) - rcr[same], axis=1) / (np.linalg.norm(rcr[same], axis=1) + 1e-30)
    assert same.mean() >= 0.97 and rel.max() < 1e-5, (same.mean(), rel.max())
    assert np.linalg.norm(c - rc) / np.linalg.norm(rc) < 5e-3
    # Train + Assign, as the configuration says
    asg, rasg = e.assign(x, c), rk.assign(x, rc)
    assert (asg == rasg).mean() >= 0.999


def test_config2_shape_matches_reference(ref):
    """Config 2's data law (anisotropic mixture, d = 1536) at n = 60 000, k = 1024, against the reference."""
    import superkmeans_b200 as skm

    n, d, k, seed = 60_000, 1536, 1024, 7
    x = datagen.config2(n, d, k, seed)
    kw = dict(iters=8, sampling_fraction=1.0, early_termination=0, seed=seed)
    rk = ref.RefKMeans(k, d, ref.default_config(False, **kw))
    rc = rk.train(x)
    e = skm.Engine(k, d, skm.default_config(False, **kw))
    e.set_rotation(rk.rotation_matrix())
    c = e.train(x)
    assert [r["partial_d"] for r in rk.stats()] == [s.partial_d for s in e.stats(0)]
    ra, a = rk.assignments(), e.assignments()
    w, rw = _wcss64(x, c, a), _wcss64(x, rc, ra)
    assert abs(w - rw) <= 1e-4 * rw, (w, rw)
    # One point of the exact first iteration is an fp32 near-tie that OpenBLAS and this engine round differently (the
    # SIMT kernels give the same single difference); the 109 cluster splits of iteration 2 spread it to ~65 points
    # (0.11 %) by iteration 5, after which it stays put.  The per-step tests (test_ops_gpu.py) hold each iteration
    # to >= 99.9 % from identical inputs; end to end this configuration is held to 99.8 %.
    assert (ra == a).mean() >= 0.998
    # ... and a cluster emptied in one run only is re-seeded by the split step, so centroids are compared where the
    # members are the same
    same = np.ones(k, dtype=bool)
    diff = a != ra
    same[a[diff]] = False
    same[ra[diff]] = False
    cr, rcr = e.rotated_centroids(), rk.rotated_centroids()
    rel = np.linalg.norm(cr[same].astype(np.float64) - rcr[same], axis=1) / (np.linalg.norm(rcr[same], axis=1) + 1e-30)
    assert same.mean() >= 0.9 and rel.max() < 1e-5, (same.mean(), rel.max())
    w2, rw2 = _wcss64(x, c, e.assign(x, c)), _wcss64(x, rc, rk.assign(x, rc))
    assert abs(w2 - rw2) <= 1e-3 * rw2


def test_config4_shape_hierarchical_matches_reference(ref):
    """Hierarchical Train + Assign on the configuration's data law at n = 200 000, k = 4096 (64 mesoclusters)."""
    import superkmeans_b200 as skm

    n, d, k, seed = 200_000, 768, 4096, 2024
    x = datagen.config4(n, d, supers=64, subs=64, seed=seed)
    kw = dict(early_termination=0, seed=seed)
    rk = ref.RefKMeans(k, d, ref.default_config(True, **kw), hierarchical=True)
    rc = rk.train(x)
    e = skm.Engine(k, d, skm.default_config(True, **kw), hierarchical=True)
    e.set_rotation(rk.rotation_matrix())
    c = e.train(x)
    assert e.n_mesoclusters == rk.n_mesoclusters() == 64
    assert len(e.stats(1)) == len(rk.stats(1)) and len(e.stats(2)) == len(rk.stats(2)) and len(e.stats(3)) == len(rk.stats(3))
    ra, a = rk.final_assignments(), e.assignments()
    w, rw = _wcss64(x, c, a), _wcss64(x, rc, ra)
    # a mesocluster whose member list differs by one point restarts from other points (see test_train_gpu.py); the
    # reference's own end-to-end bar is 5 % on WCSS
    assert abs(w - rw) <= 5e-2 * rw, (w, rw)
    asg = e.assign(x, c)
    assert _wcss64(x, c, asg) <= w * (1 + 1e-6)
    atp = e.assign_training_points(x, c)
    assert (atp == asg).mean() >= 0.98


# ---------------------------------------------------------------------------------------------------------------
# full-size runs on device-generated data
# ---------------------------------------------------------------------------------------------------------------
def _mixture_on_device(torch, n, d, centers, noise, seed, center_std=None, chunk=500_000):
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    c = torch.randn(centers, d, generator=g, device=dev, dtype=torch.float32)
    scale = None
    if center_std is not None:
        scale = torch.from_numpy(np.asarray(center_std, dtype=np.float32)).to(dev)
        c *= scale
    x = torch.empty(n, d, device=dev, dtype=torch.float32)
    for s in range(0, n, chunk):
        e = min(n, s + chunk)
        labels = torch.randint(0, centers, (e - s,), generator=g, device=dev)
        blk = torch.randn(e - s, d, generator=g, device=dev, dtype=torch.float32) * noise
        if scale is not None:
            blk *= scale
        blk += c[labels]
        blk /= blk.norm(dim=1, keepdim=True)
        x[s:e] = blk
    torch.cuda.synchronize()
    return x


def _exact_assign_is_argmin(torch, e, x, c, rows=4096, seed=0):
    """Exact assignment of sampled rows equals the float64 arg-min, except near-ties: within 1e-5 relative, plus the
    rounding of ||x||^2 + ||c||^2 - 2 x.c in fp32 (the reference's formula, batch_computers.h:152-163), which is about
    1e-7 of the norms whatever the distance."""
    g = torch.Generator(device=x.device)
    g.manual_seed(seed)
    idx = torch.randint(0, x.shape[0], (rows,), generator=g, device=x.device)
    xs = x[idx].cpu().numpy()
    a = e.assign(xs, c).astype(np.int64)
    xd, cd = xs.astype(np.float64), c.astype(np.float64)
    dist = (xd * xd).sum(1)[:, None] + (cd * cd).sum(1)[None, :] - 2.0 * xd @ cd.T
    want = dist.argmin(1)
    bad = np.nonzero(a != want)[0]
    if len(bad):
        da, dw = dist[bad, a[bad]], dist[bad, want[bad]]
        norms = (xd[bad] * xd[bad]).sum(1) + (cd[a[bad]] * cd[a[bad]]).sum(1)
        assert (np.abs(da - dw) <= 1e-5 * dw + 1e-6 * norms).all(), (da, dw)
    assert len(bad) <= max(1, rows // 500)
    return idx, a


def _centroids_are_member_means(torch, x, c, assign, k, ok_fraction=0.97):
    dev = x.device
    a = torch.from_numpy(assign.astype(np.int64)).to(dev)
    counts = torch.bincount(a, minlength=k).to(torch.float64)
    sums = torch.zeros(k, x.shape[1], device=dev, dtype=torch.float32)
    step = 1_000_000
    for s in range(0, x.shape[0], step):
        sums.index_add_(0, a[s:s + step], x[s:s + step])
    means = (sums.to(torch.float64) / counts.clamp(min=1)[:, None]).cpu().numpy()
    cnt = counts.cpu().numpy()
    rel = np.linalg.norm(means - c.astype(np.float64), axis=1) / (np.linalg.norm(c.astype(np.float64), axis=1) + 1e-30)
    good = (rel < 1e-4) | (cnt == 0)
    # clusters that were re-seeded by the last split step are perturbed copies of other centroids, not means
    assert good.mean() >= ok_fraction, float(good.mean())


def _train_properties(torch, skm, x, k, iters, seed, check_means=True, second_run=True):
    n, d = x.shape
    cfg = dict(iters=iters, sampling_fraction=1.0, early_termination=0, seed=seed)
    e = skm.Engine(k, d, skm.default_config(False, **cfg))
    c = e.train(x, n=n, on_device=True)
    st = e.stats(0)
    assert len(st) == iters and st[0].is_gemm_only
    vd = skm.engine.dimension_split(d)[1]
    for s in st[1:]:
        assert not s.is_gemm_only and 16 <= s.partial_d <= vd and 0.0 < s.not_pruned_pct < 1.0
    # Lloyd iterations do not increase the objective (the splits of the first iterations aside)
    obj = [s.objective for s in st]
    assert obj[-1] < obj[1] and all(obj[i + 1] <= obj[i] * (1 + 1e-3) for i in range(2, iters - 1))
    a_train = e.assignments()
    assert a_train.shape == (n,) and a_train.max() < k
    if check_means:
        _centroids_are_member_means(torch, x, c, a_train, k)
    _exact_assign_is_argmin(torch, e, x, c)
    # pruned assignment of the training points against exact assignment, all points, on the device
    out_exact = torch.empty(n, dtype=torch.int32, device=x.device)
    out_fast = torch.empty(n, dtype=torch.int32, device=x.device)
    cd = torch.from_numpy(c).to(x.device)
    e.assign(x, cd, n=n, on_device=True, out=out_exact)
    e.assign_training_points(x, cd, n=n, on_device=True, out=out_fast)
    torch.cuda.synchronize()
    assert float((out_exact == out_fast).float().mean()) >= 0.98
    if second_run:
        e2 = skm.Engine(k, d, skm.default_config(False, **cfg))
        c2 = e2.train(x, n=n, on_device=True)
        np.testing.assert_array_equal(c, c2)
    return e, c


def test_config2_full_size_properties():
    import torch

    torch.cuda.empty_cache()

    import superkmeans_b200 as skm

    n, d, k = 1_000_000, 1536, 4096
    s = 1.0 / np.sqrt(1.0 + np.arange(d) / 64.0)
    x = _mixture_on_device(torch, n, d, k, 0.3, 7, center_std=s)
    _train_properties(torch, skm, x, k, 10, 7)


def test_config3_full_size_properties():
    import torch

    torch.cuda.empty_cache()

    import bench
    import superkmeans_b200 as skm

    n, d, k = 10_000_000, 1024, 10_000
    free, _ = torch.cuda.mem_get_info()
    if free < 120 * 2**30:
        pytest.skip("needs 120 GB of free device memory")
    dev = torch.device("cuda", torch.cuda.current_device())
    x = bench.make_shard(torch, dev, n, d, 10_000, 0.25, 1.1, 123, 0, n, 0)
    _train_properties(torch, skm, x, k, 10, 123, second_run=False)


def test_config5_full_size_assign_properties():
    """Assign only: 5e7 x 384 points (77 GB, generated on the device) against 16 384 fixed centroids."""
    import torch

    torch.cuda.empty_cache()

    import superkmeans_b200 as skm

    n, d, k = 50_000_000, 384, 16_384
    free, _ = torch.cuda.mem_get_info()
    if free < 100 * 2**30:
        pytest.skip("needs 100 GB of free device memory")
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev)
    g.manual_seed(99)
    c = torch.randn(k, d, generator=g, device=dev, dtype=torch.float32)
    c /= c.norm(dim=1, keepdim=True)
    x = torch.empty(n, d, device=dev, dtype=torch.float32)
    step = 1_000_000
    for s in range(0, n, step):
        lab = torch.randint(0, k, (step,), generator=g, device=dev)
        blk = c[lab] + 0.3 * torch.randn(step, d, generator=g, device=dev, dtype=torch.float32)
        blk /= blk.norm(dim=1, keepdim=True)
        x[s:s + step] = blk
    e = skm.Engine(k, d, skm.default_config(False))
    out = torch.empty(n, dtype=torch.int32, device=dev)
    e.assign(x, c, n=n, on_device=True, out=out)
    torch.cuda.synchronize()
    ch = c.cpu().numpy()
    idx, a = _exact_assign_is_argmin(torch, e, x, ch, rows=2048)
    # the device-resident call and the host-chunked call give the same answer for the same rows
    assert (out[idx].cpu().numpy().astype(np.int64) == a).mean() >= 0.999
    # every centroid is used (the points were drawn around all of them)
    assert int(torch.unique(out).numel()) == k
    # idempotence: assigning the centroids themselves returns the identity
    ident = e.assign(ch, ch)
    assert (ident == np.arange(k)).all()


def test_config4_full_size_properties():
    """Hierarchical Train at n = 1e7, d = 768, k = 65 536 (256 mesoclusters), then Assign on a sample."""
    import torch

    torch.cuda.empty_cache()

    import superkmeans_b200 as skm

    n, d, k = 10_000_000, 768, 65_536
    free, _ = torch.cuda.mem_get_info()
    if free < 120 * 2**30:
        pytest.skip("needs 120 GB of free device memory")
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev)
    g.manual_seed(2024)
    sup = torch.randn(256, d, generator=g, device=dev, dtype=torch.float32)
    sub = (sup[:, None, :] + 0.2 * torch.randn(256, 256, d, generator=g, device=dev, dtype=torch.float32)).reshape(k, d)
    x = torch.empty(n, d, device=dev, dtype=torch.float32)
    step = 1_000_000
    for s in range(0, n, step):
        lab = torch.randint(0, k, (step,), generator=g, device=dev)
        blk = sub[lab] + 0.1 * torch.randn(step, d, generator=g, device=dev, dtype=torch.float32)
        blk /= blk.norm(dim=1, keepdim=True)
        x[s:s + step] = blk
    del sub
    e = skm.Engine(k, d, skm.default_config(True, early_termination=0, seed=2024, sampling_fraction=1.0), hierarchical=True)
    c = e.train(x, n=n, on_device=True)
    assert e.n_mesoclusters == 256
    assert len(e.stats(1)) == 3 and len(e.stats(2)) == 256 * 5
    a = e.assignments()
    assert a.shape == (n,) and a.max() < k
    idx, a_s = _exact_assign_is_argmin(torch, e, x, c, rows=1024)
    # the fine clustering is far tighter than the mesoclustering it started from
    meso_obj = e.stats(1)[-1].objective / n
    xs = x[idx].cpu().numpy().astype(np.float64)
    fine_obj = float(((xs - c[a_s].astype(np.float64)) ** 2).sum(1).mean())
    assert fine_obj < 0.5 * meso_obj, (fine_obj, meso_obj)
    # pruned assignment of the training points against brute force, all points
    out_exact = torch.empty(n, dtype=torch.int32, device=dev)
    out_fast = torch.empty(n, dtype=torch.int32, device=dev)
    cd = torch.from_numpy(c).to(dev)
    e.assign(x, cd, n=n, on_device=True, out=out_exact)
    e.assign_training_points(x, cd, n=n, on_device=True, out=out_fast)
    torch.cuda.synchronize()
    assert float((out_exact == out_fast).float().mean()) >= 0.98
