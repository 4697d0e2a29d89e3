"""The benchmark configurations against the compiled reference at the sizes the reference can run on the host:

* config 2 (flat, n = 1 000 000, d = 1536, k = 4096, seed 7) at FULL size;
* config 3 (flat headline shape, d = 1024, k = 10 000, Zipf sizes, seed 123) on a slice of n = 1 000 000 rows;
* config 4 (hierarchical, d = 768, two-level mixture, seed 2024) on a slice of n = 1 000 000 rows with k = 16 384
  (128 mesoclusters; the full k = 65 536 would leave 15 points per cluster on the slice).

Each flat configuration is checked twice:
  step-wise  - pruned iterations replayed from the reference's own state (its rotated points, centroids, previous
               assignment and d'): >= 99.9 % identical assignments (answers that tie within the rounding of the reference's
               own fp32 distances counted as equal; nearly all of them lie between centroids that coincide to rounding,
               which repeated splits of one cluster leave behind), every sampled disagreement explained as a near-tie
               or a threshold flip, not-pruned totals and the next d' as the reference's;
  end to end - same d' schedule, centroids of clusters with identical members within 1e-5, WCSS within 2e-3 and a
               floor on the share of identical assignments (both reported; single near-tie flips are amplified by
               the cluster splits at these sizes, see the comment at the gates).
"""
import numpy as np
import pytest

from tests import datagen, parity_util

pytestmark = pytest.mark.gpu


def _wcss64(x, c, a, block=200_000):
    tot = 0.0
    for s in range(0, x.shape[0], block):
        xs = x[s:s + block].astype(np.float64)
        tot += float(((xs - c[a[s:s + block]].astype(np.float64)) ** 2).sum())
    return tot


def _identical_cluster_centroids(c, rc, a, ra, k):
    """Share of clusters with the same (non-empty) member set in both runs, and the largest relative centroid difference
    among them, leaving out clusters that differ by no more than the 1/1024 scaling of a split (the last consolidation
    may draw other clusters to split once the runs differ anywhere); their number is returned as well."""
    same = np.ones(k, dtype=bool)
    diff = a != ra
    same[a[diff]] = False
    same[ra[diff]] = False
    same &= np.bincount(a, minlength=k) > 0
    num = np.linalg.norm(c[same].astype(np.float64) - rc[same].astype(np.float64), axis=1)
    den = np.linalg.norm(rc[same].astype(np.float64), axis=1) + 1e-30
    rel = num / den
    split_like = (rel >= 1e-5) & (rel < 2.5e-3)
    rest = rel[~split_like]
    return float(same.mean()), float(rest.max()) if rest.size else 0.0, int(split_like.sum())


def _equal_up_to_ties(xr, centroids, knn, rknn):
    """Share of points with the same answer, two answers counting as the same when their float64 distances differ by no
    more than the rounding of the reference's own fp32 formula ||x||^2 + ||c||^2 - 2 x.c (1e-7 of the norms); also the
    raw share and the mask of tied differences."""
    differ = np.nonzero(knn != rknn)[0]
    xs = xr[differ].astype(np.float64)
    ca, cb = centroids[knn[differ]].astype(np.float64), centroids[rknn[differ]].astype(np.float64)
    gap = np.abs(((xs - ca) ** 2).sum(1) - ((xs - cb) ** 2).sum(1))
    tied = gap <= 1e-7 * ((xs ** 2).sum(1) + np.maximum((ca ** 2).sum(1), (cb ** 2).sum(1)))
    return 1.0 - float((~tied).sum()) / len(knn), 1.0 - len(differ) / len(knn), differ, tied


def _flat_against_reference(ref, x, k, seed, iters, replay, end_to_end_agree, classify_cap=150, other_routes=(9, 10)):
    import superkmeans_b200 as skm
    from superkmeans_b200 import engine as eng

    n, d = x.shape
    kw = dict(iters=iters, sampling_fraction=1.0, early_termination=0, seed=seed)
    rk = ref.RefKMeans(k, d, ref.default_config(False, **kw), trace=True)
    rc = rk.train(x)
    m = rk.rotation_matrix()
    trace, stats = rk.trace(), rk.stats()
    hd, vd = eng.dimension_split(d)
    ratios = eng.ratios(d, 1.5)

    # ---- step-wise, from the reference's state
    xr = eng.rotate(m, x)
    rng = np.random.default_rng(1)
    for t in replay:
        prev, cur, st = trace[t - 1], trace[t], stats[t]
        assert not st["is_gemm_only"]
        pd = st["partial_d"]
        rknn, rdist, rnp = ref.find_nearest_pruned(xr, prev.centroids, prev.assign, pd)
        knn, dist, npc = eng.find_nearest_pruned(xr, prev.centroids, prev.assign, pd)
        # Answers that tie within the rounding of the reference's own distances count as equal: the reference forms
        # ||x||^2 + ||c||^2 - 2 x.c in fp32 (batch_computers.h:152-163), which is only good to ~1e-7 of the norms (its
        # reported distances differ from float64 ones by up to 1e-7 on unit rows).  Nearly all such ties are between
        # centroids that coincide to rounding, which several splits of one cluster in one call leave behind
        # (parity_util.coincident_centroids); their count is reported.
        rep = parity_util.coincident_centroids(prev.centroids)
        agree, raw, differ, tied = _equal_up_to_ties(xr, prev.centroids, knn, rknn)
        print(f"iteration {t + 1}: assignments equal {raw:.5f}; {int(tied.sum())} of {len(differ)} differences are ties at the reference's own rounding "
              f"({int((rep[knn[differ]] == rep[rknn[differ]]).sum())} between coincident centroids, {int((rep != np.arange(k)).sum())} such centroids); equal up to ties {agree:.5f}")
        assert agree >= 0.999, (t, agree, raw)
        # the same step through both families of kernels, whichever the automatic choice took: 9 = unordered lists with the
        # dense chain for expensive points, 10 = ordered chain with its candidate replay (what the headline workload runs)
        for route in other_routes:
            eng.set_prune_split(route)
            try:
                knn_o, dist_o, npc_o = eng.find_nearest_pruned(xr, prev.centroids, prev.assign, pd)
            finally:
                eng.set_prune_split(0)
            agree_o, raw_o, _, _ = _equal_up_to_ties(xr, prev.centroids, knn_o, rknn)
            tot_o, rtot = float(npc_o.sum()), float(rnp.sum())
            print(f"iteration {t + 1}, route {route}: assignments equal {raw_o:.5f}, up to ties {agree_o:.5f}, not-pruned total off by {abs(tot_o - rtot) / rtot:.2e}")
            assert agree_o >= 0.999, (t, route, agree_o, raw_o)
            assert abs(tot_o - rtot) <= 5e-3 * rtot + 10, (t, route, tot_o, rtot)
            same_o = knn_o == rknn
            assert np.abs(dist_o[same_o] - rdist[same_o]).max() <= 2e-5 * max(1.0, float(rdist.max()))
        bad = np.nonzero(knn != rknn)[0]
        if len(bad) > classify_cap:
            bad = rng.choice(bad, classify_cap, replace=False)
        sel = np.zeros(n, dtype=bool)
        sel[bad] = True
        a_s = np.where(sel, knn, rknn).astype(np.int64)   # only the sampled disagreements remain
        n_tie, n_flip, unexplained = parity_util.classify_disagreements(xr, prev.centroids, prev.assign.astype(np.int64), a_s, rknn.astype(np.int64), pd, vd, ratios)
        assert not unexplained, (t, n_tie, n_flip, unexplained[:8])
        same = knn == rknn
        assert np.abs(dist[same] - rdist[same]).max() <= 2e-5 * max(1.0, float(rdist.max()))
        tot, rtot = float(npc.sum()), float(rnp.sum())
        assert abs(tot - rtot) <= 5e-3 * rtot + 10, (tot, rtot)
        nd, _ = eng.tune_partial_d(tot, n, k, pd, vd)
        assert nd == cur.partial_d_next
    del xr

    # ---- end to end
    e = skm.Engine(k, d, skm.default_config(False, **kw))
    e.set_rotation(m)
    c = e.train(x)
    es = e.stats(0)
    assert [r["partial_d"] for r in stats] == [s.partial_d for s in es]
    ra, a = rk.assignments(), e.assignments()
    w, rw = _wcss64(x, c, a), _wcss64(x, rc, ra)
    agree = float((ra == a).mean())
    share, rel, n_split_like = _identical_cluster_centroids(e.rotated_centroids(), rk.rotated_centroids(), a, ra, k)
    splits = [(r["split"], s.split) for r, s in zip(stats, es)]
    print(f"end to end: assignments equal {agree:.5f}, clusters with identical members {share:.4f}, their centroids within {rel:.2e} ({n_split_like} apart by a split's scaling), "
          f"wcss rel diff {abs(w - rw) / rw:.2e}, splits (reference, engine) per iteration {splits}")
    assert rel < 1e-5, rel
    assert n_split_like <= 2 * max(1, int(stats[-1]["split"]) + int(es[-1].split)), n_split_like
    # At this size hundreds of clusters are empty after the first iterations (as many centres as clusters, Forgy start):
    # SplitClusters re-seeds them from clusters chosen by size, so one point that falls the other way at a near-tie
    # changes which clusters are split an iteration later, and the runs separate (the reference's own pruned and
    # BLAS-only runs end 0.2 - 0.4 % apart in WCSS on this law).  Every iteration on its own is held to 99.9 % above;
    # end to end the objective is held to 2e-3 and the assignments to the share stated per configuration.
    assert abs(w - rw) <= 2e-3 * rw, (w, rw)
    assert agree >= end_to_end_agree, agree
    return agree


def test_config2_full_size_against_reference(ref):
    x = datagen.config2()
    _flat_against_reference(ref, x, 4096, 7, 10, replay=(1, 2, 9), end_to_end_agree=0.99)


def test_config3_slice_against_reference(ref):
    x = datagen.config3(n=1_000_000)
    # End to end the two runs part ways at the third iteration: the second one splits 1486 empty clusters and leaves 69
    # centroids that coincide with another to rounding; ties between those decide which clusters run empty next (12 splits
    # against 13), and from there the runs descend to different optima of the same quality (WCSS within 1e-3, ~70 % of
    # the points in clusters with the same index).  Assignments are therefore only held to a loose floor here.
    _flat_against_reference(ref, x, 10_000, 123, 10, replay=(1, 2, 9), end_to_end_agree=0.5)


def test_config4_slice_hierarchical_against_reference(ref):
    import superkmeans_b200 as skm

    n, d, k, seed = 1_000_000, 768, 16_384, 2024
    x = datagen.config4(n, d, supers=128, subs=128, seed=seed)
    kw = dict(early_termination=0, seed=seed)
    rk = ref.RefKMeans(k, d, ref.default_config(True, **kw), hierarchical=True)
    rc = rk.train(x)
    e = skm.Engine(k, d, skm.default_config(True, **kw), hierarchical=True)
    e.set_rotation(rk.rotation_matrix())
    c = e.train(x)
    assert e.n_mesoclusters == rk.n_mesoclusters() == 128
    for phase in (1, 2, 3):
        assert len(e.stats(phase)) == len(rk.stats(phase))
    # mesoclustering record by record
    print("mesoclustering (reference objective, engine objective, split):", [(r["objective"], s.objective, r["split"], s.split) for r, s in zip(rk.stats(1), e.stats(1))])
    # The reference adds the 10^6 distances one after the other in fp32 (superkmeans.h:973-981: ~1e-4 of systematic rounding
    # at this size; the engine sums in float64), and the handful of empty-cluster splits of each iteration amplifies
    # single near-ties as in the flat runs: same split counts, objectives within 2e-3.
    for r, s in zip(rk.stats(1), e.stats(1)):
        assert r["partial_d"] == s.partial_d and r["is_gemm_only"] == bool(s.is_gemm_only)
        assert r["split"] == s.split
        assert abs(r["objective"] - s.objective) <= 2e-3 * r["objective"]
    ra, a = rk.final_assignments(), e.assignments()
    # When the last mesoclustering iteration split clusters, the sizes that lay out the mesoclusters' index ranges no longer
    # match the members (hierarchical_superkmeans.h:260-286), some points fall in no range, and the reference leaves their
    # entries of its freshly allocated array unwritten (:121): whatever the heap held.  The engine reports cluster 0 there.
    covered = ra < k
    print(f"hierarchical slice: {int((~covered).sum())} points outside every mesocluster's range (reference entries unwritten)")
    assert (~covered).sum() <= n // 100
    assert a.max() < k
    xc, ra, a = x[covered], ra[covered], a[covered]
    w, rw = _wcss64(xc, c, a), _wcss64(xc, rc, ra)
    del xc
    agree = float((ra == a).mean())
    print(f"hierarchical slice: assignments equal {agree:.5f}, wcss rel diff {abs(w - rw) / rw:.2e}")
    # a mesocluster whose member list differs by one point draws other starting centroids (hierarchical_superkmeans.h:333-342)
    # and ends in another local optimum: the objective is the robust gate (the reference's own bar is 5 %)
    assert abs(w - rw) <= 1e-2 * rw, (w, rw)
    asg = e.assign(x, c)
    atp = e.assign_training_points(x, c)
    assert (atp == asg).mean() >= 0.98


@pytest.mark.parametrize("fraction", [0.9, 0.3])
def test_assign_training_points_of_sampled_models(ref, fraction):
    """AssignTrainingPoints of a model trained on a sample (superkmeans.h:471-504 size-proportional seeds above 0.8,
    :505-563 two-level seeds below): against the reference's own answer, and against brute force at the reference's bar
    (tests/test_assign.cpp:163-201, python/tests/test_superkmeans.py:392-412)."""
    import superkmeans_b200 as skm

    n, d, k, seed = 40_000, 256, 600, 5
    x = datagen.gaussian_mixture(n, d, k, 0.3, seed)
    kw = dict(iters=8, sampling_fraction=fraction, max_points_per_cluster=100_000, early_termination=0, seed=seed, suppress_warnings=1)
    rk = ref.RefKMeans(k, d, ref.default_config(False, **kw))
    rc = rk.train(x)
    e = skm.Engine(k, d, skm.default_config(False, **kw))
    e.set_rotation(rk.rotation_matrix())
    c = e.train(x)
    assert e.n_samples == int(np.floor(np.float32(n) * np.float32(fraction)))
    atp, ratp = e.assign_training_points(x, c), rk.assign_training_points(x, rc)
    brute, rbrute = e.assign(x, c), rk.assign(x, rc)
    assert (atp == brute).mean() >= 0.95
    assert (ratp == rbrute).mean() >= 0.95
    same_model = np.linalg.norm(c - rc) / np.linalg.norm(rc) < 5e-3
    print(f"sampling_fraction {fraction}: fast vs brute force {float((atp == brute).mean()):.4f} (reference {float((ratp == rbrute).mean()):.4f}), same model: {bool(same_model)}")
    if same_model:
        # same model, same seeds, same search: the two fast assignments agree far beyond the 95 % either holds against
        # brute force.  (With 20 points per cluster the two training runs need not end in the same local optimum; the
        # fast assignment of each is then only held to its own brute force.)
        assert (brute == rbrute).mean() >= 0.999
        assert (atp == ratp).mean() >= 0.99, float((atp == ratp).mean())
