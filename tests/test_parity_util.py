"""The helpers that judge parity are themselves checked on constructed cases (CPU only)."""
import numpy as np

from tests import parity_util


def test_coincident_centroids_groups_what_repeated_splits_leave_behind():
    # SplitClusters (superkmeans.h:905-920): copy * (1 + e s), source * (1 - e s), e = 1/1024, s alternating.  A copy that is
    # split again returns to (1 - e^2) times the original: it coincides, up to rounding, with the copy made right after the
    # source's first scaling, and with nothing else.
    rng = np.random.default_rng(3)
    k, d, e = 500, 128, np.float32(1.0 / 1024.0)
    y = rng.standard_normal((k, d)).astype(np.float32)
    s = np.where(np.arange(d) % 2 == 0, np.float32(1), np.float32(-1))
    up, down = (np.float32(1) + e * s).astype(np.float32), (np.float32(1) - e * s).astype(np.float32)
    b0 = y[10].copy()
    y[20] = b0 * up                 # first split of cluster 10: copy 20
    y[10] = b0 * down
    y[30] = y[10] * up              # second split of cluster 10: copy 30 = b0 (1 - e^2)
    y[10] = y[10] * down
    y[40] = y[20] * up              # copy 20 is split itself: it falls back to b0 (1 + e s)(1 - e s) = b0 (1 - e^2)
    y[20] = y[20] * down
    rep = parity_util.coincident_centroids(y)
    assert rep[30] == rep[20] == 20          # the pair that coincides, named by its smaller index
    others = np.delete(np.arange(k), [30])
    assert (rep[others] == others).all()     # ordinary twins (apart by e) are not merged
    assert float(((y[30].astype(np.float64) - y[20]) ** 2).sum()) <= 1e-11 * float((y[20].astype(np.float64) ** 2).sum())


def test_classifier_accepts_ties_and_rejects_a_plainly_wrong_answer():
    rng = np.random.default_rng(5)
    n, k, d = 64, 40, 256
    y = rng.standard_normal((k, d)).astype(np.float32)
    x = (y[rng.integers(0, k, n)] + 0.1 * rng.standard_normal((n, d))).astype(np.float32)
    dist = ((x[:, None, :].astype(np.float64) - y[None].astype(np.float64)) ** 2).sum(2)
    best = dist.argmin(1)
    prev = best.copy()
    ratios = np.ones(d + 1, dtype=np.float32) * 4.0   # no test ever prunes
    ratios[d] = 1.0
    a, b = best.copy(), best.copy()
    # a tie: a second centroid made equal to the winner of point 0 up to one part in 1e8
    y2 = y.copy()
    y2[(best[0] + 1) % k] = y[best[0]] * np.float32(1 + 1e-8)
    a[0] = (best[0] + 1) % k
    n_tie, n_flip, unexplained = parity_util.classify_disagreements(x, y2, prev, a, b, 128, 192, ratios)
    assert unexplained == [] and n_tie == 1
    # a wrong answer: the farthest centroid
    a = best.copy()
    a[1] = dist[1].argmax()
    _, _, unexplained = parity_util.classify_disagreements(x, y, prev, a, b, 128, 192, ratios)
    assert [int(u) if not isinstance(u, (tuple, list)) else int(u[0]) for u in unexplained] == [1]
