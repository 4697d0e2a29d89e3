"""Helpers shared by the parity tests: classification of the points on which two implementations of the pruned
search (BatchComputer::FindNearestNeighborWithPruning, batch_computers.h:297-409) disagree.

Both implementations run the same approximate search: a candidate is dropped as soon as its partial distance over the
dimensions seen so far is not below best * ratio[dimensions seen] (pdx/pdxearch.h:67-80).  Two fp32 evaluations of
that search can legitimately differ on a point in exactly two ways:
  * near-tie: the two answers are equally good: float64 distances within 1e-5 relative, or within the rounding of the
    reference's own distance formula ||x||^2 + ||c||^2 - 2 x.c (batch_computers.h:152-163), which is about 1e-7 of the
    norms whatever the distance (twin centroids left by a split sit that close);
  * threshold flip: the better answer sat within fp32 rounding of one of its thresholds, so one side dropped it
    (an ADSampling false prune) and the other kept it.
Everything else would be a bug.  `classify_disagreements` replays the search of the affected points in float64 and
returns the points that fit neither case.  Points that the quick check (was the better answer itself near one of its
thresholds?) does not explain get the full treatment: `reachable_answers` replays the whole search and follows BOTH
outcomes of every test that is within rounding of its threshold (an earlier candidate that one side kept and the other
dropped changes `best`, and with it every later threshold); the disagreement is explained when both answers can be
reached that way."""
from __future__ import annotations

import numpy as np

CHUNK = 1024     # VECTOR_CHUNK_SIZE (common.h:89-115)
HBLOCK = 64      # H_DIM_SIZE


def _checkpoints(d, partial_d, vertical_d):
    """[(dims of the segment, ratio index after it)] in the order of PDXearch::Prune (pdxearch.h:149-216)."""
    segs = [(np.arange(0, partial_d), partial_d)]
    seen = partial_d
    for h0 in range(vertical_d, d, HBLOCK):
        seen += HBLOCK
        segs.append((np.arange(h0, min(h0 + HBLOCK, d)), seen))
    if partial_d < vertical_d:
        segs.append((np.arange(partial_d, vertical_d), d))
    return segs


def reachable_answers(xi, y64, prev_i, segs, r, thr_tol, tie_abs, max_states=64):
    """Final answers (centroid indices) that the chunk-by-chunk search can end with when every test whose partial
    distance is within thr_tol * (|x|^2 + |c|^2 over the dimensions seen) of its threshold, and every final comparison
    within tie_abs of `best`, may fall either way.  Follows the reference's order: `best` is fixed inside a chunk of
    1024 centroids and lowered at its end (pdxearch.h:290-324); the previous centroid as the only survivor of the first
    test leaves it untouched (:140-143)."""
    k = y64.shape[0]
    best0 = float(((xi - y64[prev_i]) ** 2).sum())
    states = {(best0, int(prev_i))}
    for lo in range(0, k, CHUNK):
        hi = min(lo + CHUNK, k)
        yc = y64[lo:hi]
        diff2 = (xi[None, :] - yc) ** 2
        x2, y2 = xi ** 2, yc ** 2
        pds, scales = [], []
        pd = np.zeros(hi - lo)
        sc = np.zeros(hi - lo)
        for dims, seen in segs:
            pd = pd + diff2[:, dims].sum(1)
            sc = sc + x2[dims].sum() + y2[:, dims].sum(1)
            pds.append(pd)
            scales.append(sc)
        nxt = set()
        for best, bidx in states:
            sure = np.ones(hi - lo, dtype=bool)      # passes every test beyond doubt
            maybe = np.ones(hi - lo, dtype=bool)     # passes every test when the doubtful ones fall its way
            for s, (dims, seen) in enumerate(segs):
                thr = best * r[seen]
                slack = thr_tol * scales[s]
                sure &= pds[s] < thr - slack
                maybe &= pds[s] < thr + slack
                if s == 0:
                    first_sure, first_maybe = sure.copy(), maybe.copy()
            final = pds[-1]
            win_sure = sure & (final < best - tie_abs)
            win_maybe = maybe & (final < best + tie_abs)
            # the rule for "the previous centroid is the only survivor of the first test": may apply when the counts allow it
            p_in = lo <= prev_i < hi
            only_prev_possible = p_in and first_maybe[prev_i - lo] and int(first_sure.sum() - (1 if first_sure[prev_i - lo] else 0)) == 0
            only_prev_certain = p_in and first_sure[prev_i - lo] and int(first_maybe.sum()) == 1
            outcomes = set()
            if only_prev_possible or not win_maybe.any():
                outcomes.add((best, bidx))
            if not only_prev_certain and win_maybe.any():
                idx = np.nonzero(win_maybe)[0]
                floor = final[win_sure].min() if win_sure.any() else np.inf
                if win_sure.any():
                    j = idx[np.argmin(np.where(win_sure[idx], final[idx], np.inf))]
                    outcomes.add((float(final[j]), int(lo + j)))
                else:
                    outcomes.add((best, bidx))   # none of the doubtful ones made it
                for j in idx:
                    if not win_sure[j] and final[j] <= floor + tie_abs:
                        outcomes.add((float(final[j]), int(lo + j)))
                    elif win_sure[j] and final[j] <= floor + tie_abs:
                        outcomes.add((float(final[j]), int(lo + j)))
            nxt |= outcomes
        if len(nxt) > max_states:
            nxt = set(sorted(nxt)[:max_states])
        states = nxt
    return {b for _, b in states}


def classify_disagreements(x, y, prev, a, b, partial_d, vertical_d, ratios, tie_rel=1e-5, tie_norm=1e-6, thr_tol=2e-5, margins=None):
    """x [n][d] rotated points, y [k][d] rotated centroids, prev the assignment the pass started from, a / b the two
    answers.  Returns (n_near_ties, n_threshold_flips, unexplained indices).

    thr_tol: how close (relative to ||x||^2 + ||c||^2 over the dimensions seen) a partial distance must have been to
    its threshold for a flip to count as rounding; the tensor-core accumulator is accurate to about 1e-5 of that scale."""
    idx = np.nonzero(a != b)[0]
    n_tie = n_flip = 0
    bad = []
    d = x.shape[1]
    segs = _checkpoints(d, partial_d, vertical_d)
    r = np.asarray(ratios, dtype=np.float64)
    y64 = None
    for i in idx:
        xi = x[i].astype(np.float64)
        da = float(((xi - y[a[i]].astype(np.float64)) ** 2).sum())
        db = float(((xi - y[b[i]].astype(np.float64)) ** 2).sum())
        norms = float((xi ** 2).sum()) + float((y[a[i]].astype(np.float64) ** 2).sum())
        if abs(da - db) <= tie_rel * max(min(da, db), 1e-30) + tie_norm * norms:
            n_tie += 1
            continue
        w = int(a[i]) if da < db else int(b[i])   # the better answer: the other side must have dropped it
        if w == int(prev[i]):
            # the previous centroid is never dropped (its distance is the threshold): preferring a worse centroid to
            # it cannot come from a threshold
            bad.append(int(i))
            continue
        if y64 is None:
            y64 = y.astype(np.float64)
        # float64 replay of the chunks before w's chunk gives the running best that w was tested against
        best = float(((xi - y64[prev[i]]) ** 2).sum())
        wc = w // CHUNK
        closest = np.inf
        for c in range(wc + 1):
            lo, hi = c * CHUNK, min((c + 1) * CHUNK, y.shape[0])
            diff2 = (xi[None, :] - y64[lo:hi]) ** 2
            alive = np.ones(hi - lo, dtype=bool)
            pd = np.zeros(hi - lo)
            n_first = 0
            for s, (dims, seen) in enumerate(segs):
                pd = pd + diff2[:, dims].sum(1)
                thr = best * r[seen]
                if c == wc:
                    cols = np.concatenate([sg[0] for sg in segs[: s + 1]])
                    scale = float((xi[cols] ** 2).sum() + (y64[w, cols] ** 2).sum())
                    closest = min(closest, abs(pd[w - lo] - thr) / max(scale, 1e-30))
                alive &= pd < thr
                if s == 0:
                    n_first = int(alive.sum())
                    prev_only = n_first == 1 and lo <= prev[i] < hi and alive[prev[i] - lo]
            if c < wc and alive.any() and not prev_only:
                best = float(pd[alive].min())
        if margins is not None:
            margins.append(closest)
        if closest <= thr_tol:
            n_flip += 1
            continue
        reach = reachable_answers(xi, y64, int(prev[i]), segs, r, thr_tol, tie_rel * min(da, db) + tie_norm * norms)
        if int(a[i]) in reach and int(b[i]) in reach:
            n_flip += 1
        else:
            bad.append(int(i))
    return n_tie, n_flip, bad


def coincident_centroids(y, rel=1e-11):
    """Representative (smallest index) of every group of centroids that coincide: squared distance <= rel * squared norm.

    Such groups are left by SplitClusters (superkmeans.h:890-928) when one cluster is the source of several splits in one
    call: the source is scaled by (1 - e s) each time and the copy by (1 + e s) (e = 1/1024, s = +-1 alternating over the
    dimensions), so a copy that is itself split later returns to (1 + e s)(1 - e s) = 1 - e^2 times the original, the same
    vector as the copy made right after the source's first scaling, up to the rounding of the products.  A point near such
    a pair sees two distances that differ by ~1e-8 relative: which one an fp32 search reports is rounding, in the
    reference as much as here, so parity is counted up to these groups."""
    y64 = np.asarray(y, dtype=np.float64)
    k = y64.shape[0]
    nn = (y64 ** 2).sum(1)
    proj = y64 @ np.random.default_rng(0).standard_normal(y64.shape[1])
    order = np.argsort(proj, kind="stable")
    parent = np.arange(k)

    def find(i):
        while parent[i] != i:
            parent[i] = parent[parent[i]]
            i = parent[i]
        return i

    sp = proj[order]
    scale = np.sqrt(nn[order]) + 1e-30
    for a in range(k - 1):
        b = a + 1
        # |projection difference| <= |r| * |difference|: a generous window, the exact check decides
        while b < k and sp[b] - sp[a] <= 1e-3 * scale[a]:
            i, j = order[a], order[b]
            if ((y64[i] - y64[j]) ** 2).sum() <= rel * max(nn[i], nn[j]):
                ri, rj = find(i), find(j)
                if ri != rj:
                    parent[max(ri, rj)] = min(ri, rj)
            b += 1
    return np.array([find(i) for i in range(k)])
