"""Host-side decisions of the path, checked on CPU against the compiled reference (oracle/_ref) and
against the known answers of the reference's own tests."""
import numpy as np
import pytest

from superkmeans_b200 import engine as eng

DIMS = [1, 2, 4, 8, 16, 32, 48, 63, 64, 65, 127, 128, 129, 130, 191, 192, 193, 255, 256, 257, 384, 512, 600, 768, 900, 1024,
        1536, 2048, 3072, 4096]


def test_dimension_split_invariants():
    # tests/test_pdx_layout.cpp:61-108
    for d in DIMS:
        h, v = eng.dimension_split(d)
        assert h + v == d
        assert h % 64 == 0
        if d <= 64:
            assert (h, v) == (0, d)
    for d in [64, 128, 256, 512, 768, 1024, 2048, 4096]:
        assert eng.dimension_split(d)[1] > 0
    assert eng.dimension_split(384) == (320, 64)
    assert eng.dimension_split(768) == (576, 192)
    assert eng.dimension_split(1024) == (768, 256)
    assert eng.dimension_split(1536) == (1152, 384)


def test_dimension_split_matches_reference(ref):
    for d in DIMS:
        assert eng.dimension_split(d) == ref.dimension_split(d), d


def test_ratios_match_reference(ref):
    for d, eps, hier in [(128, 1.5, False), (768, 1.5, False), (1024, 1.1, True)]:
        km = ref.RefKMeans(300, d, ref.default_config(hier), hierarchical=hier)
        np.testing.assert_array_equal(eng.ratios(d, eps), km.ratios())


def test_pdx_offsets_match_reference_layout(ref):
    # tests/test_pdx_layout.cpp:116-163: every element is addressable, including the partial chunk.
    rng = np.random.default_rng(0)
    for n, d in [(2 * 1024 + 17, 128), (1500, 384), (1024, 256), (700, 130)]:
        x = rng.standard_normal((n, d), dtype=np.float32)
        p = ref.pdxify(x).ravel()
        rows = rng.integers(0, n, 400)
        dims = rng.integers(0, d, 400)
        for r, j in zip(rows, dims):
            assert p[eng.pdx_offset(int(r), int(j), n, d)] == x[r, j]


def test_rotation_matrix_is_orthonormal_and_seeded():
    # tests/test_rotation.cpp: orthonormality and seed determinism
    m = eng.rotation_matrix(96, 7)
    assert np.abs(m @ m.T - np.eye(96)).max() < 1e-5
    np.testing.assert_array_equal(m, eng.rotation_matrix(96, 7))
    assert np.abs(m - eng.rotation_matrix(96, 8)).max() > 1e-2


def test_rotation_matrix_close_to_reference(ref):
    # Same Gaussian draws and Householder sign convention: equal up to rounding.
    d = 64
    km = ref.RefKMeans(10, d, ref.default_config(False, seed=5))
    assert np.abs(km.rotation_matrix() - eng.rotation_matrix(d, 5)).max() < 1e-4


@pytest.fixture(scope="module")
def flat_trace(ref):
    from tests import datagen

    n, d, k = 6000, 128, 300
    x = datagen.gaussian_mixture(n, d, k, 0.3, 3)
    cfg = ref.default_config(False, iters=6, sampling_fraction=1.0, early_termination=0, seed=11)
    km = ref.RefKMeans(k, d, cfg, trace=True)
    km.train(x)
    return n, k, km.trace(), km.stats(), 11


def test_split_clusters_replays_reference(flat_trace):
    n, k, trace, stats, seed = flat_trace
    assert any((s.sizes_pre == 0).any() for s in trace), "the fixture must exercise empty clusters"
    for snap, st in zip(trace, stats):
        sizes, ops, n_split = eng.split_clusters(snap.sizes_pre, n, seed, hierarchical=False)
        np.testing.assert_array_equal(sizes, snap.sizes_post)
        assert n_split == st["split"]
        assert len(ops) == n_split


def test_split_clusters_hierarchical_replays_reference(ref):
    from tests import datagen

    n, d, k = 8000, 64, 400
    x = datagen.gaussian_mixture(n, d, 50, 0.3, 4)
    cfg = ref.default_config(True, iters_mesoclustering=3, iters_fineclustering=3, early_termination=0, seed=9)
    km = ref.RefKMeans(k, d, cfg, hierarchical=True, trace=True)
    km.train(x)
    trace = km.trace()
    stats = km.stats(1) + km.stats(2)
    assert len(trace) == len(stats)
    n_balanced = 0
    for snap, st in zip(trace, stats):
        sizes, ops, n_split = eng.split_clusters(snap.sizes_pre, snap.n_samples, 9, hierarchical=True)
        np.testing.assert_array_equal(sizes, snap.sizes_post)
        assert n_split == st["split"]
        n_balanced += int((ops[:, 2] == 1).sum()) if len(ops) else 0
    assert n_balanced > 0, "the fixture must exercise the balancing branch"


def test_tune_partial_d_replays_reference(flat_trace):
    n, k, trace, stats, _ = flat_trace
    v = eng.dimension_split(128)[1]
    seen = 0
    for i, st in enumerate(stats):
        if st["is_gemm_only"]:
            continue
        total = round(st["not_pruned_pct"] * n * k)
        nd, avg = eng.tune_partial_d(float(total), n, k, st["partial_d"], v)
        assert nd == trace[i].partial_d_next
        assert abs(avg - st["not_pruned_pct"]) < 1e-6
        seen += 1
    assert seen >= 3


def test_tune_partial_d_bounds():
    assert eng.tune_partial_d(1e9, 1000, 1000, 250, 256)[0] == 256       # capped at vertical_d
    assert eng.tune_partial_d(0.0, 1000, 1000, 17, 256)[0] == 16          # floored at MIN_PARTIAL_D
    assert eng.tune_partial_d(0.04 * 1e6, 1000, 1000, 100, 256)[0] == 100  # inside the 3-5 % band
    assert eng.tune_partial_d(0.06 * 1e6, 1000, 1000, 100, 256)[0] == 140
    assert eng.tune_partial_d(0.01 * 1e6, 1000, 1000, 100, 256)[0] == 80


def test_arrange_fine_clusters():
    sizes = np.array([100, 0, 300, 600], dtype=np.uint32)
    out = eng.arrange_fine_clusters(100, 1000, sizes)
    assert out.sum() == 100 and out[1] == 0 and (out[[0, 2, 3]] >= 1).all()
    assert list(out) == [10, 0, 30, 60]
    # every non-empty mesocluster gets at least one cluster even when k is tiny
    out = eng.arrange_fine_clusters(3, 1000, np.array([1, 1, 998], dtype=np.uint32))
    assert list(out) == [1, 1, 1]


def test_forgy_indices_are_a_seeded_sample_without_replacement():
    a = eng.forgy_indices(1000, 50, 42)
    assert len(set(a.tolist())) == 50 and a.max() < 1000
    np.testing.assert_array_equal(a, eng.forgy_indices(1000, 50, 42))
    assert (a != eng.forgy_indices(1000, 50, 43)).any()


def test_dct_rotation_matrix_is_the_orthonormal_dct_of_sign_flipped_rows():
    """adsampling.h:53-73, :169-188: out = DCT-II(x * signs), FFTW REDFT10 scaled to be orthonormal."""
    import scipy.fft

    from superkmeans_b200 import engine as eng

    for d, seed in ((512, 42), (1024, 7), (64, 3)):
        m = eng.dct_rotation_matrix(d, seed).astype(np.float64)
        assert np.abs(m @ m.T - np.eye(d)).max() < 1e-6
        signs = m[0] / np.abs(m[0])          # row 0 of the DCT is constant, so it shows the signs
        assert set(np.unique(signs)) <= {-1.0, 1.0} and 0.3 < (signs > 0).mean() < 0.7
        x = np.random.default_rng(seed).standard_normal((5, d))
        want = scipy.fft.dct(x * signs, type=2, norm="ortho", axis=1)
        assert np.abs(x @ m.T - want).max() < 1e-5
