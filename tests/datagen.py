"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations
(they stand in for the public embedding sets the reference is benchmarked on)."""
from __future__ import annotations

import numpy as np


def _normalize(x: np.ndarray) -> np.ndarray:
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return x


def gaussian_mixture(n: int, d: int, centers: int, noise: float, seed: int, normalize: bool = True, center_std=None,
                     zipf_s: float = 0.0) -> np.ndarray:
    """Points = centre + N(0, noise^2); centres N(0, center_std^2) per dimension; optional Zipf sizes."""
    rng = np.random.default_rng(seed)
    scale = np.ones(d, dtype=np.float32) if center_std is None else np.asarray(center_std, dtype=np.float32)
    c = rng.standard_normal((centers, d), dtype=np.float32) * scale
    if zipf_s > 0:
        w = np.arange(1, centers + 1, dtype=np.float64) ** (-zipf_s)
        sizes = np.maximum(1, np.floor(w / w.sum() * n)).astype(np.int64)
        sizes[0] += n - sizes.sum()
        labels = np.repeat(np.arange(centers), sizes)
        rng.shuffle(labels)
    else:
        labels = rng.integers(0, centers, size=n)
    x = c[labels] + rng.standard_normal((n, d), dtype=np.float32) * (noise * scale)
    x = x.astype(np.float32)
    return _normalize(x) if normalize else x


def config1(n=100_000, d=768, k=1000, seed=42):
    return gaussian_mixture(n, d, k, 0.3, seed)


def config2(n=1_000_000, d=1536, k=4096, seed=7):
    s = 1.0 / np.sqrt(1.0 + np.arange(d) / 64.0)
    return gaussian_mixture(n, d, k, 0.3, seed, center_std=s)


def config3(n=10_000_000, d=1024, k=10_000, seed=123):
    return gaussian_mixture(n, d, k, 0.25, seed, zipf_s=1.1)


def config4(n, d=768, supers=256, subs=256, seed=2024):
    rng = np.random.default_rng(seed)
    sc = rng.standard_normal((supers, d), dtype=np.float32)
    sub = sc[:, None, :] + 0.2 * rng.standard_normal((supers, subs, d), dtype=np.float32)
    sub = sub.reshape(supers * subs, d)
    labels = rng.integers(0, supers * subs, size=n)
    x = sub[labels] + 0.1 * rng.standard_normal((n, d), dtype=np.float32)
    return _normalize(x.astype(np.float32))


def config5(n, d=384, k=16384, seed=99):
    rng = np.random.default_rng(seed)
    c = _normalize(rng.standard_normal((k, d), dtype=np.float32))
    labels = rng.integers(0, k, size=n)
    x = c[labels] + 0.3 * rng.standard_normal((n, d), dtype=np.float32)
    return _normalize(x.astype(np.float32)), c
