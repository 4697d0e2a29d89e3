"""Generates tests/golden/*.npz from the compiled reference (oracle/_ref).  Run where the reference
sources exist:  make -C oracle ref && python tests/golden/make_golden.py

The fixtures let the oracle restatement and the CUDA engine be checked against reference OUTPUTS on
machines where the reference itself is not available."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import ref  # noqa: E402
from tests import datagen  # noqa: E402

DIMS = [1, 2, 4, 8, 16, 32, 48, 63, 64, 65, 127, 128, 129, 130, 191, 192, 193, 255, 256, 257, 384, 512, 600, 768, 900, 1024, 1536, 2048, 3072, 4096]


def micro():
    splits = np.array([ref.dimension_split(d) for d in DIMS], dtype=np.int64)
    rng = np.random.default_rng(0)
    # the input is its own index map (exact in float32), so only the output needs storing
    y = np.arange((1024 + 77) * 192, dtype=np.float32).reshape(1024 + 77, 192)
    a = rng.standard_normal(333, dtype=np.float32)
    b = rng.standard_normal(333, dtype=np.float32)
    hor = np.array([ref.horizontal(a[:m], b[:m]) for m in (1, 15, 16, 17, 64, 100, 333)], dtype=np.float32)
    km = ref.RefKMeans(300, 768, ref.default_config(False))
    kh = ref.RefKMeans(300, 1024, ref.default_config(True), hierarchical=True)
    np.savez_compressed(os.path.join(HERE, "micro.npz"), dims=np.array(DIMS), splits=splits, pdx_shape=np.array(y.shape), pdx_out=ref.pdxify(y), hor_a=a, hor_b=b, hor=hor,
                        ratios_768_eps15=km.ratios(), ratios_1024_eps11=kh.ratios())


def flat_run(name, n, d, k, iters, seed, **kw):
    x = datagen.gaussian_mixture(n, d, k, 0.3, seed)
    cfg = ref.default_config(False, iters=iters, sampling_fraction=1.0, early_termination=0, seed=seed, **kw)
    km = ref.RefKMeans(k, d, cfg, trace=True)
    cent = km.train(x)
    tr, st = km.trace(), km.stats()
    np.savez_compressed(
        os.path.join(HERE, name), x=x, rotation=km.rotation_matrix(), centroids=cent, rotated_centroids=km.rotated_centroids(),
        assign=np.stack([s.assign for s in tr]), dist=np.stack([s.dist for s in tr]), sizes_pre=np.stack([s.sizes_pre for s in tr]),
        sizes_post=np.stack([s.sizes_post for s in tr]), partial_d_next=np.array([s.partial_d_next for s in tr]),
        objective=np.array([s["objective"] for s in st], dtype=np.float32), shift=np.array([s["shift"] for s in st], dtype=np.float32),
        split=np.array([s["split"] for s in st]), partial_d=np.array([s["partial_d"] for s in st]), not_pruned_pct=np.array([s["not_pruned_pct"] for s in st], dtype=np.float32),
        is_gemm_only=np.array([s["is_gemm_only"] for s in st]), meta=np.array([n, d, k, iters, seed]),
        assign_brute=km.assign(x, cent), assign_fast=km.assign_training_points(x, cent),
    )


if __name__ == "__main__":
    micro()
    flat_run("flat_pruned.npz", 2500, 128, 300, 6, 21)
    flat_run("flat_gemm_only.npz", 2000, 64, 40, 5, 22)
    print("written:", [f for f in os.listdir(HERE) if f.endswith(".npz")])
