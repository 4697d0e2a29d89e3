"""The C-ABI library loads on a machine without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "skm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = set(re.findall(r"\b(skm_[a-z0-9_]+)\s*\(", text))
    names.discard("skm_allreduce_fn")
    return sorted(names)


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ["skm_create", "skm_train", "skm_assign", "skm_assign_training_points", "skm_destroy",
                 "skm_op_find_nearest", "skm_op_find_nearest_pruned", "skm_op_update_centroids"]:
        assert must in names


def test_library_exports_every_declared_symbol():
    from superkmeans_b200 import _lib

    lib = ctypes.CDLL(_lib.LIB_PATH)
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing
    # and the Python binding table covers the same set
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_engine_refuses_to_run_without_a_gpu():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import superkmeans_b200 as skm

    with pytest.raises(RuntimeError, match="no CPU path"):
        skm.Engine(16, 64)


def test_constructor_validation_matches_reference_exception_classes():
    # superkmeans.h:125-131: non-positive values and sampling_fraction > 1 are invalid_argument.
    import superkmeans_b200 as skm

    for kw in [dict(iters=0), dict(sampling_fraction=0.0), dict(sampling_fraction=1.5)]:
        cfg = skm.default_config(False, **kw)
        with pytest.raises(ValueError):
            skm.Engine(16, 64, cfg)
    with pytest.raises(ValueError):
        skm.Engine(0, 64)
    with pytest.raises(ValueError):
        skm.Engine(16, 0)
    cfg = skm.default_config(True, iters_mesoclustering=0)
    with pytest.raises(ValueError):
        skm.Engine(16, 64, cfg, hierarchical=True)
    with pytest.raises(ValueError):
        skm.SuperKMeans(0, 8)
    with pytest.raises(ValueError):
        skm.SuperKMeans(8, 8, sampling_fraction=1.5)
