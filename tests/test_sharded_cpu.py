"""Multi-rank path on CPU: world-size-2 (and 3) gloo runs of the sharded training protocol -
contiguous row shards, Forgy rows from the global index space, one sum all-reduce of
[k*d sums | k counts | wcss, not-pruned] per iteration, replicated consolidation."""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from superkmeans_b200 import distributed as skd

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_bounds_partition_rows_evenly():
    for n, world in [(10, 1), (10, 3), (7, 8), (10_000_000, 8), (5, 5)]:
        spans = [skd.shard_bounds(n, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for (a, b), (c, _) in zip(spans, spans[1:]):
            assert b == c
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        skd.shard_bounds(10, 3, 3)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_protocol_matches_single_process(tmp_path, world):
    from oracle import restate
    from superkmeans_b200 import engine as eng
    from tests import datagen

    n, d, k, iters, seed = 6000, 128, 300, 5, 13
    x = datagen.gaussian_mixture(n, d, k, 0.3, seed)
    m = eng.rotation_matrix(d, seed)
    base = str(tmp_path / "run")
    np.save(base + ".rotation.npy", m)
    cent1, _, assign1, stats1 = restate.train_flat(x, k, m, iters=iters, seed=seed)

    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "_gloo_worker.py"), base, str(n), str(d), str(k), str(iters), str(seed)]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]

    ranks = [np.load(f"{base}.rank{r}.npz") for r in range(world)]
    assign = np.concatenate([r["assign"] for r in ranks])
    assert [int(r["lo"]) for r in ranks] == [skd.shard_bounds(n, r, world)[0] for r in range(world)]
    # every rank ends with the same centroids, bit for bit
    for r in ranks[1:]:
        np.testing.assert_array_equal(r["cent"], ranks[0]["cent"])
        np.testing.assert_array_equal(r["partial_d"], ranks[0]["partial_d"])
    # and the sharded run reproduces the single-process run up to the order of the partial sums
    assert list(ranks[0]["partial_d"]) == [s.partial_d for s in stats1]
    assert list(ranks[0]["split"]) == [s.split for s in stats1]
    assert (assign == assign1).mean() >= 0.999
    np.testing.assert_allclose(ranks[0]["objective"], [s.objective for s in stats1], rtol=1e-5)
    assert np.linalg.norm(ranks[0]["cent"] - cent1) <= 1e-4 * np.linalg.norm(cent1)


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_assign_gathers_rows_in_order(tmp_path, world):
    """Assign over row shards (n not a multiple of the world size): the gathered result, on every rank or on one, is the
    single-process assignment."""
    from oracle import restate
    from tests import datagen

    n, d, k, seed = 5003, 64, 97, 21
    x = datagen.gaussian_mixture(n, d, k, 0.3, seed)
    c = x[np.random.default_rng(seed).choice(n, k, replace=False)].copy()
    base = str(tmp_path / "assign")
    np.save(base + ".centroids.npy", c)
    want, _ = restate.find_nearest(x, c)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "_gloo_assign_worker.py"), base, str(n), str(d), str(k), str(seed)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ, OMP_NUM_THREADS="2"), cwd=ROOT)
    assert res.returncode == 0, res.stderr[-2000:]
    ranks = [np.load(f"{base}.rank{r}.npz") for r in range(world)]
    for r, z in enumerate(ranks):
        lo, hi = skd.shard_bounds(n, r, world)
        assert (int(z["lo"]), int(z["hi"])) == (lo, hi)
        np.testing.assert_array_equal(z["mine"], want[lo:hi])
        assert z["everywhere"].dtype == np.uint32
        np.testing.assert_array_equal(z["everywhere"], want)
        assert len(z["on_last"]) == (n if r == world - 1 else 0)
    np.testing.assert_array_equal(ranks[-1]["on_last"], want)


def test_allreduce_callback_through_the_c_callback_type():
    """The closure the engine calls (ptr, count, dtype) sums a host buffer in place; single rank."""
    import ctypes as C

    import torch.distributed as dist

    from superkmeans_b200 import _lib

    if not dist.is_initialized():
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{_free_port()}", rank=0, world_size=1)
    try:
        fn = skd.make_allreduce("cpu")
        cb = _lib.ALLREDUCE_FN(lambda user, buf, count, dtype: (fn(buf, count, dtype), 0)[1])
        for dtype, np_dtype in [(0, np.float32), (1, np.float64), (2, np.int32)]:
            a = np.arange(17, dtype=np_dtype)
            assert cb(None, a.ctypes.data, a.size, dtype) == 0
            np.testing.assert_array_equal(a, np.arange(17, dtype=np_dtype))
    finally:
        dist.destroy_process_group()
