"""N shards against one GPU on real devices (needs at least two): sharded training through the NCCL communicator inside
the library, and through the torch.distributed callback, must reproduce the unsharded run - same d' schedule and split
counts, objectives within fp32 summation noise, the same assignments up to near-ties."""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(world, mode):
    import torch

    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port", "29517",
           os.path.join(ROOT, "tests", "_nccl_worker.py"), mode]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


@pytest.mark.parametrize("mode", ["nccl", "callback"])
def test_two_shards_reproduce_the_single_gpu_run(mode):
    r = _run(2, mode)
    assert r["all_ranks_same_centroids"]
    assert r["partial_d_equal"] and r["split_equal"], r
    assert r["objective_rel_diff"] <= 1e-5, r
    assert r["assignments_equal"] >= 0.999, r
    assert r["centroid_max_abs_diff"] <= 1e-3, r
