"""Worker of tests/test_multi_gpu.py (one process per GPU, started by torch.distributed.run): the same data set trained
in shards with the sums done by NCCL inside the library, and whole on rank 0; prints one JSON line on rank 0."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import superkmeans_b200 as skm  # noqa: E402
from superkmeans_b200 import distributed as skd  # noqa: E402
from tests import datagen  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    use_callback = len(sys.argv) > 1 and sys.argv[1] == "callback"
    n, d, k, seed = 60_000, 256, 700, 11
    x = datagen.gaussian_mixture(n, d, k, 0.3, seed)   # every rank draws the same data and keeps its rows
    lo, hi = skd.shard_bounds(n, rank, world)
    cfg = dict(iters=6, sampling_fraction=1.0, early_termination=0, seed=seed)
    rot = skm.engine.rotation_matrix(d, seed)
    e = skm.Engine(k, d, skm.default_config(False, **cfg), device=local)
    e.set_rotation(rot)
    comm = None
    if use_callback:
        e.set_shard(n, lo, skd.make_allreduce(torch.device("cuda", local)))
    else:
        comm = skd.make_comm(local)
        e.set_shard_comm(n, lo, comm)
    c = e.train(np.ascontiguousarray(x[lo:hi]))
    out = None
    if rank == 0:
        e1 = skm.Engine(k, d, skm.default_config(False, **cfg), device=local)
        e1.set_rotation(rot)
        c1 = e1.train(x)
        s, s1 = e.stats(0), e1.stats(0)
        out = {
            "world": world, "sums": "callback" if use_callback else "nccl",
            "partial_d_equal": [q.partial_d for q in s] == [q.partial_d for q in s1],
            "split_equal": [q.split for q in s] == [q.split for q in s1],
            "objective_rel_diff": max(abs(a.objective - b.objective) / b.objective for a, b in zip(s, s1)),
            "centroid_max_abs_diff": float(np.abs(c - c1).max()),
            "assignments_equal": float((e.assignments() == e1.assignments()[lo:hi]).mean()),
            "allreduce_ms": e.phase_times()["allreduce"][0],
        }
    # all ranks hold the same centroids
    t = torch.from_numpy(c).cuda()
    ref_t = t.clone()
    dist.broadcast(ref_t, src=0)
    same = bool(torch.equal(t, ref_t))
    flags = [None] * world
    dist.all_gather_object(flags, same)
    if rank == 0:
        out["all_ranks_same_centroids"] = all(flags)
        print("RESULT " + json.dumps(out), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
