"""Worker of tests/test_sharded_cpu.py: one rank of a world-size-N gloo run of the sharded protocol.

The rank logic under test is the package's own (shard_bounds, make_allreduce through the C callback
type); the k-means arithmetic is supplied by the CPU oracle because the engine needs a GPU."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch.distributed as dist

    from oracle import restate
    from superkmeans_b200 import distributed as skd
    from tests import datagen

    out_path, n, d, k, iters, seed = sys.argv[1], *(int(v) for v in sys.argv[2:7])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    x = datagen.gaussian_mixture(n, d, k, 0.3, seed)
    m = np.load(out_path + ".rotation.npy")
    lo, hi = skd.shard_bounds(n, rank, world)
    reduce = skd.make_allreduce("cpu")
    cent, rcent, assign, stats = restate.train_flat(x, k, m, iters=iters, seed=seed, rows=(lo, hi), reduce=reduce)
    np.savez(f"{out_path}.rank{rank}.npz", cent=cent, assign=assign, lo=lo, hi=hi, objective=np.array([s.objective for s in stats]),
             partial_d=np.array([s.partial_d for s in stats]), split=np.array([s.split for s in stats]))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
