"""Worker of tests/test_sharded_cpu.py: one rank of a world-size-N gloo run of the sharded Assign.

Under test are the package's shard split and gather (shard_bounds, assign_sharded, gather_rows); the nearest-centroid
search of each shard is supplied by the CPU oracle because the engine needs a GPU."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class _OracleEngine:
    """Stands in for superkmeans_b200.Engine.assign with the oracle's exact search."""

    def assign(self, vectors, centroids, n=None, on_device=False, out=None):
        from oracle import restate

        knn, _ = restate.find_nearest(np.ascontiguousarray(vectors[:n]), centroids)
        return knn.astype(np.uint32)


def main():
    import torch.distributed as dist

    from superkmeans_b200 import distributed as skd
    from tests import datagen

    out_path, n, d, k, seed = sys.argv[1], *(int(v) for v in sys.argv[2:6])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    x = datagen.gaussian_mixture(n, d, k, 0.3, seed)
    c = np.load(out_path + ".centroids.npy")
    lo, hi = skd.shard_bounds(n, rank, world)
    e = _OracleEngine()
    mine = skd.assign_sharded(e, x[lo:hi], c, hi - lo, n, on_device=False)
    everywhere = skd.assign_sharded(e, x[lo:hi], c, hi - lo, n, on_device=False, gather=True)
    on_last = skd.assign_sharded(e, x[lo:hi], c, hi - lo, n, on_device=False, gather=True, dst=world - 1)
    assert (on_last is None) == (rank != world - 1)
    np.savez(f"{out_path}.rank{rank}.npz", mine=mine, everywhere=everywhere, on_last=on_last if on_last is not None else np.zeros(0, np.uint32), lo=lo, hi=hi)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
