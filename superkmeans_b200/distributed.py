"""Sharded training: one process per GPU, rows split evenly, one sum all-reduce per iteration.

`torch.distributed` is used for the plumbing only (process group, NCCL over NVLink).  The engine
calls back into `make_allreduce(...)`'s closure with a raw buffer pointer; the closure wraps it
zero-copy in a tensor and runs `dist.all_reduce`.  With the gloo backend the same closure works on
host buffers, which is how the protocol is tested without GPUs.
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Tuple

import numpy as np

_DTYPES = {0: ("<f4", np.float32, 4), 1: ("<f8", np.float64, 8), 2: ("<i4", np.int32, 4)}


def shard_bounds(n: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous, even split of [0, n): the first n % world ranks hold one extra row."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank/world out of range")
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class _CudaView:
    def __init__(self, ptr: int, count: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False), "version": 2}


def make_allreduce(device, group=None) -> Callable[[int, int, int], None]:
    """Returns fn(ptr, count, dtype) that sums the buffer across the process group in place."""
    import torch
    import torch.distributed as dist

    dev = torch.device(device)

    def fn(ptr: int, count: int, dtype: int) -> None:
        typestr, np_dtype, size = _DTYPES[dtype]
        if dev.type == "cuda":
            t = torch.as_tensor(_CudaView(ptr, count, typestr), device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
            torch.cuda.synchronize(dev)
        else:
            buf = (C.c_char * (count * size)).from_address(ptr)
            t = torch.from_numpy(np.frombuffer(buf, dtype=np_dtype))
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)

    return fn


def make_comm(device_index: int, group=None):
    """An NCCL communicator inside the library for the ranks of `group` (default: all ranks): rank 0 draws the unique id,
    torch.distributed carries it to the others (any backend), every rank joins.  The per-iteration sums then run on the
    engine's own stream without a callback into Python."""
    import torch.distributed as dist

    from .engine import Comm

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    box = [Comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    return Comm(box[0], rank, world, device_index)


def train_sharded(engine, local_rows, n_local: int, n_global: int, row_offset: int, device, on_device: bool = True, group=None, comm=None):
    """Trains `engine` on this rank's rows; every rank returns the same centroids.  With `comm` (make_comm) the sums go
    through NCCL inside the library, else through torch.distributed."""
    if comm is not None:
        engine.set_shard_comm(n_global, row_offset, comm)
    else:
        engine.set_shard(n_global, row_offset, make_allreduce(device, group))
    return engine.train(local_rows, n=n_local, on_device=on_device)


def gather_rows(local, n_global: int, group=None, dst=None):
    """Concatenates the ranks' contiguous shards (split as `shard_bounds`) of a per-row result in rank order.  `local` is
    a 1-d numpy array or torch tensor (host or device); the result has `n_global` entries and lives where `local` does.
    With `dst` only that rank receives it (the others get None).  Shards differ by at most one row, so every rank sends
    `ceil(n_global / world)` entries and the padding is cut on arrival."""
    import torch
    import torch.distributed as dist

    rank, world = dist.get_rank(group), dist.get_world_size(group)
    lo, hi = shard_bounds(n_global, rank, world)
    as_numpy = isinstance(local, np.ndarray)
    np_dtype = local.dtype if as_numpy else None
    if as_numpy and np_dtype == np.uint32:   # carried as int32: the collectives have no unsigned 32-bit type
        local = local.view(np.int32)
    t = torch.from_numpy(np.ascontiguousarray(local)) if as_numpy else local.contiguous()
    if t.dim() != 1 or t.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} holds rows [{lo}, {hi}) but passed {tuple(t.shape)} entries")
    width = -(-n_global // world)
    send = torch.zeros(width, dtype=t.dtype, device=t.device)
    send[: hi - lo] = t
    if dst is None:
        parts = [torch.empty_like(send) for _ in range(world)]
        dist.all_gather(parts, send, group=group)
    else:
        parts = [torch.empty_like(send) for _ in range(world)] if rank == dst else None
        dist.gather(send, parts, dst=dist.get_global_rank(group, dst) if group is not None else dst, group=group)
        if rank != dst:
            return None
    sizes = [shard_bounds(n_global, r, world) for r in range(world)]
    out = torch.cat([p[: b - a] for p, (a, b) in zip(parts, sizes)])
    return out.numpy().view(np_dtype) if as_numpy else out


def assign_sharded(engine, local_rows, centroids, n_local: int, n_global: int, on_device: bool = True, out=None, gather: bool = False, dst=None,
                   group=None):
    """Assign over row shards: every rank assigns its own rows to the (replicated) centroids - no exchange on the data
    path, the ranks run independently.  Returns this rank's assignments, or with `gather` the assignments of all
    `n_global` rows in row order (on every rank, or on `dst` only)."""
    res = engine.assign(local_rows, centroids, n=n_local, on_device=on_device, out=out)
    if not gather:
        return res
    return gather_rows(res, n_global, group=group, dst=dst)
