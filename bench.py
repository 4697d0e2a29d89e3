#!/usr/bin/env python
"""Benchmark of the k-means hot path.

Default workload: flat Train on the headline configuration (n = 10 000 000, d = 1024, k = 10 000, 10 iterations,
fp32; seeded synthetic mixture with Zipf cluster sizes standing in for the public embedding set the reference is
benchmarked on).  `--workload c1|c2|c4|c5` runs the other benchmark configurations (c3 is the default).

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (the reference's CPU code, bounded sample)

One step = one complete pass of the workload (a Train, or an Assign for c5).  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# The benchmark configurations: shapes, the law of the synthetic data and the seed.
WORKLOADS = {
    "c1": dict(kind="flat", n=100_000, d=768, k=1_000, iters=10, centers=1_000, noise=0.3, zipf=0.0, seed=42, law="mixture",
               text="flat Train+Assign n=100000 d=768 k=1000 iters=10 (Gaussian mixture, 1000 centres, noise 0.3, unit rows, seed 42)"),
    "c2": dict(kind="flat", n=1_000_000, d=1536, k=4_096, iters=10, centers=4_096, noise=0.3, zipf=0.0, seed=7, law="anisotropic",
               text="flat Train n=1000000 d=1536 k=4096 iters=10 (anisotropic mixture, std 1/sqrt(1+j/64), unit rows, seed 7)"),
    "c3": dict(kind="flat", n=10_000_000, d=1024, k=10_000, iters=10, centers=10_000, noise=0.25, zipf=1.1, seed=123, law="mixture",
               text="flat Train n=10000000 d=1024 k=10000 iters=10 (Gaussian mixture, Zipf(1.1) sizes, unit rows, seed 123)"),
    "c4": dict(kind="hierarchical", n=10_000_000, d=768, k=65_536, iters=8, centers=65_536, noise=0.1, zipf=0.0, seed=2024, law="two_level",
               text="hierarchical Train+Assign n=10000000 d=768 k=65536 (256 mesoclusters, 3+5+0 iterations; two-level mixture, unit rows, seed 2024)"),
    "c5": dict(kind="assign", n=50_000_000, d=384, k=16_384, iters=1, centers=16_384, noise=0.3, zipf=0.0, seed=99, law="around_centroids",
               text="Assign n=50000000 d=384 to k=16384 fixed unit centroids (points = centroid + N(0, 0.3^2), unit rows, seed 99)"),
}
HEADLINE = WORKLOADS["c3"]
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)
BLOCK = 500_000   # rows per seeded block of the synthetic data: the data set does not depend on how it is sharded


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    p.add_argument("--n", type=int, default=0, help="override the number of rows (0 = the workload's)")
    p.add_argument("--iters", type=int, default=0, help="override the iterations of a flat workload (0 = the workload's), for short profiling runs")
    p.add_argument("--cpu-sample", type=int, default=0,
                   help="rows of the workload given to the CPU reference by the cpu_baseline leg (0 = 1 000 000, or 400 000 when warm-up + steps exceed 8, "
                        "so that a long run still ends within its time limit: the reference needs ~270 s per million rows of the headline workload)")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-pageable", action="store_true", help="skip the end-to-end figure from pageable host memory")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-cache", action="store_true", help="do not keep device buffers between Train calls")
    p.add_argument("--prune-split", type=int, default=0, help="force one route of the pruned pass (skm_set_prune_split; 0 = automatic), for profiling")
    return p.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


def measure_tf32_peak(torch, device, size=8192, reps=10):
    """Dense TF32 tensor throughput of the library GEMM (torch.matmul with TF32 allowed) on this GPU, best of `reps`:
    the denominator for the three TF32 products behind every fp32-accurate term.  Only a yardstick: nothing on the
    measured path calls it."""
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        a = torch.randn(size, size, device=device)
        b = torch.randn(size, size, device=device)
        torch.matmul(a, b)
        best = float("inf")
        for _ in range(reps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b)
            e1.record()
            torch.cuda.synchronize(device)
            best = min(best, e0.elapsed_time(e1))
        del a, b
        return 2.0 * size ** 3 / (best / 1e3) / 1e12
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev


# ---------------------------------------------------------------------------------------------
# Synthetic workloads, generated on the device in blocks of BLOCK rows, each block from its own seed
# ---------------------------------------------------------------------------------------------
def zipf_sizes(n, centers, s):
    w = np.arange(1, centers + 1, dtype=np.float64) ** (-s)
    sizes = np.maximum(1, np.floor(w / w.sum() * n)).astype(np.int64)
    sizes[0] += n - sizes.sum()
    return sizes


class Generator:
    """Rows [lo, hi) of a workload's data set, identical whatever the shard bounds."""

    def __init__(self, torch, device, spec, n):
        self.torch, self.device, self.spec, self.n = torch, device, spec, n
        g = torch.Generator(device=device)
        g.manual_seed(spec["seed"])
        d = spec["d"]
        law = spec["law"]
        self.scale = None
        if law == "two_level":
            supers = int(round(np.sqrt(spec["centers"])))
            sup = torch.randn(supers, d, generator=g, device=device, dtype=torch.float32)
            self.centers = (sup[:, None, :] + 0.2 * torch.randn(supers, spec["centers"] // supers, d, generator=g, device=device, dtype=torch.float32)).reshape(-1, d)
        else:
            self.centers = torch.randn(spec["centers"], d, generator=g, device=device, dtype=torch.float32)
            if law == "anisotropic":
                self.scale = torch.from_numpy((1.0 / np.sqrt(1.0 + np.arange(d) / 64.0)).astype(np.float32)).to(device)
                self.centers *= self.scale
            if law == "around_centroids":
                self.centers /= self.centers.norm(dim=1, keepdim=True)
        self.cum = None
        if spec["zipf"] > 0:
            self.cum = torch.from_numpy(np.cumsum(zipf_sizes(n, spec["centers"], spec["zipf"]))).to(device)

    def block(self, b):
        torch, spec = self.torch, self.spec
        lo, hi = b * BLOCK, min(self.n, (b + 1) * BLOCK)
        g = torch.Generator(device=self.device)
        g.manual_seed(spec["seed"] * 1_000_003 + 17 + b)
        if self.cum is not None:
            # Zipf sizes: a position drawn uniformly in [0, n) falls into a centre's interval
            pos = torch.randint(0, self.n, (hi - lo,), generator=g, device=self.device)
            labels = torch.searchsorted(self.cum, pos, right=True).clamp_(max=spec["centers"] - 1)
        else:
            labels = torch.randint(0, spec["centers"], (hi - lo,), generator=g, device=self.device)
        noise = torch.randn(hi - lo, spec["d"], generator=g, device=self.device, dtype=torch.float32) * spec["noise"]
        if self.scale is not None:
            noise *= self.scale
        noise += self.centers[labels]
        noise /= noise.norm(dim=1, keepdim=True)
        return noise

    def rows(self, lo, hi):
        torch = self.torch
        x = torch.empty(hi - lo, self.spec["d"], device=self.device, dtype=torch.float32)
        for b in range(lo // BLOCK, (hi + BLOCK - 1) // BLOCK):
            blk = self.block(b)
            s, e = max(lo, b * BLOCK), min(hi, (b + 1) * BLOCK)
            x[s - lo:e - lo] = blk[s - b * BLOCK:e - b * BLOCK]
            del blk
        torch.cuda.synchronize(self.device)
        return x


def make_shard(torch, device, n, d, centers, noise, zipf, seed, lo, hi, rank=0):
    """Rows [lo, hi) of a Gaussian mixture with the given law (kept for the tests that generate config 3 on the device)."""
    spec = dict(d=d, centers=centers, noise=noise, zipf=zipf, seed=seed, law="mixture")
    return Generator(torch, device, spec, n).rows(lo, hi)


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.gpu_index = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu_index)],
                                         stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.tmp.flush()
        rows = []
        with open(self.tmp.name) as f:
            for line in f:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 9:
                    rows.append(parts)
        os.unlink(self.tmp.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        sm = sorted(float(r[1]) for r in rows)
        reasons = set()
        for r in rows:
            for name, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "power_w_max": max(float(r[3]) for r in rows), "samples": len(rows),
                "reasons": sorted(reasons)}


# ---------------------------------------------------------------------------------------------
# Reference arm / CPU baseline: the unmodified reference (oracle/_ref) on a bounded sample
# ---------------------------------------------------------------------------------------------
def host_cores() -> int:
    """Cores this process may use (torchrun exports OMP_NUM_THREADS=1, which would otherwise throttle the reference)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def reference_run(spec, sample: np.ndarray, centroids=None):
    """One pass of the workload by the reference on `sample`; returns (seconds, iterations)."""
    from oracle import ref

    ref.lib().ref_set_blas_threads(host_cores())
    hier = spec["kind"] == "hierarchical"
    k, d = spec["k"], spec["d"]
    if spec["kind"] == "assign":
        km = ref.RefKMeans(k, d, ref.default_config(False, n_threads=host_cores()))
        t0 = time.perf_counter()
        km.assign(sample, centroids)
        return time.perf_counter() - t0, 1
    kw = dict(sampling_fraction=1.0, early_termination=0, seed=spec["seed"], n_threads=host_cores())
    if not hier:
        kw["iters"] = spec["iters"]
    km = ref.RefKMeans(k, d, ref.default_config(hier, **kw), hierarchical=hier)  # the rotation matrix is built here, outside the timed call, as in the reference's own drivers
    t0 = time.perf_counter()
    km.train(sample)
    dt = time.perf_counter() - t0
    n_it = len(km.stats()) if not hier else spec["iters"]
    return dt, n_it


def host_rows(spec, n, rows):
    """The first `rows` rows of the workload (and the centroids of the assign workload) as host arrays; needs the GPU the
    data is generated on."""
    import torch

    dev = torch.device("cuda", torch.cuda.current_device())
    gen = Generator(torch, dev, spec, n)
    x = gen.rows(0, rows).cpu().numpy()
    c = gen.centers.cpu().numpy() if spec["kind"] == "assign" else None
    return np.ascontiguousarray(x), c


def host_rows_numpy(spec, rows):
    """A host-side draw with the workload's law (the reference arm must run where no GPU is visible too)."""
    rng = np.random.default_rng(spec["seed"])
    d, centers = spec["d"], spec["centers"]
    if spec["law"] == "two_level":
        supers = int(round(np.sqrt(centers)))
        sup = rng.standard_normal((supers, d), dtype=np.float32)
        c = (sup[:, None, :] + 0.2 * rng.standard_normal((supers, centers // supers, d), dtype=np.float32)).reshape(-1, d)
    else:
        c = rng.standard_normal((centers, d), dtype=np.float32)
    scale = None
    if spec["law"] == "anisotropic":
        scale = (1.0 / np.sqrt(1.0 + np.arange(d) / 64.0)).astype(np.float32)
        c *= scale
    if spec["law"] == "around_centroids":
        c /= np.linalg.norm(c, axis=1, keepdims=True)
    if spec["zipf"] > 0:
        w = np.arange(1, centers + 1, dtype=np.float64) ** (-spec["zipf"])
        labels = rng.choice(centers, size=rows, p=w / w.sum())
    else:
        labels = rng.integers(0, centers, size=rows)
    noise = spec["noise"] * rng.standard_normal((rows, d), dtype=np.float32)
    if scale is not None:
        noise *= scale
    x = c[labels] + noise
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return np.ascontiguousarray(x, dtype=np.float32), (np.ascontiguousarray(c, dtype=np.float32) if spec["kind"] == "assign" else None)


def unit_of(spec):
    return ("assign_points_per_s", "points/s") if spec["kind"] == "assign" else ("train_points_iters_per_s", "points*iters/s")


def run_reference_arm(args, spec, n):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref

    metric, unit = unit_of(spec)
    if not ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref was not built (reference sources absent at build time)"}))
        return
    cores = host_cores()
    # The whole arm is given about seven minutes of CPU work.  The reference needs ~3 s + 0.27 s per 1000 rows for one
    # Train of the headline shape on 16 cores (measured: 30 s at 100 000 rows, 274 s at 1 000 000), and a sample with
    # only a handful of points per cluster is not the workload any more (thousands of empty clusters per iteration,
    # whose re-seeding walk then dominates).  So the passes are capped at one warm-up + three timed ones, each on as
    # many rows as the budget allows; the line reports the passes actually run.
    n_warm = min(args.warmup, 1)
    n_timed = max(1, min(args.steps, 3))
    per_pass_s = 420.0 / (n_warm + n_timed)
    if spec["kind"] == "assign":
        rows = int(min(n, max(10_000, 2.0e6 * per_pass_s / 60.0 * cores / 16.0)))
    else:
        rows = int(min(n, 1_000_000, max(3 * spec["k"], (per_pass_s - 3.0) / 0.271e-3 * cores / 16.0 * (1024 * 10_000) / (spec["d"] * spec["k"]))))
    rows = max(rows, spec["k"])
    sample, cent = host_rows_numpy(spec, rows)
    times, n_it = [], 1
    for i in range(n_warm + n_timed):
        dt, n_it = reference_run(spec, sample, cent)
        if i >= n_warm:
            times.append(dt)
    t = float(np.mean(times))
    value = rows * n_it / t
    sample_text = (f"{rows} rows drawn on the host with the workload's law (a separate numpy draw, not the GPU arm's rows), same d, k and iterations; "
                   f"{n_warm} warm-up + {n_timed} timed passes (asked for: {args.warmup} + {args.steps}), sized so that they take about seven minutes; "
                   f"SuperKMeans reference headers + SciPy OpenBLAS")
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus, "steps": n_timed, "warmup": n_warm,
        "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": spec["text"], "sample_rows": rows},
        "cpu_baseline": {"value": value, "unit": unit, "cores": int(cores), "kind": "reference", "sample": sample_text},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# Our arm
# ---------------------------------------------------------------------------------------------
# DRAM traffic per row of the headline shape: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the
# kernel at n = 400 000 rows (same d and k), divided by the rows.  Traffic of these kernels grows with the rows (the
# centroid side stays in L2), so a launch over r rows moves about r times this.
TRAFFIC_PER_ROW = {
    ("gemm_tc_kernel<ARGMIN>", 1024, 10_000): 3.59e9 / 4e5,
    ("gemm_tc_kernel<PRUNE>", 1024, 10_000): 0.377e9 / 4e5,
    ("walk_lists_kernel", 1024, 10_000): 5.86e9 / 4e5,
    # optimistic chain pass, captured at n = 1 000 000 in the first pruned iteration (the one with the longest centroid
    # lists: an upper figure for the later ones)
    ("sparse_chain_kernel", 1024, 10_000): 137.9e9 / 1e6,
}


def work_rows(kernel, n_local, stats, engine):
    """Rows one step sends through `kernel`."""
    pruned = sum(1 for s in stats if not s.is_gemm_only)
    if kernel.endswith("<ARGMIN>"):
        return n_local * max(1, sum(1 for s in stats if s.is_gemm_only))
    if kernel == "sparse_chain_kernel" and engine is not None:
        return engine.chain_counters()["rows"]
    if engine is not None:
        return max(0, n_local * pruned - engine.chain_counters()["rows"])
    return n_local * pruned


def main():
    args = parse_args()
    spec = dict(WORKLOADS[args.workload])
    n = args.n or spec["n"]
    if args.iters and spec["kind"] == "flat":
        spec["iters"] = args.iters
        spec["text"] += f" [iterations overridden: {args.iters}]"
    if args.impl == "reference":
        run_reference_arm(args, spec, n)
        return

    import torch
    import torch.distributed as dist

    import superkmeans_b200 as skm
    from superkmeans_b200 import distributed as skd
    from superkmeans_b200 import engine as eng

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        if spec["kind"] == "hierarchical" or args.workload in ("c1", "c2"):
            raise SystemExit(f"workload {args.workload} runs on one GPU (hierarchical and the small flat configurations are not sharded)")
        dist.init_process_group("nccl", device_id=device)
        if spec["kind"] == "flat":
            comm = skd.make_comm(local_rank)   # the per-iteration sums run inside the library, on the engine's stream
    if not args.no_cache:
        eng.set_workspace_cache(True)
    if args.prune_split:
        eng.set_prune_split(args.prune_split)

    d, k, kind = spec["d"], spec["k"], spec["kind"]
    metric, unit = unit_of(spec)
    lo, hi = skd.shard_bounds(n, rank, world)
    n_local = hi - lo
    gen = Generator(torch, device, spec, n)
    x = gen.rows(lo, hi)
    hier = kind == "hierarchical"
    cfg_kw = dict(sampling_fraction=1.0, early_termination=0, seed=spec["seed"])
    if not hier:
        cfg_kw["iters"] = spec["iters"]
    rotation = eng.rotation_matrix(d, spec["seed"]) if kind != "assign" else None  # built at construction in the reference, outside Train
    cent_dev = gen.centers if kind == "assign" else None
    out_dev = torch.empty(n_local, dtype=torch.int32, device=device) if kind == "assign" else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def one_pass(data, on_device):
        """One step: a Train (flat / hierarchical) or an Assign.  Returns (engine, result, wall seconds)."""
        e = skm.Engine(k, d, skm.default_config(hier, **cfg_kw), hierarchical=hier, device=local_rank)
        if rotation is not None:
            e.set_rotation(rotation)
        if comm is not None:
            e.set_shard_comm(n, lo, comm)
        barrier()
        t0 = time.perf_counter()
        if kind == "assign":
            # row shards, replicated centroids, no exchange on the data path (the ranks' answers stay on their GPUs / hosts)
            res = skd.assign_sharded(e, data, cent_dev if on_device else cent_host, n_local, n, on_device=on_device, out=out_dev if on_device else None)
        else:
            res = e.train(data, n=n_local, on_device=on_device)
        torch.cuda.synchronize(device)
        wall = time.perf_counter() - t0
        return e, res, wall

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    cent_host = cent_dev.cpu().numpy() if cent_dev is not None else None

    # ---- device-resident throughput ("value")
    for _ in range(args.warmup):
        one_pass(x, True)
    sampler = ClockSampler(local_rank)
    if kind == "flat":
        eng.chain_role_cycles()   # clear the role counters of the warm-up steps
    launches0 = eng.kernel_launches()
    allocs0 = eng.device_allocations()
    if rank == 0:
        sampler.start()
    dev_ms, walls, phase_acc, stats, prune_path = [], [], {}, [], 0
    timed_phase = "search/1st_blas" if kind == "assign" else "train"
    for _ in range(args.steps):
        e, res, wall = one_pass(x, True)
        pt = e.phase_times()
        dev_ms.append(max_over_ranks(pt[timed_phase][0]))
        walls.append(max_over_ranks(wall * 1e3))
        for name, (ms, calls) in pt.items():
            a = phase_acc.setdefault(name, [0.0, 0])
            a[0] += ms
            a[1] += calls
        if kind == "flat":
            stats = e.stats(0)
        prune_path = e.last_prune_path
    clocks = sampler.stop() if rank == 0 else None
    launches = eng.kernel_launches() - launches0
    allocs = eng.device_allocations() - allocs0
    n_it = len(stats) if kind == "flat" else spec["iters"]
    ms_per_step = float(np.mean(dev_ms))
    value = n * n_it / (ms_per_step / 1e3)
    phases = {name: v[0] / args.steps for name, v in phase_acc.items()}
    if kind != "assign":
        covered = sum(phases[p] for p in ("rotator", "norms_calc", "search/1st_blas", "search", "update_centroids", "consolidate", "shift", "alloc_free", "init_centroids", "allreduce"))
        phases["unaccounted"] = phases["train"] - covered

    # ---- roofline of the dominant kernel (device time by CUDA events inside the engine)
    pk = peaks()
    peak_tf = float(pk.get("bf16_tflops_sustained", pk.get("bf16_tflops")))
    peak_gbs = float(pk["hbm_gbs"])
    cands = []   # (kernel, phase ms over all timed steps, launches, bound, work per step)
    if kind == "assign":
        ms, calls = phase_acc["search/1st_blas"]
        cands.append(("gemm_tc_kernel<ARGMIN>", ms, calls, "tensor", 2.0 * n_local * k * d))
    elif hier:
        n_meso = int(round(np.sqrt(k)))
        ms, calls = phase_acc["search/1st_blas"]
        # every phase sees ~k / n_meso centroids per point: 3 mesoclustering + 5 fine iterations, all exact
        cands.append(("gemm_tc_kernel<ARGMIN>", ms, calls, "tensor", 2.0 * n_local * d * (3.0 * n_meso + 5.0 * k / n_meso)))
        ms, calls = phase_acc["update_centroids"]
        cands.append(("segsum_tile_kernel", ms, calls, "hbm", 8.0 * n_local * d * 4.0))
        ms, calls = phase_acc["rotator"]
        cands.append(("rotation", ms, calls, "tensor", 2.0 * n_local * d * d))
    else:
        counters = e.prune_counters()   # of the last timed Train
        chain = e.chain_counters()
        d_partial = [s.partial_d for s in stats if not s.is_gemm_only]
        mean_pd = float(np.mean(d_partial)) if d_partial else 0.0
        ms, calls = phase_acc["search/1st_blas"]
        cands.append(("gemm_tc_kernel<ARGMIN>", ms, calls, "tensor", sum(2.0 * n_local * k * d for s in stats if s.is_gemm_only)))
        ms, calls = phase_acc["search/first_test"]
        # a Train can mix routes (the automatic choice is taken per pass): rows that went through the ordered chain, rows
        # of the unordered dense chain, and rows that took first test + list walk
        chain_rows = chain["rows"]
        legacy_dense_rows = max(0, counters["dense_rows"] - chain_rows)
        listed_rows = max(0, n_local * len(d_partial) - chain_rows)
        cands.append(("gemm_tc_kernel<PRUNE>", ms, calls, "tensor", 2.0 * listed_rows * k * mean_pd if ms > 0 else 0.0))
        ms, calls = phase_acc["search/dense"]
        if chain_rows >= legacy_dense_rows:
            # union pass over the first d' dimensions of every centroid + the chain over the gathered columns (128 rows per unit)
            cands.append(("sparse_chain_kernel", ms, calls, "tensor", 2.0 * 128 * chain["columns"] * d + 2.0 * chain_rows * k * mean_pd))
        else:
            cands.append(("chain_tc_kernel", ms, calls, "tensor", 2.0 * legacy_dense_rows * k * d))
        ms, calls = phase_acc["search/walk"]
        # every (pair, 64-dimension block) step gathers 256 B of the centroid's PDX block, served by L2
        cands.append(("walk_lists_kernel", ms, calls, "l2", 256.0 * counters["walk_pair_steps"]))
        ms, calls = phase_acc["rotator"]
        cands.append(("rotation", ms, calls, "tensor", 2.0 * n_local * d * d))
    dom, dom_ms, dom_calls, bound, work = max(cands, key=lambda c: c[1])
    dom_ms_per_step = dom_ms / args.steps
    if bound == "tensor":
        achieved = work / (dom_ms_per_step / 1e3) / 1e12 if dom_ms > 0 else 0.0
        roofline = {"kernel": dom, "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf, "traffic": None,
                    "peak_source": f"bf16 dense sustained, {pk['_source']}", "avg_launch_ms": dom_ms / max(dom_calls, 1),
                    "note": "fp32-accurate distances from three TF32 products per term; flops counted once as 2*rows*columns*K"}
        tf32 = pk.get("tf32_tflops") or (measure_tf32_peak(torch, device) if rank == 0 else None)
        if tf32:
            # the tensor cores execute three TF32 products per counted term
            roofline["tf32_peak"] = float(tf32)
            roofline["tf32_peak_source"] = "torch.matmul 8192^3 with TF32 allowed, best of 10, measured in this run (burst)"
            roofline["frac_of_tf32_dense"] = 3.0 * achieved / float(tf32)
    else:
        achieved = work / (dom_ms_per_step / 1e3) / 1e9 if dom_ms > 0 else 0.0
        roofline = {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs, "traffic": None,
                    "peak_source": f"HBM copy, {pk['_source']}", "avg_launch_ms": dom_ms / max(dom_calls, 1),
                    "note": ("gathered 256-byte centroid blocks served by L2, not HBM: the fraction is against the HBM copy peak for scale only" if bound == "l2"
                             else "rows read once per iteration")}
    roofline["kernels_ms_per_step"] = {c[0]: round(c[1] / args.steps, 3) for c in cands}
    if kind == "flat":
        roles = eng.chain_role_cycles()   # of the timed steps (and whatever ran after them)
        if roles["steps"]:
            roofline["chain_role_cycles_per_step"] = roles
    traffic = TRAFFIC_PER_ROW.get((dom, d, k))
    if traffic is not None and dom_calls:
        rows_per_launch = work_rows(dom, n_local, stats, e if kind == "flat" else None) * args.steps / dom_calls
        roofline["traffic"] = traffic * rows_per_launch
        roofline["traffic_note"] = "DRAM bytes of an ncu capture of this kernel on a slice of the workload (same d and k), per row, times the rows one launch covers"
        if dom == "sparse_chain_kernel":
            roofline["traffic_note"] += ("; captured in the first pruned iteration of a 1 000 000-row slice, where a tile reaches about twice as many centroids as in "
                                         "the later iterations of the full workload: an upper figure")

    # ---- the configurations that say "Train + Assign": Assign and AssignTrainingPoints of the training rows, device-resident
    extra_calls = None
    if args.workload in ("c1", "c4") and world == 1:
        cd = torch.from_numpy(res).to(device)
        out_a = torch.empty(n_local, dtype=torch.int32, device=device)
        out_f = torch.empty(n_local, dtype=torch.int32, device=device)
        times = {}
        for name, fn, out in (("assign", e.assign, out_a), ("assign_training_points", e.assign_training_points, out_f)):
            fn(x, cd, n=n_local, on_device=True, out=out)   # warm-up (allocations)
            torch.cuda.synchronize(device)
            t0 = time.perf_counter()
            fn(x, cd, n=n_local, on_device=True, out=out)
            torch.cuda.synchronize(device)
            times[name + "_s"] = time.perf_counter() - t0
        times["fast_equals_brute_force"] = float((out_a == out_f).float().mean())
        extra_calls = times
        del cd, out_a, out_f

    # ---- end to end through the public API with host input: pinned, then pageable (what a caller of Train(const float*, n) has)
    e2e, e2e_pageable = None, None
    if not args.no_e2e:
        rows_e2e = n_local if kind != "assign" else min(n_local, 16_000_000)
        xh = torch.empty((rows_e2e, d), dtype=torch.float32, pin_memory=True)
        xh.copy_(x[:rows_e2e])
        torch.cuda.synchronize(device)
        saved_n_local = n_local
        n_local = rows_e2e   # one_pass reads it
        xh_np = xh.numpy()
        one_pass(xh_np, False)
        ts = []
        for _ in range(max(1, min(args.steps, 2))):
            _, _, wall = one_pass(xh_np, False)
            ts.append(max_over_ranks(wall * 1e3))
        e2e_ms = float(np.mean(ts))
        rows_global = n if kind != "assign" else rows_e2e * world
        e2e = {"value": rows_global * n_it / (e2e_ms / 1e3), "unit": unit, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": int(rows_e2e * d * 4 + k * d * 4 + (d * d * 4 if kind != "assign" else 0)),
               "d2h_bytes_per_step": int(rows_e2e * 4 if kind == "assign" else k * d * 4 + n_it * (k * 4 + 24)), "host_memory": "pinned"}
        if kind == "assign" and rows_e2e < saved_n_local:
            e2e["note"] = f"measured on the first {rows_e2e} rows of each shard (host memory)"
        del xh_np, xh
        if not args.no_pageable and world == 1:
            xp = np.empty((rows_e2e, d), dtype=np.float32)   # ordinary (pageable) host memory
            step = 1_000_000
            for s0 in range(0, rows_e2e, step):
                xp[s0:s0 + step] = x[s0:s0 + step].cpu().numpy()
            _, _, wall = one_pass(xp, False)
            _, _, wall = one_pass(xp, False)
            e2e_pageable = {"value": rows_global * n_it / wall, "unit": unit, "ms_per_step": wall * 1e3, "host_memory": "pageable"}
            del xp
        n_local = saved_n_local

    # ---- CPU baseline and parity on a bounded sample (rank 0, single-GPU run only)
    cpu_baseline, parity = None, None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import ref

        if ref.available():
            cpu_rows = args.cpu_sample or (1_000_000 if args.warmup + args.steps <= 8 else 400_000)
            rows = max(k, min(cpu_rows, n))
            sample = np.ascontiguousarray(x[:rows].cpu().numpy())
            dt, r_it = reference_run(spec, sample, cent_host)
            cpu_baseline = {"value": rows * r_it / dt, "unit": unit, "cores": host_cores(), "kind": "reference", "seconds": dt,
                            "sample": f"first {rows} rows of the workload, same d, k and iterations, one run"}
            if kind == "flat":
                # Parity against the reference on a separate, well-conditioned sample of the same dimensionality: as many
                # mixture centres as clusters (k_p > 256 keeps the pruned path on), ~300 points per cluster.
                rows_p = min(rows, 100_000)
                k_p = max(257, rows_p // 300)
                prng = np.random.default_rng(spec["seed"] + 7)
                pc = prng.standard_normal((k_p, d), dtype=np.float32)
                psample = pc[prng.integers(0, k_p, size=rows_p)] + spec["noise"] * prng.standard_normal((rows_p, d), dtype=np.float32)
                psample /= np.linalg.norm(psample, axis=1, keepdims=True)
                psample = np.ascontiguousarray(psample, dtype=np.float32)
                rcfg = ref.default_config(False, iters=spec["iters"], sampling_fraction=1.0, early_termination=0, seed=spec["seed"])
                kmp = ref.RefKMeans(k_p, d, rcfg)
                rcp = kmp.train(psample)
                e2 = skm.Engine(k_p, d, skm.default_config(False, **cfg_kw), device=local_rank)
                e2.set_rotation(kmp.rotation_matrix())
                c2 = e2.train(psample)
                a2, ra = e2.assign(psample, c2), kmp.assign(psample, rcp)
                w2 = float(((psample.astype(np.float64) - c2[a2]) ** 2).sum())
                rw = float(((psample.astype(np.float64) - rcp[ra]) ** 2).sum())
                parity = {"sample": f"{rows_p} rows, {k_p} mixture centres, same d and noise as the workload", "k": k_p, "prune_path": e2.last_prune_path, "wcss": w2,
                          "wcss_reference": rw, "wcss_rel_diff": abs(w2 - rw) / rw, "assignments_equal": float((a2 == ra).mean()),
                          "centroid_rel_l2": float(np.linalg.norm(c2 - rcp) / np.linalg.norm(rcp))}

    # ---- N ranks against one: the same small data set trained in shards (all ranks) and whole (rank 0)
    sharded_parity = None
    if world > 1 and kind == "flat":
        pspec = dict(d=256, centers=1000, noise=0.3, zipf=0.0, seed=77, law="mixture")
        pn, pk_ = 200_000, 1000
        pgen = Generator(torch, device, pspec, pn)
        plo, phi = skd.shard_bounds(pn, rank, world)
        pcfg = dict(iters=6, sampling_fraction=1.0, early_termination=0, seed=77)
        prot = eng.rotation_matrix(256, 77)
        es = skm.Engine(pk_, 256, skm.default_config(False, **pcfg), device=local_rank)
        es.set_rotation(prot)
        es.set_shard_comm(pn, plo, comm)
        cs = es.train(pgen.rows(plo, phi), n=phi - plo, on_device=True)
        obj_s = float(es.stats(0)[-1].objective)
        if rank == 0:
            e1 = skm.Engine(pk_, 256, skm.default_config(False, **pcfg), device=local_rank)
            e1.set_rotation(prot)
            c1 = e1.train(pgen.rows(0, pn), n=pn, on_device=True)
            obj_1 = float(e1.stats(0)[-1].objective)
            a_s, a_1 = es.assignments(), e1.assignments()[plo:phi]
            sharded_parity = {"data": "200000 x 256, 1000 centres, k = 1000, 6 iterations", "objective_sharded": obj_s, "objective_single": obj_1,
                              "objective_rel_diff": abs(obj_s - obj_1) / obj_1, "centroid_max_rel_diff": float(np.abs(cs - c1).max() / np.abs(c1).max()),
                              "assignments_equal_rank0_shard": float((a_s == a_1).mean()),
                              "partial_d_equal": [s.partial_d for s in es.stats(0)] == [s.partial_d for s in e1.stats(0)]}

    if rank == 0:
        config = {"workload": spec["text"] if n == spec["n"] else spec["text"] + f" [rows overridden: {n}]", "rows_per_gpu": n_local,
                  "l2": "inputs (rows_per_gpu*d*4 bytes) exceed L2; no explicit flush", "workspace_cache": not args.no_cache,
                  "sums_across_shards": "NCCL group on the engine's stream" if comm is not None else None}
        if kind == "flat":
            config.update({"partial_d": [int(s.partial_d) for s in stats], "not_pruned_pct": [round(float(s.not_pruned_pct), 6) for s in stats],
                           "objective": float(stats[-1].objective), "prune_path": prune_path, "chain": e.chain_counters()})
            if args.prune_split:
                config["prune_split_forced"] = args.prune_split
        line = {
            "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "seconds_per_step": ms_per_step / 1e3, "wall_ms_per_step": float(np.mean(walls)), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
            "phases_ms_per_step": {name: round(v, 3) for name, v in phases.items()},
            "after_train": extra_calls, "roofline": roofline, "cpu_baseline": cpu_baseline, "parity_on_sample": parity, "sharded_parity": sharded_parity, "e2e": e2e, "e2e_pageable": e2e_pageable,
            "gpu_launches": int(launches), "device_allocations_in_timed_region": int(allocs), "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
