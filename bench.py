#!/usr/bin/env python
"""Benchmark of the k-means hot path: flat Train on the headline configuration
(n = 10 000 000, d = 1024, k = 10 000, 10 iterations, fp32; seeded synthetic mixture with Zipf
cluster sizes standing in for the public embedding set the reference is benchmarked on).

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched by torchrun)
    python bench.py --impl reference ...                     (the reference's CPU code, bounded sample)

One step = one complete Train() over the data set.  Rank 0 prints one JSON line.
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

HEADLINE = dict(n=10_000_000, d=1024, k=10_000, iters=10, centers=10_000, noise=0.25, zipf=1.1, seed=123)
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0, bf16_tflops_sustained=1400.0)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--n", type=int, default=HEADLINE["n"])
    p.add_argument("--d", type=int, default=HEADLINE["d"])
    p.add_argument("--k", type=int, default=HEADLINE["k"])
    p.add_argument("--iters", type=int, default=HEADLINE["iters"])
    p.add_argument("--cpu-sample", type=int, default=100_000, help="rows of the workload given to the CPU reference")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu-baseline", action="store_true")
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


# ---------------------------------------------------------------------------------------------
# Synthetic workload (generated on the device, shard by shard)
# ---------------------------------------------------------------------------------------------
def zipf_sizes(n, centers, s):
    w = np.arange(1, centers + 1, dtype=np.float64) ** (-s)
    sizes = np.maximum(1, np.floor(w / w.sum() * n)).astype(np.int64)
    sizes[0] += n - sizes.sum()
    return sizes


def make_shard(torch, device, n, d, centers, noise, zipf, seed, lo, hi, rank):
    """Rows [lo, hi) of the global data set: Gaussian mixture, Zipf sizes, rows L2-normalised."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    c = torch.randn(centers, d, generator=g, device=device, dtype=torch.float32)
    perm = torch.randperm(n, generator=g, device=device)
    cum = torch.from_numpy(np.cumsum(zipf_sizes(n, centers, zipf))).to(device)
    labels = torch.searchsorted(cum, perm[lo:hi], right=True).clamp_(max=centers - 1)
    del perm
    x = torch.empty(hi - lo, d, device=device, dtype=torch.float32)
    g2 = torch.Generator(device=device)
    g2.manual_seed(seed + 1000 + rank)
    step = 500_000
    for s in range(0, hi - lo, step):
        e = min(hi - lo, s + step)
        blk = c[labels[s:e]] + noise * torch.randn(e - s, d, generator=g2, device=device, dtype=torch.float32)
        blk /= blk.norm(dim=1, keepdim=True)
        x[s:e] = blk
    torch.cuda.synchronize(device)
    return x


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


def reference_train(sample: np.ndarray, k: int, iters: int, seed: int):
    from oracle import ref

    ref.lib().ref_set_blas_threads(host_cores())
    cfg = ref.default_config(False, iters=iters, sampling_fraction=1.0, early_termination=0, seed=seed, n_threads=host_cores())
    km = ref.RefKMeans(k, sample.shape[1], cfg)  # rotation matrix is built here, outside the timed call, as in the reference's own drivers
    t0 = time.perf_counter()
    cent = km.train(sample)
    dt = time.perf_counter() - t0
    return dt, km, cent


def host_sample(args, rows: int) -> np.ndarray:
    """The first `rows` rows of the workload, generated on the host with the same recipe."""
    rng = np.random.default_rng(HEADLINE["seed"])
    c = rng.standard_normal((HEADLINE["centers"], args.d), dtype=np.float32)
    w = np.arange(1, HEADLINE["centers"] + 1, dtype=np.float64) ** (-HEADLINE["zipf"])
    labels = rng.choice(HEADLINE["centers"], size=rows, p=w / w.sum())
    x = c[labels] + HEADLINE["noise"] * rng.standard_normal((rows, args.d), dtype=np.float32)
    x /= np.linalg.norm(x, axis=1, keepdims=True)
    return np.ascontiguousarray(x, dtype=np.float32)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import ref

    if not ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref was not built (reference sources absent at build time)"}))
        return
    rows = max(args.k, min(args.cpu_sample, args.n))
    sample = host_sample(args, rows)
    cores = host_cores()
    times = []
    for i in range(args.warmup + args.steps):
        dt, km, _ = reference_train(sample, args.k, args.iters, HEADLINE["seed"])
        if i >= args.warmup:
            times.append(dt)
    t = float(np.mean(times))
    n_it = len(km.stats())
    value = rows * n_it / t
    line = {
        "impl": "reference", "metric": "train_points_iters_per_s", "value": value, "unit": "points*iters/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"flat Train n={args.n} d={args.d} k={args.k} iters={args.iters} (Zipf mixture, unit rows)", "sample_rows": rows},
        "cpu_baseline": {"value": value, "unit": "points*iters/s", "cores": int(cores), "kind": "reference",
                         "sample": f"first {rows} rows of the workload, same d, k and iterations; SuperKMeans reference headers + SciPy OpenBLAS"},
        "e2e": {"value": value, "unit": "points*iters/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# Our arm
# ---------------------------------------------------------------------------------------------
def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
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
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    n, d, k, iters = args.n, args.d, args.k, args.iters
    lo, hi = skd.shard_bounds(n, rank, world)
    n_local = hi - lo
    x = make_shard(torch, device, n, d, HEADLINE["centers"], HEADLINE["noise"], HEADLINE["zipf"], HEADLINE["seed"], lo, hi, rank)

    cfg_kw = dict(iters=iters, sampling_fraction=1.0, early_termination=0, seed=HEADLINE["seed"])
    rotation = eng.rotation_matrix(d, HEADLINE["seed"])  # built at construction in the reference, outside Train

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    def one_train(data, on_device):
        e = skm.Engine(k, d, skm.default_config(False, **cfg_kw), device=local_rank)
        e.set_rotation(rotation)
        if world > 1:
            e.set_shard(n, lo, skd.make_allreduce(device))
        barrier()
        t0 = time.perf_counter()
        cent = e.train(data, n=n_local, on_device=on_device)
        torch.cuda.synchronize(device)
        wall = time.perf_counter() - t0
        return e, cent, wall

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput ("value")
    for _ in range(args.warmup):
        one_train(x, True)
    sampler = ClockSampler(local_rank)
    launches0 = eng.kernel_launches()
    if rank == 0:
        sampler.start()
    dev_ms, walls, phase_acc, stats, prune_path = [], [], {}, None, 0
    for _ in range(args.steps):
        e, cent, wall = one_train(x, True)
        pt = e.phase_times()
        dev_ms.append(max_over_ranks(pt["train"][0]))
        walls.append(max_over_ranks(wall * 1e3))
        for name, (ms, calls) in pt.items():
            a = phase_acc.setdefault(name, [0.0, 0])
            a[0] += ms
            a[1] += calls
        stats = e.stats(0)
        prune_path = e.last_prune_path
    clocks = sampler.stop() if rank == 0 else None
    launches = eng.kernel_launches() - launches0
    n_it = len(stats)
    ms_per_step = float(np.mean(dev_ms))
    value = n * n_it / (ms_per_step / 1e3)

    # ---- roofline of the dominant kernel (device time by CUDA events inside the engine)
    pk = peaks()
    peak_tf = float(pk.get("bf16_tflops_sustained", pk.get("bf16_tflops")))
    peak_gbs = float(pk["hbm_gbs"])
    counters = e.prune_counters()   # of the last timed Train
    chain_all = prune_path == 3
    d_partial = [s.partial_d for s in stats if not s.is_gemm_only]
    cands = []   # (kernel, phase ms, launches, bound, work per Train, unit)
    ms, calls = phase_acc["search/1st_blas"]
    cands.append(("gemm_tc_kernel<ARGMIN>", ms, calls, "tensor", sum(2.0 * n_local * k * d for s in stats if s.is_gemm_only)))
    chain = e.chain_counters()      # of the last timed Train
    ms, calls = phase_acc["search/first_test"]
    listed_rows = n_local * len(d_partial) - chain["rows"] if prune_path == 6 else n_local * len(d_partial)
    cands.append(("gemm_tc_kernel<PRUNE>", ms, calls, "tensor", 2.0 * listed_rows * k * float(np.mean(d_partial)) if prune_path in (4, 6) and d_partial else 0.0))
    ms, calls = phase_acc["search/dense"]
    if prune_path == 6:
        # union pass over the first d' dimensions of every centroid + the chain over the gathered columns (128 rows per unit)
        cands.append(("sparse_chain_kernel", ms, calls, "tensor", 2.0 * 128 * chain["columns"] * d + 2.0 * chain["rows"] * k * float(np.mean(d_partial) if d_partial else 0)))
    else:
        cands.append(("chain_tc_kernel", ms, calls, "tensor", 2.0 * counters["dense_rows"] * k * d))
    ms, calls = phase_acc["search/walk"]
    # every (pair, 64-dimension block) step gathers 256 B of the centroid's PDX block (the point's 256 B stay in
    # registers across the pairs of a point)
    cands.append(("walk_lists_kernel", ms, calls, "hbm", 256.0 * counters["walk_pair_steps"]))
    if prune_path not in (3, 4, 6):
        ms, calls = phase_acc["search"]
        cands.append(("assign_pruned_kernel", ms, calls, "tensor", sum(2.0 * n_local * k * pd for pd in d_partial)))
    dom, dom_ms, dom_calls, bound, work = max(cands, key=lambda c: c[1])
    dom_ms_per_train = dom_ms / args.steps
    if bound == "tensor":
        achieved = work / (dom_ms_per_train / 1e3) / 1e12 if dom_ms > 0 else 0.0
        roofline = {"kernel": dom, "bound": "tensor", "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s", "frac": achieved / peak_tf, "traffic": None,
                    "peak_source": f"bf16 dense sustained, {pk['_source']}", "avg_launch_ms": dom_ms / max(dom_calls, 1),
                    "note": "fp32-accurate distances from three TF32 products per term; flops counted once as 2*rows*k*K"}
    else:
        achieved = work / (dom_ms_per_train / 1e3) / 1e9 if dom_ms > 0 else 0.0
        roofline = {"kernel": dom, "bound": "hbm", "achieved": achieved, "peak": peak_gbs, "unit": "GB/s", "frac": achieved / peak_gbs, "traffic": None,
                    "peak_source": f"HBM copy, {pk['_source']}", "avg_launch_ms": dom_ms / max(dom_calls, 1),
                    "note": "gathered 256-byte centroid blocks, served by L2 rather than HBM (hence a fraction near or above 1); bytes = 256 B per (pair, 64-dimension block) step, counted by the kernel"}
    roofline["kernels_ms_per_train"] = {c[0]: round(c[1] / args.steps, 3) for c in cands}
    # DRAM bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture at n = 400 000 (same d and
    # k), per row, times the rows one launch covers here.  Traffic of
    # these kernels grows with the rows (the centroid side stays in L2).  The chain's rows per launch vary: not scaled.
    dram_per_row = {"gemm_tc_kernel<ARGMIN>": 3.59e9 / 4e5, "gemm_tc_kernel<PRUNE>": 0.377e9 / 4e5, "walk_lists_kernel": 5.86e9 / 4e5}
    if dom in dram_per_row and dom_calls and (d, k) == (1024, 10000):
        rows_per_launch = n_local * (1 if dom.endswith("<ARGMIN>") else len(d_partial)) * args.steps / dom_calls
        roofline["traffic"] = dram_per_row[dom] * rows_per_launch
        roofline["traffic_note"] = "scaled by rows per launch from an ncu capture at n=400000"

    # ---- end to end through the public API with host (pinned) input
    e2e = None
    if not args.no_e2e:
        xh = torch.empty((n_local, d), dtype=torch.float32, pin_memory=True)
        xh.copy_(x)
        torch.cuda.synchronize(device)
        xh_np = xh.numpy()
        one_train(xh_np, False)
        ts = []
        for _ in range(max(1, min(args.steps, 2))):
            _, _, wall = one_train(xh_np, False)
            ts.append(max_over_ranks(wall * 1e3))
        e2e_ms = float(np.mean(ts))
        e2e = {"value": n * n_it / (e2e_ms / 1e3), "unit": "points*iters/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": int(n_local * d * 4 + k * d * 4 + d * d * 4),
               "d2h_bytes_per_step": int(k * d * 4 + n_it * (k * 4 + 24))}
        del xh, xh_np

    # ---- CPU baseline and parity on a bounded sample (rank 0, single-GPU run only)
    cpu_baseline, parity = None, None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import ref

        if ref.available():
            rows = max(k, min(args.cpu_sample, n))
            sample = np.ascontiguousarray(x[:rows].cpu().numpy())
            dt, km, rc = reference_train(sample, k, iters, HEADLINE["seed"])
            r_it = len(km.stats())
            cpu_baseline = {"value": rows * r_it / dt, "unit": "points*iters/s", "cores": host_cores(), "kind": "reference", "train_s": dt,
                            "sample": f"first {rows} rows of the workload, same d, k and iterations"}
            # Parity against the reference on a separate, well-conditioned sample of the same dimensionality: as many
            # mixture centres as clusters (k_p > 256 keeps the pruned path on), ~300 points per cluster.  On the
            # workload's own first rows k-means is far from converged after ten iterations (ten points per cluster at
            # k = 10 000), single near-tie flips reshuffle whole clusters, and assignment agreement would measure
            # that chaos rather than the kernels.
            k_p = max(257, rows // 300)
            prng = np.random.default_rng(HEADLINE["seed"] + 7)
            pc = prng.standard_normal((k_p, d), dtype=np.float32)
            psample = pc[prng.integers(0, k_p, size=rows)] + HEADLINE["noise"] * prng.standard_normal((rows, d), dtype=np.float32)
            psample /= np.linalg.norm(psample, axis=1, keepdims=True)
            psample = np.ascontiguousarray(psample, dtype=np.float32)
            rcfg = ref.default_config(False, iters=iters, sampling_fraction=1.0, early_termination=0, seed=HEADLINE["seed"])
            kmp = ref.RefKMeans(k_p, d, rcfg)
            rcp = kmp.train(psample)
            e2 = skm.Engine(k_p, d, skm.default_config(False, **cfg_kw), device=local_rank)
            e2.set_rotation(kmp.rotation_matrix())
            c2 = e2.train(psample)
            a2, ra = e2.assign(psample, c2), kmp.assign(psample, rcp)
            w2 = float(((psample.astype(np.float64) - c2[a2]) ** 2).sum())
            rw = float(((psample.astype(np.float64) - rcp[ra]) ** 2).sum())
            parity = {"sample": f"{rows} rows, {k_p} mixture centres, same d and noise as the workload", "k": k_p, "prune_path": e2.last_prune_path, "wcss": w2,
                      "wcss_reference": rw, "wcss_rel_diff": abs(w2 - rw) / rw, "assignments_equal": float((a2 == ra).mean()),
                      "centroid_rel_l2": float(np.linalg.norm(c2 - rcp) / np.linalg.norm(rcp))}

    if rank == 0:
        line = {
            "metric": "train_points_iters_per_s", "value": value, "unit": "points*iters/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "train_s": ms_per_step / 1e3, "wall_ms_per_step": float(np.mean(walls)), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"flat Train n={n} d={d} k={k} iters={n_it} (Gaussian mixture, Zipf(1.1) sizes, unit rows, seed {HEADLINE['seed']})",
                       "rows_per_gpu": n_local, "l2": "inputs (rows_per_gpu*d*4 bytes) exceed L2; no explicit flush", "partial_d": [int(s.partial_d) for s in stats],
                       "not_pruned_pct": [round(float(s.not_pruned_pct), 6) for s in stats], "objective": float(stats[-1].objective)},
            "phases_ms_per_step": {name: v[0] / args.steps for name, v in phase_acc.items()},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "parity_on_sample": parity, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
