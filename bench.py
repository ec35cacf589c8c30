#!/usr/bin/env python3
"""Benchmark of the dense GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload bf16_8192|tf32_4096|tf32_8192|proj_a|proj_b|proj_c|cfg5] [--gather]

One "step" is one GEMM over one set of synthetic operands.  Default workload:
bf16 8192^3 (A row-major, B column-major = B^T[N,K] row-major, normal(0,1),
f32 accumulate/output) per GPU.  With N > 1 (launched by torchrun, one rank per
GPU) B and C are column-sharded and A replicated, each rank runs the same
8192^3 shard of a GEMM with N_total = 8192*N columns (weak scaling, no
data-path collective); `--workload cfg5` is the fixed M=32768 N=65536 K=8192
problem sharded over the ranks (strong scaling).

Protocol, after the reference's bench (bench/bench.py:32-34,176-212): CUDA-event
timing on the launching stream, an L2 flush (zero a slab of max(2*L2, 128 MiB))
before every step, at least 5 warm-up steps by default, correctness checked
before timing, operand re-layout outside the timed region.  cuBLAS
(torch.matmul, bf16 in/out as in the reference's comparison, bench.py:307-311)
is timed in the same run, interleaved.  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    # name: (kind, M, N, K, distribution, std, seed)
    "bf16_8192": ("bf16", 8192, 8192, 8192, "normal", 1.0, 2),
    "tf32_4096": ("tf32", 4096, 4096, 4096, "uniform", 1.0, 1),
    "tf32_8192": ("tf32", 8192, 8192, 8192, "uniform", 1.0, 1),
    "proj_a": ("bf16", 8192, 28672, 8192, "normal", 0.02, 3),
    "proj_b": ("bf16", 8192, 8192, 28672, "normal", 0.02, 3),
    "proj_c": ("bf16", 128, 8192, 8192, "normal", 0.02, 3),
    "cfg5": ("bf16", 32768, 65536, 8192, "normal", 1.0, 4),
}
# DRAM bytes (read + write) of one launch of the dominant kernel, from one ncu
# capture of the same kernel (profiles/umma_gemm_*.md); None = not captured.
NCU_TRAFFIC_BYTES = {"bf16_8192": 1.085e9, "tf32_4096": 0.247e9, "proj_c": 0.1406e9}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only)
    every 20 ms while the device-timed windows run."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20,
                 "sw_power_cap": 0x4, "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.samples.append((mhz, watts))
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            self._stop.wait(0.02)

    def __enter__(self):
        if self.nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread:
            self._thread.join(1.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        # "under load": samples drawing at least half of the largest power seen
        top = max(w for _, w in self.samples)
        load = [m for m, w in self.samples if w >= 0.5 * top] or [m for m, _ in self.samples]
        return {"sm_mhz": statistics.median(load), "sm_max_mhz": self.max_mhz,
                "power_w_max": round(top, 1), "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cpu_sample(kind: str, m: int, n: int, k: int, dist: str, std: float, seed: int, target_s: float,
               threads: int | None = None):
    """Prepare a bounded sample of the workload for the oracle (the C restatement
    of the reference's host triple loop, all host threads): `rows` rows of A
    against the first min(N, 2048) rows of B^T, sized from a short probe so one
    pass takes about `target_s` seconds.  Returns (run, a_sample, rows, n_sample,
    threads); run(a_sample) executes one pass."""
    import oracle
    from oxcamlgpu_b200 import synth
    threads = threads or oracle.max_threads()
    gen = (lambda cnt, off: synth.normal(seed, cnt, std, off)) if dist == "normal" else \
        (lambda cnt, off: synth.uniform_pm1(seed, cnt, off))
    n_s = min(n, 2048)
    bt = gen(n_s * k, m * k).reshape(n_s, k)
    if kind == "bf16":
        bt_in = oracle.to_bf16(bt)
        prep = oracle.to_bf16
        run = lambda aa: oracle.gemm_kmajor_bf16(aa, bt_in, threads=threads)
    else:
        bt_in = bt
        prep = lambda x: x
        run = lambda aa: oracle.gemm_kmajor(aa, bt_in, oracle.MODE_TF32, threads=threads)
    probe_rows = max(1, threads)
    a = prep(gen(probe_rows * k, 0).reshape(probe_rows, k))
    t0 = time.perf_counter()
    run(a)
    probe = time.perf_counter() - t0
    rows = int(min(m, max(probe_rows, round(probe_rows * target_s / max(probe, 1e-6)))))
    rows = max(threads, (rows // threads) * threads)
    a = prep(gen(rows * k, 0).reshape(rows, k))
    return run, a, rows, n_s, threads


def run_reference(args):
    """--impl reference: the reference's CPU implementation of the path (the
    oracle port of its host triple loop, OpenMP over output rows, all host
    threads), each step a bounded row sample of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind, m, n, k, dist, std, seed = WORKLOADS[args.workload]
    run, a_in, rows, n_s, threads = cpu_sample(kind, m, n, k, dist, std, seed, target_s=1.5)
    for _ in range(min(args.warmup, 1)):
        run(a_in)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        run(a_in)
        times.append(time.perf_counter() - t0)
    sec = sum(times) / len(times)
    tflops = 2.0 * rows * n_s * k / sec * 1e-12
    sample = f"{rows} of {m} rows of A against {n_s} of {n} rows of B^T ({rows}x{n_s}x{k}) per step, {threads} threads"
    line = {
        "impl": "reference", "metric": metric_name(args.workload), "value": tflops, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.workload == "cfg5" else "weak", "vs_baseline": None,
        "dtype": "bf16" if kind == "bf16" else "tf32", "data": "synthetic",
        "config": dict(workload_config(args.workload, args.gpus), variant=args.variant),
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def metric_name(workload: str) -> str:
    return {"bf16_8192": "bf16 GEMM TFLOPS @8192^3", "tf32_4096": "TF32 GEMM TFLOPS @4096^3",
            "tf32_8192": "TF32 GEMM TFLOPS @8192^3",
            "cfg5": "bf16 sharded GEMM TFLOPS M=32768 N=65536 K=8192"}.get(
                workload, f"bf16 GEMM TFLOPS {workload}")


def workload_config(workload: str, gpus: int) -> dict:
    kind, m, n, k, dist, std, seed = WORKLOADS[workload]
    if workload == "cfg5":
        shard = f"B^T and C column-sharded over {gpus} GPU(s), A replicated; strong scaling"
        per_gpu = [m, n // gpus, k]
    else:
        shard = ("single GPU" if gpus == 1 else
                 f"N_total = {n}*{gpus} columns, B^T and C column-sharded, A replicated; weak scaling")
        per_gpu = [m, n, k]
    return {"workload": workload, "kind": kind, "M": m, "N": n if workload == "cfg5" else n * gpus, "K": k,
            "per_gpu_mnk": per_gpu, "layout": "A[M,K] row-major, B column-major (B^T[N,K] K-major), C f32 row-major",
            "inputs": f"{dist}" + (f"(0,{std})" if dist == "normal" else "[-1,1)") + f" seed {seed}, counter-based generator",
            "sharding": shard,
            "l2": "flushed before every timed step (zeroing a slab of max(2*L2,128 MiB)); operands+C also exceed L2"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="bf16_8192")
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--stages", type=int, default=0)
    ap.add_argument("--group-m", type=int, default=0)
    ap.add_argument("--gather", action="store_true", help="also time a replicated C: NCCL all-gather vs the fused fan-out epilogue (N > 1)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-flush", action="store_true", help="back-to-back launches, no L2 flush")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from oxcamlgpu_b200 import build
    build.build_library()
    from oxcamlgpu_b200 import gemm, sharded

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N ranks with torchrun")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: there is no CPU path for --impl ours")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    kind, m, n_total, k, distname, std, seed = WORKLOADS[args.workload]
    if args.workload == "cfg5":
        parts = sharded.column_partition(n_total, world)
        n0, n1 = parts[rank]
        n = n1 - n0
        scaling = "strong"
        global_n = n_total
    else:
        n, n0 = n_total, rank * n_total
        scaling = "weak"
        global_n = n_total * world
    dtype = torch.bfloat16 if kind == "bf16" else torch.float32
    flags = gemm.make_flags(args.variant, stages=args.stages, group_m=args.group_m)

    # operands: A replicated (same seed/indices on every rank), this rank's rows of B^T
    a = torch.empty(m, k, device=dev, dtype=dtype)
    bt = torch.empty(n, k, device=dev, dtype=dtype)
    c = torch.empty(m, n, device=dev, dtype=torch.float32)
    if distname == "normal":
        gemm.fill_normal(a, seed, std, 0)
        gemm.fill_normal(bt, seed, std, m * k + n0 * k)
    else:
        gemm.fill_uniform(a, seed, 0)
        gemm.fill_uniform(bt, seed, m * k + n0 * k)
    run_gemm = (lambda: gemm.gemm_bf16(a, bt, c, flags=flags)) if kind == "bf16" else \
        (lambda: gemm.gemm_tf32(a, bt, c, flags=flags))

    # correctness before timing: sampled rows against the exact device kernel
    # (the bit-exact restatement of the host loop) -- the full oracle comparison
    # lives in tests/
    run_gemm()
    rows = torch.tensor([0, m // 2 + 1, m - 1], device=dev)
    exact = gemm.gemm_exact(a[rows].contiguous(), bt, gemm.INPUT_BF16 if kind == "bf16" else gemm.INPUT_TF32)
    err = float((c[rows] - exact).abs().max())
    tol = 5e-5 * (k ** 0.5) * float(a.float().abs().max()) * float(bt.float().abs().max())
    if not err <= tol:
        raise SystemExit(f"GEMM result off by {err} (tolerance {tol}): refusing to time a wrong kernel")
    gemm.device_status()

    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    slab = torch.empty(max(2 * l2, 128 << 20), dtype=torch.int8, device=dev)
    flush = (lambda: None) if args.no_flush else (lambda: slab.zero_())

    def timed_steps(fn, steps, warmup):
        for _ in range(warmup):
            flush()
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for s, e in evs:
            flush()
            s.record()
            fn()
            e.record()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        return [s.elapsed_time(e) for s, e in evs]

    def reduce_max(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    sampler = ClockSampler(local)
    launches0 = gemm.launch_count()
    sampler.__enter__()
    ours_ms = timed_steps(run_gemm, args.steps, args.warmup)
    launches = gemm.launch_count() - launches0 - args.warmup
    total_ms = reduce_max(sum(ours_ms))
    ms_per_step = total_ms / args.steps
    median_ms = reduce_max(statistics.median(ours_ms))
    flops_all = 2.0 * m * global_n * k
    value = flops_all / (ms_per_step * 1e-3) * 1e-12

    # cuBLAS in the same run (bf16 out for bf16, TF32-enabled f32 matmul for tf32)
    torch.backends.cuda.matmul.allow_tf32 = True
    c_ref = torch.empty(m, n, device=dev, dtype=dtype)
    bt_t = bt.t()
    cublas_ms = timed_steps(lambda: torch.matmul(a, bt_t, out=c_ref), args.steps, args.warmup)
    cublas_med = reduce_max(statistics.median(cublas_ms))
    cublas_mean = reduce_max(sum(cublas_ms) / args.steps)
    ours2_ms = timed_steps(run_gemm, args.steps, 2)        # second window after cuBLAS (interleaved)
    ours2_med = reduce_max(statistics.median(ours2_ms))
    cublas_f32_med = None
    if kind == "bf16":
        # the same work as ours: bf16 operands, f32 C (cuBLASLt through torch.mm's out_dtype)
        try:
            f32_ms = timed_steps(lambda: torch.mm(a, bt_t, out_dtype=torch.float32), args.steps, 3)
            cublas_f32_med = reduce_max(statistics.median(f32_ms))
        except Exception:
            cublas_f32_med = None
    out16_med = None
    if kind == "bf16":
        # the same work as cuBLAS's bf16-C path: the library's bf16-output entry point
        c16 = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        try:
            out16_ms = timed_steps(lambda: gemm.gemm_bf16_out16(a, bt, c16, flags=flags), args.steps, 3)
            out16_med = reduce_max(statistics.median(out16_ms))
        except Exception:
            out16_med = None      # the pinned variant has no bf16-output kernel
        del c16
    sampler.__exit__()
    del c_ref

    gather_ms = None
    gather = None
    if args.gather and world > 1:
        # A replicated row-major C, two ways.  Separate: GEMM, NCCL all-gather of the
        # shards, re-interleave of the gathered blocks.  Fused: the GEMM's fan-out
        # epilogue stores every tile into all ranks' C over NVLink as it is produced.
        g_steps = max(3, args.steps // 5)
        g_ms = timed_steps(lambda: sharded.all_gather_c(c), g_steps, 2)
        gather_ms = reduce_max(statistics.median(g_ms))
        sep_ms = timed_steps(lambda: (run_gemm(), sharded.blocks_to_row_major(sharded.all_gather_c(c))), g_steps, 2)
        sep_med = reduce_max(statistics.median(sep_ms))
        torch.cuda.empty_cache()
        fused = sharded.FusedGatherGemm(m, global_n, k, flags=flags)
        if (fused.n0, fused.n1) != (n0, n0 + n):
            raise SystemExit("fused gather: shard windows disagree with the bench's partition")
        fused_ms = timed_steps(lambda: fused.run(a, bt), g_steps, 2)
        fused_med = reduce_max(statistics.median(fused_ms))
        full = fused.finish()
        # every rank's window of this rank's replica against that rank's own C rows
        mine = c[rows].contiguous()
        theirs = torch.empty(world * rows.numel(), n, device=dev)
        dist.all_gather_into_tensor(theirs, mine)
        theirs = theirs.view(world, rows.numel(), n).permute(1, 0, 2).reshape(rows.numel(), world * n)
        if not float((full[rows] - theirs).abs().max()) <= tol:
            raise SystemExit("fused gather: replicated C disagrees with the ranks' own shards")
        recv_bytes = (world - 1) * m * n * 4
        gather = {"nccl_allgather_median_ms": gather_ms, "separate_gemm_allgather_interleave_median_ms": sep_med,
                  "fused_gemm_gather_median_ms": fused_med, "separate_over_fused": sep_med / fused_med,
                  "nvlink_in_bytes_per_gpu": recv_bytes,
                  "nvlink_bound_ms_at_770GBs": recv_bytes / 770e9 * 1e3,
                  "gemm_alone_median_ms": median_ms}
        del full, theirs
        fused.close()

    # end to end through the host-buffer entry point: pinned host operands in,
    # pinned host C out, every step
    e2e = None
    if not args.no_e2e and kind in ("bf16", "tf32"):
        a_h = torch.empty(m, k, dtype=dtype).pin_memory()
        bt_h = torch.empty(n, k, dtype=dtype).pin_memory()
        c_h = torch.empty(m, n, dtype=torch.float32).pin_memory()
        a_h.copy_(a)
        bt_h.copy_(bt)
        host_fn = gemm.gemm_bf16_host if kind == "bf16" else gemm.gemm_tf32_host
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(3):
            host_fn(a_h, bt_h, c_h, flags)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_fn(a_h, bt_h, c_h, flags)           # returns when C is on the host
        sec = time.perf_counter() - t0
        sec = reduce_max(sec)
        # (block-wise GEMMs may pick other tiles or K slicings than the whole problem:
        # same tolerance as against the exact kernel, not bit equality)
        if not float((c_h[rows.cpu()] - exact.cpu()).abs().max()) <= tol:
            raise SystemExit("host-buffer path disagrees with the exact kernel")
        e2e = {"value": flops_all / (sec / e2e_steps) * 1e-12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": (a_h.numel() + bt_h.numel()) * a_h.element_size(),
               "d2h_bytes_per_step": c_h.numel() * 4, "ms_per_step": sec / e2e_steps * 1e3,
               "steps": e2e_steps, "api": "oxgpu_b200_gemm_%s_host" % kind}
        del a_h, bt_h, c_h
    gemm.device_status()

    peaks = measured_peaks()
    peak = peaks["bf16_tflops"] if kind == "bf16" else peaks["bf16_tflops"] / 2.0
    per_launch_flops = 2.0 * m * n * k
    kernel_ms = sum(ours_ms) / len(ours_ms)            # this rank's average launch duration
    achieved = per_launch_flops / (kernel_ms * 1e-3) * 1e-12
    algorithmic_bytes = (m * k + n * k) * a.element_size() + m * n * 4
    ridge = peak * 1e12 / (peaks["hbm_gbs"] * 1e9)              # flop per byte where the two roofs meet
    if per_launch_flops / algorithmic_bytes >= ridge:
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                    "frac": achieved / peak,
                    "peak_source": ("burst cuBLAS bf16 8192^3 of %s" % peaks["source"]) +
                                   ("" if kind == "bf16" else " / 2 (no TF32 figure measured)")}
    else:                                                       # skinny shapes stream one operand
        gbs = algorithmic_bytes / (kernel_ms * 1e-3) / 1e9
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "peak_source": "copy bandwidth of %s" % peaks["source"]}
    roofline.update({
        "traffic": NCU_TRAFFIC_BYTES.get(args.workload),
        "algorithmic_bytes": algorithmic_bytes,
        "hbm_frac_of_measured": algorithmic_bytes / (kernel_ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
    })

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        run, a_in, nrows, n_s, threads = cpu_sample(kind, m, n, k, distname, std, seed, target_s=12.0)
        t0 = time.perf_counter()
        run(a_in)
        sec = time.perf_counter() - t0
        cpu = {"value": 2.0 * nrows * n_s * k / sec * 1e-12, "unit": "TFLOP/s", "cores": threads, "kind": "port",
               "sample": f"{nrows} of {m} rows of A against {n_s} of {n} rows of B^T in {sec:.1f} s; "
                         "the reference's triple loop restated in C, OpenMP over output rows",
               "extrapolated_full_problem_s": sec * (m / nrows) * (n / n_s)}

    if rank == 0:
        line = {
            "metric": metric_name(args.workload), "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "bf16" if kind == "bf16" else "tf32", "data": "synthetic",
            "config": dict(workload_config(args.workload, world), variant=args.variant),
            "median_ms": median_ms, "value_at_median": flops_all / (median_ms * 1e-3) * 1e-12,
            "cublas": {"what": "torch.matmul, same operands, %s out" % ("bf16" if kind == "bf16" else "f32 (TF32 on)"),
                       "median_ms": cublas_med, "mean_ms": cublas_mean,
                       "tflops_at_median": flops_all / (cublas_med * 1e-3) * 1e-12,
                       "ours_over_cublas_median": cublas_med / median_ms,
                       "ours_second_window_median_ms": ours2_med,
                       "ours_over_cublas_second_window": cublas_med / ours2_med,
                       "f32_out_median_ms": cublas_f32_med,
                       "ours_over_cublas_f32_out": (cublas_f32_med / median_ms) if cublas_f32_med else None,
                       "ours_bf16_out_median_ms": out16_med,
                       "ours_bf16_out_over_cublas": (cublas_med / out16_med) if out16_med else None},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": sampler.summary(),
            "check": {"max_abs_err_sampled_rows": err, "tolerance": tol},
        }
        if gather_ms is not None:
            line["allgather_c_median_ms"] = gather_ms
            line["gather"] = gather
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
