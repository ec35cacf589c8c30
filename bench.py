#!/usr/bin/env python3
"""Benchmark of the dense GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload bf16_8192|tf32_4096|tf32_8192|proj_a|proj_b|proj_c|bf16_16384|cfg5|helpers|profile]
                    [--case NAME] [--gather] [--no-flush] [--no-also] [--no-cfg5]

One "step" is one GEMM over one set of synthetic operands.  Default workload:
bf16 8192^3 (A row-major, B column-major = B^T[N,K] row-major, normal(0,1),
f32 accumulate/output) per GPU.  With N > 1 (launched by torchrun, one rank per
GPU) B and C are column-sharded and A replicated, each rank runs the same
8192^3 shard of a GEMM with N_total = 8192*N columns (weak scaling, no
data-path collective).

Every default line also carries
  * `cfg5`: the fixed problem M=32768 N=65536 K=8192 column-sharded over the N
    GPUs (strong scaling) through the library's one-process multi-GPU driver
    (oxgpu_b200_mg_gemm_bf16), run by rank 0 over all N devices while the other
    ranks wait on the host; for N > 1 with the replicated-C timings (NCCL
    all-gather against the fused peer-store epilogue);
  * at N = 1, `also`: TF32 8192^3, TF32 4096^3 and the three bf16 projection
    shapes, each with its cuBLAS ratio on the same work and its roofline.

Protocol, after the reference's bench (bench/bench.py:32-34,176-212,307-309):
CUDA-event timing on the launching stream, an L2 flush (zero a slab of
max(2*L2, 128 MiB)) before every step, at least 5 warm-up steps by default,
correctness checked before timing, operand re-layout outside the timed region,
a cool-down before each engine's window.  cuBLAS (torch.matmul / torch.mm) is
timed in the same run, between two windows of ours.  Rank 0 prints ONE JSON line.
"""
from __future__ import annotations

import argparse
import json
import math
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
    "bf16_16384": ("bf16", 16384, 16384, 8192, "normal", 1.0, 2),
    "cfg5": ("bf16", 32768, 65536, 8192, "normal", 1.0, 4),
}
# the short launches first: a launch of tens of microseconds measured right after seconds of
# power-capped work reads 1-2 us longer (both engines, not equally) than on a GPU that has idled
ALSO = ("proj_c", "tf32_4096", "tf32_8192", "proj_a", "proj_b")
# DRAM bytes (read + write) of one launch of the dominant kernel, from one ncu
# capture of the same kernel (profiles/umma_gemm_*.md); None = not captured.
NCU_TRAFFIC_BYTES = {"bf16_8192": 1.043e9, "tf32_4096": 0.247e9, "proj_c": 0.1406e9}
COOLDOWN_S = 1.0   # before each engine's window (the reference uses 3 s, bench/bench.py:307-309)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


def host_threads() -> int:
    """Host threads this process may use: the affinity mask, not OMP_NUM_THREADS
    (which torchrun sets to 1 for every rank)."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


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


def nvlink_rx_bytes(devices):
    """Bytes each device has received over NVLink so far (payload, all links
    summed), read through NVML's field queries -- counters only, nothing is set.
    Returns (list, None), or (None, reason) when the driver does not expose them."""
    try:
        import pynvml
        pynvml.nvmlInit()
        fid = pynvml.NVML_FI_DEV_NVLINK_THROUGHPUT_DATA_RX      # value in KiB
        out = []
        for d in devices:
            h = pynvml.nvmlDeviceGetHandleByIndex(d)
            v = pynvml.nvmlDeviceGetFieldValues(h, [(fid, 0xFFFFFFFF)])[0]   # scope: all links of the device
            if v.nvmlReturn == 0:
                out.append(int(v.value.ullVal) * 1024)
                continue
            total, seen = 0, 0
            for link in range(18):                                           # else link by link
                w = pynvml.nvmlDeviceGetFieldValues(h, [(fid, link)])[0]
                if w.nvmlReturn == 0:
                    total += int(w.value.ullVal) * 1024
                    seen += 1
            if not seen:
                return None, "NVML returned %d for the NVLink throughput field" % v.nvmlReturn
            out.append(total)
        return out, None
    except Exception as exc:                                                 # noqa: BLE001 - optional evidence
        return None, "%s: %s" % (type(exc).__name__, exc)


def cpu_sample(kind: str, m: int, n: int, k: int, dist: str, std: float, seed: int, target_s: float,
               threads: int | None = None):
    """Prepare a bounded sample of the workload for the oracle (the C restatement
    of the reference's host triple loop, all host threads): `rows` rows of A
    against the first min(N, 2048) rows of B^T, sized from a short probe so one
    pass takes about `target_s` seconds.  Returns (run, a_sample, rows, n_sample,
    threads); run(a_sample) executes one pass."""
    import oracle
    from oxcamlgpu_b200 import synth
    threads = threads or host_threads()
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
    oracle port of its host triple loop, OpenMP over output rows, every host
    thread the process may use), each step a bounded row sample of the same
    workload.  Under torchrun rank 0 alone runs it."""
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


def workload_config(workload: str, gpus: int, flush: bool = True) -> dict:
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
            "l2": ("flushed before every timed step (zeroing a slab of max(2*L2,128 MiB)); operands+C also exceed L2"
                   if flush else
                   "not flushed: back-to-back launches after 0.5 s of the same launches (sustained clocks); "
                   "operands+C exceed L2")}


def tolerance(kind: str, k: int, a_max: float, b_max: float) -> float:
    """1e-5 * sqrt(K) * max|A| * max|B| (inputs rounded identically on both
    sides); TF32 with K >= 4096 gets 5e-5 (the matrix unit's truncating
    accumulator: 1.9e-5 * sqrt(K) measured at 4096^3 uniform[-1,1))."""
    scale = 5e-5 if (kind == "tf32" and k >= 4096) else 1e-5
    return scale * math.sqrt(k) * a_max * b_max


def roofline_of(kind: str, m: int, n: int, k: int, kernel_ms: float, peaks: dict, traffic):
    peak = peaks["bf16_tflops"] if kind == "bf16" else peaks["bf16_tflops"] / 2.0
    flops = 2.0 * m * n * k
    esize = 2 if kind == "bf16" else 4
    achieved = flops / (kernel_ms * 1e-3) * 1e-12
    algorithmic_bytes = (m * k + n * k) * esize + m * n * 4
    ridge = peak * 1e12 / (peaks["hbm_gbs"] * 1e9)              # flop per byte where the two roofs meet
    gbs = algorithmic_bytes / (kernel_ms * 1e-3) / 1e9
    if flops / algorithmic_bytes >= ridge:
        r = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
             "peak_source": ("burst cuBLAS bf16 8192^3 of %s" % peaks["source"]) +
                            ("" if kind == "bf16" else " / 2 (no TF32 figure measured)")}
    else:                                                       # skinny shapes stream one operand
        r = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
             "frac": gbs / peaks["hbm_gbs"], "peak_source": "copy bandwidth of %s" % peaks["source"]}
    r.update({"traffic": traffic, "algorithmic_bytes": algorithmic_bytes,
              "hbm_frac_of_measured": gbs / peaks["hbm_gbs"]})
    return r


class Windows:
    """Device-timed windows on this rank's GPU: CUDA events on the current
    stream, an L2 flush before every step, max over ranks."""

    def __init__(self, torch, dist, dev, world, flush: bool):
        self.torch, self.dist, self.dev, self.world = torch, dist, dev, world
        l2 = torch.cuda.get_device_properties(dev).L2_cache_size
        self.slab = torch.empty(max(2 * l2, 128 << 20), dtype=torch.int8, device=dev)
        self.flush = (lambda: self.slab.zero_()) if flush else (lambda: None)
        # --no-flush is the sustained protocol: back-to-back launches, and every
        # window is preceded by half a second of the same launches, so each engine
        # is timed at the clock the power governor settles on for it (a window that
        # starts on a cool GPU drifts from boost to capped clocks while it is timed)
        self.preheat_s = 0.0 if flush else 0.5

    def sync(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def cooldown(self):
        self.torch.cuda.synchronize()
        if not self.preheat_s:
            time.sleep(COOLDOWN_S)

    def timed(self, fn, steps, warmup, counter=None):
        """Returns the per-step milliseconds; with `counter` (a function returning the
        library's launch count) self.launches is what the timed steps alone launched."""
        torch = self.torch
        if self.preheat_s:
            t0 = time.perf_counter()
            while time.perf_counter() - t0 < self.preheat_s:
                for _ in range(4):
                    fn()
                torch.cuda.synchronize()
        for _ in range(warmup):
            self.flush()
            fn()
        self.sync()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        before = counter() if counter else 0
        for s, e in evs:
            self.flush()
            s.record()
            fn()
            e.record()
        self.launches = (counter() - before) if counter else None
        self.sync()
        return [s.elapsed_time(e) for s, e in evs]

    def reduce_max(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t)


def make_operands(torch, gemm, dev, kind, m, n, k, distname, std, seed, n0=0):
    dtype = torch.bfloat16 if kind == "bf16" else torch.float32
    a = torch.empty(m, k, device=dev, dtype=dtype)
    bt = torch.empty(n, k, device=dev, dtype=dtype)
    if distname == "normal":
        gemm.fill_normal(a, seed, std, 0)
        gemm.fill_normal(bt, seed, std, m * k + n0 * k)
    else:
        gemm.fill_uniform(a, seed, 0)
        gemm.fill_uniform(bt, seed, m * k + n0 * k)
    return a, bt


def check_rows(torch, gemm, kind, a, bt, c):
    """Correctness before timing: sampled rows (first, middle, last) against the
    exact device kernel, the bit-exact restatement of the host loop
    (test/hardware/run_gemm_h100.cu:150-162); the comparison with the CPU oracle
    itself lives in tests/."""
    m, k = a.shape
    rows = torch.tensor(sorted({0, m // 2 + 1, m - 1}), device=a.device)
    exact = gemm.gemm_exact(a[rows].contiguous(), bt, gemm.INPUT_BF16 if kind == "bf16" else gemm.INPUT_TF32)
    err = float((c[rows] - exact).abs().max())
    tol = tolerance(kind, k, float(a.float().abs().max()), float(bt[:8192].float().abs().max()))
    if not err <= tol:
        raise SystemExit(f"GEMM result off by {err} (tolerance {tol}): refusing to time a wrong kernel")
    return rows, exact, err, tol


def cublas_same_work(torch, kind, a, bt_t, c_out):
    """cuBLAS doing the same work as ours: f32 C for both kinds (bf16 operands go
    through cuBLASLt's f32-output path)."""
    if kind == "bf16":
        return lambda: torch.mm(a, bt_t, out_dtype=torch.float32)
    return lambda: torch.matmul(a, bt_t, out=c_out)


def back_to_back(torch, run_ours, run_cublas, launches=20, rounds=5, replays=10):
    """Device time per launch when the same GEMM is launched `launches` times in a
    row with nothing between the launches (a CUDA graph of them, replayed): what a
    caller that chains kernels sees.  The library's kernels start their set-up
    under the tail of the kernel before them (programmatic dependent launch), which
    only shows here; a lone launch between two events pays the events instead.  No
    L2 flush inside the chain, so this is for operands larger than L2 only.  The
    two engines are measured in alternation, `rounds` times; medians."""
    def graph_of(fn):
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for _ in range(3):
                fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(launches):
                fn()
        return g

    def per_launch_us(g):
        for _ in range(2):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(replays):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) / launches * 1e3)
        return statistics.median(ts)

    graphs = {"ours": graph_of(run_ours), "cublas": graph_of(run_cublas)}
    seen = {k: [] for k in graphs}
    for _ in range(rounds):
        for k, g in graphs.items():
            seen[k].append(per_launch_us(g))
    ours, cub = statistics.median(seen["ours"]), statistics.median(seen["cublas"])
    return {"launches_per_graph": launches, "ours_us_per_launch": ours, "cublas_us_per_launch": cub,
            "ours_over_cublas": cub / ours, "l2": "not flushed inside the chain (operands larger than L2)"}


def central(ms_list):
    """Per-step time of a window.  The median, except for launches under 0.1 ms:
    CUDA events on some of these boxes tick every 2.048 us, a median of such
    readings is a multiple of the tick (36.9 or 38.9 us, nothing between), and a
    5 % step hides what is being compared.  The readings fall on either side of the
    tick at random, so their mean resolves below it; the mean of the middle 80 % is
    used (outliers dropped)."""
    med = statistics.median(ms_list)
    if med >= 0.1 or len(ms_list) < 10:
        return med
    xs = sorted(ms_list)
    cut = len(xs) // 10
    return statistics.fmean(xs[cut:len(xs) - cut])


def measure_also(torch, gemm, win, name, peaks, steps=10, warmup=5):
    """One extra workload on one GPU: ours, cuBLAS on the same work, ours again.
    Launches shorter than a millisecond get 40 steps after 100 warm-up steps, so
    that a window is neither over nor begun before the clocks have settled."""
    kind, m, n, k, distname, std, seed = WORKLOADS[name]
    if 2.0 * m * n * k < 1e12:
        steps, warmup = max(steps, 40), max(warmup, 100)   # (both engines; 100 flushed steps are 10-25 ms)
    if 2.0 * m * n * k < 1e11:
        steps = max(steps, 100)                            # under 0.1 ms: enough readings to average over the event tick
    a, bt = make_operands(torch, gemm, win.dev, kind, m, n, k, distname, std, seed)
    c = torch.empty(m, n, device=win.dev, dtype=torch.float32)
    run = (lambda: gemm.gemm_bf16(a, bt, c)) if kind == "bf16" else (lambda: gemm.gemm_tf32(a, bt, c))
    run()
    _, _, err, tol = check_rows(torch, gemm, kind, a, bt, c)
    win.cooldown()                                    # as before every other window
    ours = win.timed(run, steps, warmup)
    torch.backends.cuda.matmul.allow_tf32 = True
    bt_t = bt.t()
    c_ref = torch.empty(m, n, device=win.dev, dtype=torch.float32) if kind == "tf32" else None
    win.cooldown()
    try:
        cub = win.timed(cublas_same_work(torch, kind, a, bt_t, c_ref), steps, warmup)
        same = "f32 C"
    except Exception:                                 # no f32-output bf16 path in this torch: bf16 C
        c16 = torch.empty(m, n, device=win.dev, dtype=torch.bfloat16)
        cub = win.timed(lambda: torch.matmul(a, bt_t, out=c16), steps, warmup)
        same = "bf16 C (f32-output path unavailable)"
    win.cooldown()
    ours2 = win.timed(run, steps, 2)
    ms, ms2, cms = central(ours), central(ours2), central(cub)
    flops = 2.0 * m * n * k
    out = {"workload": name, "kind": kind, "mnk": [m, n, k], "steps": steps, "warmup": warmup,
           "median_ms": ms, "tflops": flops / (ms * 1e-3) * 1e-12,
           "second_window_median_ms": ms2,
           "per_step": "median" if statistics.median(ours) >= 0.1 else "mean of the middle 80 % (event tick, see central())",
           "cublas": {"what": "same operands, " + same, "median_ms": cms,
                      "tflops": flops / (cms * 1e-3) * 1e-12},
           "ours_over_cublas": cms / ms, "ours_over_cublas_second_window": cms / ms2,
           "roofline": roofline_of(kind, m, n, k, sum(ours) / len(ours), peaks, NCU_TRAFFIC_BYTES.get(name)),
           "check": {"max_abs_err_sampled_rows": err, "tolerance": tol}}
    operand_bytes = (m + n) * k * (2 if kind == "bf16" else 4) + m * n * 4
    if kind == "bf16" and ms < 0.1 and operand_bytes > torch.cuda.get_device_properties(win.dev).L2_cache_size:
        # a short kernel: also what it costs inside a chain of launches
        try:
            out["back_to_back"] = back_to_back(torch, run, cublas_same_work(torch, kind, a, bt_t, None))
        except Exception as exc:                      # graph capture of the f32-output matmul unavailable
            out["back_to_back"] = {"unavailable": str(exc)[:200]}
    del a, bt, c, c_ref
    torch.cuda.empty_cache()
    return out


def measure_cfg5(torch, gemm, ngpu: int, flags: int, peaks: dict, do_gather: bool, flush: bool):
    """M=32768 N=65536 K=8192 column-sharded over `ngpu` devices by the library's
    one-process driver.  Device time per step = max over devices of the driver's
    own event pair around each device's work; wall time is the host clock around
    launch + sync.  Runs in ONE process (rank 0) over all devices."""
    from oxcamlgpu_b200 import multi_gpu
    kind, m, n, k, distname, std, seed = WORKLOADS["cfg5"]
    flops = 2.0 * m * n * k
    out = {"workload": "cfg5", "mnk": [m, n, k], "n_gpus": ngpu, "scaling": "strong",
           "api": "oxgpu_b200_mg_gemm_bf16 (one process, one host thread and stream per device)"}

    def run_on(devices, steps_hint=None, gather_modes=()):
        g = len(devices)
        res = {}
        with multi_gpu.MultiGpu(devices=devices) as mg:
            parts = mg.partition(n)
            devs = [torch.device("cuda", d) for d in devices]
            a, bt, c, slabs = [], [], [], []
            for d, (lo, hi) in zip(devs, parts):
                with torch.cuda.device(d):
                    ai, bi = make_operands(torch, gemm, d, kind, m, hi - lo, k, distname, std, seed, n0=lo)
                    a.append(ai)
                    bt.append(bi)
                    c.append(torch.empty(m, hi - lo, device=d, dtype=torch.float32))
                    l2 = torch.cuda.get_device_properties(d).L2_cache_size
                    slabs.append(torch.empty(max(2 * l2, 128 << 20), dtype=torch.int8, device=d))

            def sync_all():
                for d in devs:
                    torch.cuda.synchronize(d)

            def step(gather=0, c_full=None):
                if flush:
                    for s in slabs:
                        s.zero_()
                sync_all()
                t0 = time.perf_counter()
                mg.gemm_bf16(a, bt, c, m, n, k, gather=gather, c_full=c_full, flags=flags)
                mg.sync()
                wall = (time.perf_counter() - t0) * 1e3
                total, gemm_only = mg.elapsed_ms()
                return max(total), max(gemm_only), wall

            step()
            with torch.cuda.device(devs[-1]):                       # the shard holding column N-1, row M-1 included
                _, _, err, tol = check_rows(torch, gemm, kind, a[-1], bt[-1], c[-1])
            first = step()[0]
            steps = steps_hint or int(min(200, max(10, math.ceil(600.0 / max(first, 1e-3)))))
            for _ in range(2):
                step()
            samplers = [ClockSampler(d) for d in devices]
            for s in samplers:
                s.__enter__()
            runs = [step() for _ in range(steps)]
            for s in samplers:
                s.__exit__()
            dev_ms = statistics.median(r[0] for r in runs)
            wall_ms = statistics.median(r[2] for r in runs)
            clocks = [s.summary() for s in samplers]
            mhz = [cl["sm_mhz"] for cl in clocks if cl["sm_mhz"]]
            res.update({"median_ms": dev_ms, "mean_ms": sum(r[0] for r in runs) / len(runs),
                        "wall_median_ms": wall_ms, "steps": steps,
                        "value": flops / (dev_ms * 1e-3) * 1e-12, "unit": "TFLOP/s",
                        "value_wall": flops / (wall_ms * 1e-3) * 1e-12,
                        "per_gpu_mnk": [m, parts[0][1] - parts[0][0], k],
                        "sm_mhz_median_under_load": statistics.mean(mhz) if mhz else None,
                        "clock_reasons": sorted({r for cl in clocks for r in cl["reasons"]}),
                        "check": {"max_abs_err_sampled_rows": err, "tolerance": tol},
                        "timing": "max over devices of the driver's CUDA-event pair around each device's work; "
                                  + ("L2 flushed on every device before every step" if flush else "no L2 flush")})
            res["roofline"] = {"bound": "tensor", "achieved": res["value"] / g, "peak": peaks["bf16_tflops"],
                               "peak_sustained": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s per GPU",
                               "frac": res["value"] / g / peaks["bf16_tflops"],
                               "frac_of_sustained": (res["value"] / g / peaks["bf16_tflops_sustained"])
                               if peaks["bf16_tflops_sustained"] else None}
            # cuBLAS on device 0's shard, same work (f32 C) and its default (bf16 C)
            with torch.cuda.device(devs[0]):
                d0 = devs[0]
                bt_t = bt[0].t()

                def window(fn, nsteps):
                    for _ in range(3):
                        if flush:
                            slabs[0].zero_()
                        fn()
                    torch.cuda.synchronize(d0)
                    evs = []
                    for _ in range(nsteps):
                        if flush:
                            slabs[0].zero_()
                        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                        s.record()
                        fn()
                        e.record()
                        evs.append((s, e))
                    torch.cuda.synchronize(d0)
                    return statistics.median(s.elapsed_time(e) for s, e in evs)
                time.sleep(COOLDOWN_S)
                csteps = min(steps, 20)
                try:
                    f32_ms = window(lambda: torch.mm(a[0], bt_t, out_dtype=torch.float32), csteps)
                except Exception:
                    f32_ms = None
                c16 = torch.empty(m, parts[0][1] - parts[0][0], device=d0, dtype=torch.bfloat16)
                bf16_ms = window(lambda: torch.matmul(a[0], bt_t, out=c16), csteps)
                del c16
                time.sleep(COOLDOWN_S)
                ours0_ms = window(lambda: gemm.gemm_bf16(a[0], bt[0], c[0], flags=flags), csteps)
                res["cublas_shard_device0"] = {
                    "f32_out_median_ms": f32_ms, "bf16_out_median_ms": bf16_ms, "ours_median_ms": ours0_ms,
                    "ours_over_cublas": (f32_ms / ours0_ms) if f32_ms else None,
                    "ours_over_cublas_bf16_out": bf16_ms / ours0_ms}
            # replicated row-major C: NCCL all-gather + re-interleave against the fused epilogue
            if gather_modes and g > 1:
                recv = (g - 1) * m * (n // g) * 4
                gat = {"nvlink_in_bytes_per_gpu": recv, "nvlink_bound_ms_at_770GBs": recv / 770e9 * 1e3,
                       "gemm_alone_median_ms": dev_ms}
                full = []
                for d in devs:
                    with torch.cuda.device(d):
                        full.append(torch.empty(m, n, device=d, dtype=torch.float32))
                rows = torch.tensor([0, m // 2 + 1, m - 1])
                mine = torch.cat([ci[rows.to(ci.device)].cpu() for ci in c], dim=1)    # the shards' own rows
                for mode in gather_modes:
                    if mode == "fused" and not mg.peer_access:
                        gat["fused"] = "no peer access between the devices"
                        continue
                    for f in full:
                        f.zero_()
                    for _ in range(2):
                        step(gather=mode, c_full=full)
                    rx0, why = nvlink_rx_bytes(devices)
                    gruns = [step(gather=mode, c_full=full) for _ in range(5)]
                    rx1, why1 = nvlink_rx_bytes(devices)
                    if not (rx0 and rx1):
                        gat["nvlink_counters"] = "unavailable (%s)" % (why or why1)
                    if rx0 and rx1:
                        # NVLink payload bytes into each GPU per step, from the driver's counters,
                        # beside the (g-1)/g of C that must arrive
                        per_step = [(b - a0) / 5.0 for a0, b in zip(rx0, rx1)]
                        gat[mode + "_nvlink_rx_bytes_per_gpu_per_step"] = {"min": min(per_step), "max": max(per_step),
                                                                           "expected": recv}
                    ok = all(bool(torch.equal(f[rows.to(f.device)].cpu(), mine)) for f in full)
                    if not ok:
                        raise SystemExit(f"replicated C ({mode}) disagrees with the shards")
                    gat[mode + "_median_ms"] = statistics.median(r[0] for r in gruns)
                    gat[mode + "_gemm_part_median_ms"] = statistics.median(r[1] for r in gruns)
                if "nccl_median_ms" in gat and "fused_median_ms" in gat:
                    gat["separate_over_fused"] = gat["nccl_median_ms"] / gat["fused_median_ms"]
                    bound = max(gat["nvlink_bound_ms_at_770GBs"], dev_ms)
                    gat["fused_frac_of_bound"] = bound / gat["fused_median_ms"]
                res["gather"] = gat
                del full
            del a, bt, c, slabs
        for d in devices:
            with torch.cuda.device(d):
                torch.cuda.empty_cache()
        return res

    out.update(run_on(list(range(ngpu)), gather_modes=("nccl", "fused") if do_gather else ()))
    if ngpu > 1:
        one = run_on([0], steps_hint=8)
        out["one_gpu_same_run"] = {k2: one[k2] for k2 in ("median_ms", "value", "sm_mhz_median_under_load",
                                                          "clock_reasons", "cublas_shard_device0")}
        out["speedup_vs_one_gpu"] = one["median_ms"] / out["median_ms"]
        if one["sm_mhz_median_under_load"] and out["sm_mhz_median_under_load"]:
            # the one-GPU launch runs at the power-capped clock, the short shards near boost:
            # compare time x clock (cycles) as well as time
            out["speedup_clock_normalised"] = (one["median_ms"] * one["sm_mhz_median_under_load"]) / \
                                              (out["median_ms"] * out["sm_mhz_median_under_load"])
    return out


def pcie_rates(torch, dev, a_h, c_h, reps=4):
    """Pinned-memory copy rates of this process, both directions at once (the
    host-operand entry point keeps both busy): GB/s up, GB/s down."""
    up = torch.empty(a_h.numel() * a_h.element_size(), dtype=torch.uint8, device=dev)
    down = torch.empty(c_h.numel() * c_h.element_size(), dtype=torch.uint8, device=dev)
    a_b, c_b = a_h.view(torch.uint8).view(-1), c_h.view(torch.uint8).view(-1)
    s_up, s_down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    best = [0.0, 0.0]
    for _ in range(reps):
        torch.cuda.synchronize()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
        with torch.cuda.stream(s_up):
            e[0].record()
            up.copy_(a_b, non_blocking=True)
            e[1].record()
        with torch.cuda.stream(s_down):
            e[2].record()
            c_b.copy_(down, non_blocking=True)
            e[3].record()
        torch.cuda.synchronize()
        best[0] = max(best[0], up.numel() / (e[0].elapsed_time(e[1]) * 1e-3) / 1e9)
        best[1] = max(best[1], down.numel() / (e[2].elapsed_time(e[3]) * 1e-3) / 1e9)
    return best


def run_helpers(torch, gemm, dev, peaks, size=8192, repeat=10):
    """--workload helpers: the kernels either side of the GEMM (operand re-layout,
    conversion, generators, the exact and split-f32 GEMMs) against the copy rate."""
    slab = torch.empty(256 << 20, dtype=torch.int8, device=dev)

    def median_ms(fn, reps):
        for _ in range(3):
            slab.zero_()
            fn()
        torch.cuda.synchronize()
        evs = []
        for _ in range(reps):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            slab.zero_()
            s.record()
            fn()
            e.record()
            evs.append((s, e))
        torch.cuda.synchronize()
        return statistics.median(s.elapsed_time(e) for s, e in evs)
    n = size
    f32 = torch.empty(n, n, device=dev)
    gemm.fill_uniform(f32, 1, 0)
    b16 = gemm.f32_to_bf16(f32)
    rows = []

    def report(name, nbytes, ms):
        gbs = nbytes / (ms * 1e-3) / 1e9
        rows.append({"kernel": name, "ms": ms, "GB/s": gbs, "frac_of_copy_rate": gbs / peaks["hbm_gbs"]})
    report("transpose f32", 2 * n * n * 4, median_ms(lambda: gemm.transpose(f32), repeat))
    report("transpose bf16", 2 * n * n * 2, median_ms(lambda: gemm.transpose(b16), repeat))
    report("transpose + f32 -> bf16, one pass", n * n * 6, median_ms(lambda: gemm.transpose_to_bf16(f32), repeat))
    report("f32 -> bf16", n * n * 6, median_ms(lambda: gemm.f32_to_bf16(f32), repeat))
    report("fill uniform f32", n * n * 4, median_ms(lambda: gemm.fill_uniform(f32, 1, 0), repeat))
    report("fill normal bf16", n * n * 2, median_ms(lambda: gemm.fill_normal(b16, 2, 1.0, 0), repeat))
    report("torch copy f32 (for scale)", 2 * n * n * 4, median_ms(lambda: f32.clone(), repeat))
    m = min(n, 2048)
    a = f32[:m, :m].contiguous()
    ms = median_ms(lambda: gemm.gemm_exact(a, a, gemm.INPUT_NONE), max(3, repeat // 3))
    rows.append({"kernel": f"exact f32 GEMM {m}^3", "ms": ms, "TFLOP/s": 2.0 * m ** 3 / ms * 1e-9})
    m2 = min(n, 4096)
    a2 = f32[:m2, :m2].contiguous()
    ws = torch.empty(gemm.lib().oxgpu_b200_f32_split_workspace_bytes(m2, m2, m2), dtype=torch.uint8, device=dev)
    ms = median_ms(lambda: gemm.gemm_f32_split(a2, a2, workspace=ws), max(3, repeat // 2))
    rows.append({"kernel": f"f32 split GEMM {m2}^3 (three TF32 pieces over 3K)", "ms": ms,
                 "TFLOP/s f32-equivalent": 2.0 * m2 ** 3 / ms * 1e-9})
    gemm.device_status()
    print(json.dumps({"metric": "helper kernels around the GEMM", "size": n, "unit": "GB/s",
                      "peak_hbm_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"], "kernels": rows}), flush=True)


PROFILE_CASES = ("entry_bf16_fast", "out16", "affine", "fanout8", "tf32_8192", "proj_a", "proj_b", "big_dynamic",
                 "big_static")


def run_profile_case(torch, gemm, dev, case: str, launches: int):
    """--workload profile --case NAME: a few plain launches of one instantiation on
    a small problem (a few GB at most), nothing timed -- the command an `ncu`
    capture wraps.  entry_bf16_fast: the catalog entry `gemm_bf16_fast` with the
    reference's own maps (runs the 256 x 512 pair tile); out16: bf16 C; affine:
    alpha, beta * C_in and a bias row; fanout8: eight local destinations per tile;
    tf32_8192, proj_a, proj_b: the default kernel on those shapes; big_dynamic /
    big_static: 16384 x 32768 x 8192 with the queue-driven and the fixed-stride
    tile schedule."""
    shapes = {"tf32_8192": WORKLOADS["tf32_8192"][1:4], "proj_a": WORKLOADS["proj_a"][1:4],
              "proj_b": WORKLOADS["proj_b"][1:4], "big_dynamic": (16384, 32768, 8192),
              "big_static": (16384, 32768, 8192)}
    m, n, k = shapes.get(case, (4096, 4096, 4096))
    kind = "tf32" if case == "tf32_8192" else "bf16"
    a, bt = make_operands(torch, gemm, dev, kind, m, n, k, "normal" if kind == "bf16" else "uniform", 1.0, 7)
    if case == "big_static":
        os.environ["OXGPU_TILE_SCHEDULE"] = "static"
    if case == "entry_bf16_fast":
        c = torch.empty(m, n, device=dev)
        run = lambda: gemm.run_catalog_entry("gemm_bf16_fast", a, bt, c)
    elif case == "out16":
        c = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        run = lambda: gemm.gemm_bf16_out16(a, bt, c)
    elif case == "affine":
        c = torch.empty(m, n, device=dev)
        c_in = torch.ones(m, n, device=dev)
        bias = torch.ones(n, device=dev)
        run = lambda: gemm.gemm_affine(a, bt, c, alpha=2.0, beta=0.5, bias=bias, c_in=c_in)
    elif case == "fanout8":
        dests = [torch.empty(m, n, device=dev) for _ in range(8)]
        run = lambda: gemm.gemm_fanout(a, bt, dests)
    elif kind == "tf32":
        c = torch.empty(m, n, device=dev)
        run = lambda: gemm.gemm_tf32(a, bt, c)
    else:
        c = torch.empty(m, n, device=dev)
        run = lambda: gemm.gemm_bf16(a, bt, c)
    for _ in range(launches):
        run()
    if case.startswith("big_"):           # the vendor library on the same operands, for the same counters
        torch.mm(a, bt.t(), out_dtype=torch.float32)
    torch.cuda.synchronize()
    gemm.device_status()
    print(json.dumps({"profile_case": case, "mnk": [m, n, k], "launches": launches}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS) + ["helpers", "profile"], default="bf16_8192")
    ap.add_argument("--case", choices=PROFILE_CASES, default="out16", help="with --workload profile")
    ap.add_argument("--variant", default="auto")
    ap.add_argument("--stages", type=int, default=0)
    ap.add_argument("--group-m", type=int, default=0)
    ap.add_argument("--reorder", type=int, default=0)
    ap.add_argument("--gather", action="store_true", help="also time a replicated C: NCCL all-gather vs the fused fan-out epilogue (N > 1)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-also", action="store_true", help="skip the extra single-GPU workloads of the default line")
    ap.add_argument("--no-cfg5", action="store_true", help="skip the sharded M=32768 N=65536 K=8192 object")
    ap.add_argument("--no-flush", action="store_true", help="back-to-back launches, no L2 flush")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.workload in ("helpers", "profile") and args.impl == "reference":
        raise SystemExit("--workload %s has no reference arm" % args.workload)

    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from oxcamlgpu_b200 import build
    build.build_library()
    from oxcamlgpu_b200 import gemm, multi_gpu, sharded

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch N ranks with torchrun")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: there is no CPU path for --impl ours")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    host_group = None
    if world > 1:
        os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")    # single node; the host name may not resolve
        dist.init_process_group("nccl", device_id=dev)
        host_group = dist.new_group(backend="gloo")      # waits that must not put a kernel on a GPU
    peaks = measured_peaks()
    if args.workload == "helpers":
        return run_helpers(torch, gemm, dev, peaks)
    if args.workload == "profile":
        return run_profile_case(torch, gemm, dev, args.case, max(1, min(args.steps, 5)))

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
    flags = gemm.make_flags(args.variant, stages=args.stages, group_m=args.group_m, reorder=args.reorder)

    # operands: A replicated (same seed/indices on every rank), this rank's rows of B^T
    a, bt = make_operands(torch, gemm, dev, kind, m, n, k, distname, std, seed, n0=n0)
    c = torch.empty(m, n, device=dev, dtype=torch.float32)
    run_gemm = (lambda: gemm.gemm_bf16(a, bt, c, flags=flags)) if kind == "bf16" else \
        (lambda: gemm.gemm_tf32(a, bt, c, flags=flags))

    run_gemm()
    rows, exact, err, tol = check_rows(torch, gemm, kind, a, bt, c)
    gemm.device_status()

    win = Windows(torch, dist, dev, world, flush=not args.no_flush)
    timed_steps, reduce_max = win.timed, win.reduce_max

    sampler = ClockSampler(local)
    sampler.__enter__()
    ours_ms = timed_steps(run_gemm, args.steps, args.warmup, counter=gemm.launch_count)
    launches = win.launches
    total_ms = reduce_max(sum(ours_ms))
    ms_per_step = total_ms / args.steps
    median_ms = reduce_max(central(ours_ms))
    flops_all = 2.0 * m * global_n * k
    value = flops_all / (ms_per_step * 1e-3) * 1e-12

    # cuBLAS in the same run (bf16 out for bf16, TF32-enabled f32 matmul for tf32)
    torch.backends.cuda.matmul.allow_tf32 = True
    c_ref = torch.empty(m, n, device=dev, dtype=dtype)
    bt_t = bt.t()
    win.cooldown()
    cublas_ms = timed_steps(lambda: torch.matmul(a, bt_t, out=c_ref), args.steps, args.warmup)
    cublas_med = reduce_max(central(cublas_ms))
    cublas_mean = reduce_max(sum(cublas_ms) / args.steps)
    win.cooldown()
    ours2_ms = timed_steps(run_gemm, args.steps, 2)        # second window after cuBLAS (interleaved)
    ours2_med = reduce_max(central(ours2_ms))
    cublas_f32_med = None
    if kind == "bf16":
        # the same work as ours: bf16 operands, f32 C (cuBLASLt through torch.mm's out_dtype)
        try:
            win.cooldown()
            f32_ms = timed_steps(lambda: torch.mm(a, bt_t, out_dtype=torch.float32), args.steps, 3)
            cublas_f32_med = reduce_max(central(f32_ms))
        except Exception:
            cublas_f32_med = None
    out16_med = None
    if kind == "bf16":
        # the same work as cuBLAS's bf16-C path: the library's bf16-output entry point
        c16 = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        try:
            win.cooldown()
            out16_ms = timed_steps(lambda: gemm.gemm_bf16_out16(a, bt, c16, flags=flags), args.steps, 3)
            out16_med = reduce_max(central(out16_ms))
        except Exception:
            out16_med = None      # the pinned variant has no bf16-output kernel
        del c16
    sampler.__exit__()
    del c_ref

    gather_ms = None
    gather = None
    if args.gather and world > 1:
        # A replicated row-major C through the one-process-per-GPU wrapper.  Separate:
        # GEMM, NCCL all-gather of the shards, re-interleave of the gathered blocks.
        # Fused: the GEMM's fan-out epilogue stores every tile into all ranks' C over
        # NVLink as it is produced.
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
    # pinned host C out, every step.  The buffers sit on the NUMA node of this
    # rank's GPU (oxgpu_b200_host_alloc).
    e2e = None
    if not args.no_e2e and kind in ("bf16", "tf32"):
        es = a.element_size()
        bufs = [multi_gpu.PinnedHostBuffer(m * k * es, local), multi_gpu.PinnedHostBuffer(n * k * es, local),
                multi_gpu.PinnedHostBuffer(m * n * 4, local)]
        a_h = bufs[0].tensor((m, k), dtype)
        bt_h = bufs[1].tensor((n, k), dtype)
        c_h = bufs[2].tensor((m, n), torch.float32)
        a_h.copy_(a)
        bt_h.copy_(bt)
        host_fn = gemm.gemm_bf16_host if kind == "bf16" else gemm.gemm_tf32_host
        e2e_steps = max(3, min(args.steps, 10))
        for _ in range(3):
            host_fn(a_h, bt_h, c_h, flags)
        win.sync()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_fn(a_h, bt_h, c_h, flags)           # returns when C is on the host
        sec = time.perf_counter() - t0
        sec = reduce_max(sec)
        # (block-wise GEMMs may pick other tiles or K slicings than the whole problem:
        # same tolerance as against the exact kernel, not bit equality)
        if not float((c_h[rows.cpu()] - exact.cpu()).abs().max()) <= tol:
            raise SystemExit("host-buffer path disagrees with the exact kernel")
        h2d = (a_h.numel() + bt_h.numel()) * es
        d2h = c_h.numel() * 4
        # what PCIe allows: both directions measured at once, on every rank at the same time
        win.sync()
        up_gbs, down_gbs = pcie_rates(torch, dev, a_h, c_h)
        up_gbs, down_gbs = -reduce_max(-up_gbs), -reduce_max(-down_gbs)      # the slowest rank's rates
        bound_ms = max(h2d / (up_gbs * 1e9), d2h / (down_gbs * 1e9)) * 1e3
        e2e = {"value": flops_all / (sec / e2e_steps) * 1e-12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": sec / e2e_steps * 1e3,
               "steps": e2e_steps, "api": "oxgpu_b200_gemm_%s_host" % kind,
               "host_memory": "pinned, placed on the GPU's NUMA node (oxgpu_b200_host_alloc)",
               "pcie_gbs_duplex_slowest_rank": {"h2d": up_gbs, "d2h": down_gbs},
               "bound_ms": bound_ms, "frac_of_bound": bound_ms / (sec / e2e_steps * 1e3),
               "bound": "max(H2D bytes / H2D rate, D2H bytes / D2H rate), both directions busy, all ranks at once"}
        if kind == "bf16":
            # the same call with bf16 C: half the bytes come back, the upload alone bounds it
            c16_buf = multi_gpu.PinnedHostBuffer(m * n * 2, local)
            c16_h = c16_buf.tensor((m, n), torch.bfloat16)
            for _ in range(2):
                gemm.gemm_bf16_out16_host(a_h, bt_h, c16_h, flags)
            win.sync()
            t0 = time.perf_counter()
            for _ in range(e2e_steps):
                gemm.gemm_bf16_out16_host(a_h, bt_h, c16_h, flags)
            sec16 = reduce_max(time.perf_counter() - t0)
            ok16 = float((c16_h[rows.cpu()].float() - exact.cpu()).abs().max()) <= tol + float(exact.abs().max()) * 2.0 ** -8
            if not ok16:
                raise SystemExit("host-buffer path with bf16 C disagrees with the exact kernel")
            e2e["bf16_out"] = {"api": "oxgpu_b200_gemm_bf16_out16_host", "ms_per_step": sec16 / e2e_steps * 1e3,
                               "value": flops_all / (sec16 / e2e_steps) * 1e-12, "d2h_bytes_per_step": m * n * 2,
                               "bound_ms": max(h2d / (up_gbs * 1e9), m * n * 2 / (down_gbs * 1e9)) * 1e3}
            del c16_h
            c16_buf.free()
        del a_h, bt_h, c_h
        for b in bufs:
            b.free()
    gemm.device_status()

    kernel_ms = sum(ours_ms) / len(ours_ms)            # this rank's average launch duration
    roofline = roofline_of(kind, m, n, k, kernel_ms, peaks, NCU_TRAFFIC_BYTES.get(args.workload))

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

    default_line = args.workload == "bf16_8192"
    also = None
    if default_line and world == 1 and not args.no_also:
        del a, bt, c
        a = bt = c = None
        torch.cuda.empty_cache()
        also = [measure_also(torch, gemm, win, name, peaks) for name in ALSO]

    cfg5 = None
    if default_line and not args.no_cfg5:
        # One process (rank 0) drives all N devices through the library's driver; the
        # other ranks free their memory and wait ON THE HOST (a gloo barrier), so none
        # of their kernels shares a GPU with the driver's.
        a = bt = c = None
        win.slab = None
        torch.cuda.empty_cache()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier(group=host_group)
        if rank == 0:
            cfg5 = measure_cfg5(torch, gemm, world, flags, peaks, do_gather=world > 1, flush=not args.no_flush)
        if world > 1:
            dist.barrier(group=host_group)
        torch.cuda.set_device(local)

    if rank == 0:
        line = {
            "metric": metric_name(args.workload), "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "bf16" if kind == "bf16" else "tf32", "data": "synthetic",
            "config": dict(workload_config(args.workload, world, not args.no_flush), variant=args.variant),
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
                       "ours_bf16_out_over_cublas": (cublas_med / out16_med) if out16_med else None,
                       "cooldown_s_before_each_window": COOLDOWN_S},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": sampler.summary(),
            "check": {"max_abs_err_sampled_rows": err, "tolerance": tol},
        }
        if also is not None:
            line["also"] = also
        if cfg5 is not None:
            line["cfg5"] = cfg5
        if gather_ms is not None:
            line["allgather_c_median_ms"] = gather_ms
            line["gather"] = gather
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier(group=host_group)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
