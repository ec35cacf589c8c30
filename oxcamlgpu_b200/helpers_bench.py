"""Throughput of the kernels around the GEMM -- operand re-layout (B -> B^T),
f32 -> bf16 conversion, the synthetic generators and the exact-f32 GEMM -- on
one B200, against the HBM copy rate.  These run outside the timed region of the
reference's bench (bench/bench.py:255-271) but are what a caller holding
row-major f32 data pays once per operand.

    python -m oxcamlgpu_b200.helpers_bench [--size 8192] [--repeat 10]
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import torch

from . import gemm


def _peak_gbs() -> float:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"])
    except Exception:
        return 6650.0  # the fallback copy rate when no measurement file is present


def _median_ms(fn, slab, repeat: int) -> float:
    for _ in range(3):
        slab.zero_()
        fn()
    torch.cuda.synchronize()
    evs = []
    for _ in range(repeat):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        slab.zero_()
        s.record()
        fn()
        e.record()
        evs.append((s, e))
    torch.cuda.synchronize()
    return statistics.median(s.elapsed_time(e) for s, e in evs)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=8192, help="matrices are size x size")
    ap.add_argument("--repeat", type=int, default=10)
    args = ap.parse_args()
    n = args.size
    dev = torch.device("cuda", torch.cuda.current_device())
    peak = _peak_gbs()
    slab = torch.empty(256 << 20, dtype=torch.int8, device=dev)  # L2 flush between launches
    f32 = torch.empty(n, n, device=dev)
    gemm.fill_uniform(f32, 1, 0)
    b16 = gemm.f32_to_bf16(f32)
    rows = []

    def report(name, nbytes, ms):
        gbs = nbytes / (ms * 1e-3) / 1e9
        rows.append((name, ms, gbs, gbs / peak))
        print(f"{name:34s} {ms:8.4f} ms {gbs:8.1f} GB/s  {100 * gbs / peak:5.1f} % of the copy rate", flush=True)

    report("transpose f32", 2 * n * n * 4, _median_ms(lambda: gemm.transpose(f32), slab, args.repeat))
    report("transpose bf16", 2 * n * n * 2, _median_ms(lambda: gemm.transpose(b16), slab, args.repeat))
    report("transpose + f32 -> bf16, one pass", n * n * 6,
           _median_ms(lambda: gemm.transpose_to_bf16(f32), slab, args.repeat))
    report("f32 -> bf16", n * n * 6, _median_ms(lambda: gemm.f32_to_bf16(f32), slab, args.repeat))
    report("fill uniform f32", n * n * 4, _median_ms(lambda: gemm.fill_uniform(f32, 1, 0), slab, args.repeat))
    report("fill normal bf16", n * n * 2, _median_ms(lambda: gemm.fill_normal(b16, 2, 1.0, 0), slab, args.repeat))
    report("torch copy f32 (for scale)", 2 * n * n * 4, _median_ms(lambda: f32.clone(), slab, args.repeat))
    # exact GEMM: CUDA-core bound (one multiply and one add per MAC, never fused)
    m = min(n, 2048)
    a = f32[:m, :m].contiguous()
    ms = _median_ms(lambda: gemm.gemm_exact(a, a, gemm.INPUT_NONE), slab, max(3, args.repeat // 3))
    print(f"{'exact f32 GEMM ' + str(m) + '^3':34s} {ms:8.4f} ms {2.0 * m ** 3 / ms * 1e-9:8.2f} TFLOP/s "
          "(2 rounded operations per MAC on the CUDA cores)", flush=True)
    # the same f32 problem on the tensor cores at close to f32 accuracy (three TF32 pieces over 3K)
    m2 = min(n, 4096)
    a2 = f32[:m2, :m2].contiguous()
    ws = torch.empty(gemm.lib().oxgpu_b200_f32_split_workspace_bytes(m2, m2, m2), dtype=torch.uint8, device=dev)
    ms = _median_ms(lambda: gemm.gemm_f32_split(a2, a2, workspace=ws), slab, max(3, args.repeat // 2))
    print(f"{'f32 split GEMM ' + str(m2) + '^3':34s} {ms:8.4f} ms {2.0 * m2 ** 3 / ms * 1e-9:8.2f} TFLOP/s "
          "of f32-equivalent work (split kernels + one TF32 GEMM over 3K)", flush=True)
    gemm.device_status()


if __name__ == "__main__":
    main()
