"""Autotune sweep: every kernel variant / ring depth / group height on one
problem size against cuBLAS, best first.  The counterpart of the reference's
tools/gemm_autotune.sh:38-90 (which walks `--list-catalog`, rebuilds each tile
and keeps the best TFLOPS): here the candidates are the B200 variants behind
the buffer entry points plus the catalog entry points by name.

    python -m oxcamlgpu_b200.autotune M N K [--element bf16|f32] [--repeat 10] [--warmup 3]

Timing protocol as in the reference's bench (bench/bench.py:186-212): CUDA
events, L2 flushed before every launch, median; one short cool-down before each
candidate's window (the reference passes --cooldown 1).  Like the reference's
sweep, which goes through its bench and so refuses to time a kernel whose
result is wrong (bench/bench.py:294-305), every candidate's output is checked
once before its window -- three sampled rows against the exact kernel (the
bit-exact restatement of the host loop) -- and a candidate that fails is
reported and dropped, not timed.
"""
from __future__ import annotations

import argparse
import statistics
import sys
import time

import torch

from . import catalog, gemm

BUFFER_VARIANTS = ("2cta_512x256", "2cta_256x512", "2cta_256x256", "2cta_256x128", "1cta_256x256", "1cta_128x256",
                   "1cta_256x128", "1cta_128x128")


def candidates(m: int, n: int, k: int, element: str):
    """(label, callable factory) pairs valid for this size."""
    out = [("auto (library default)", dict(variant="auto"))]
    if k >= 2048 and m <= 512:
        for v, splits in (("cluster_splitk_128x256", 4), ("cluster_splitk_128x256", 2),
                          ("cluster_splitk_128x128", 2), ("cluster_splitk_128x128", 4)):
            out.append((f"{v},splits={splits}", dict(variant=v, splits=splits)))
    for v in BUFFER_VARIANTS:
        for group in (8, 16):
            out.append((f"{v},group_m={group}", dict(variant=v, group_m=group)))
    out.append(("2cta_512x256,group_m=4", dict(variant="2cta_512x256", group_m=4)))
    out.append(("2cta_256x256,group_m=8,stages=5", dict(variant="2cta_256x256", group_m=8, stages=5)))
    if element == "bf16" and n % 4 == 0:
        for splits in (2, 4):
            out.append((f"splitk,splits={splits}", dict(variant="splitk", splits=splits)))
    names = [nm for nm in catalog.ENTRY_NAMES
             if (nm == "gemm_bf16_fast") == (element == "bf16")]
    for nm in names:
        tile, _ = catalog.kernel_tile(nm)
        if m % tile.bm or n % tile.bn or k % tile.bk:
            continue  # the reference skips sizes the tile does not divide (gemm_autotune.sh:49-52)
        out.append((f"entry:{nm}", nm))
    return out


def _median_ms(fn, slab, warmup: int, repeat: int, cooldown: float) -> float:
    torch.cuda.synchronize()
    time.sleep(cooldown)
    for _ in range(warmup):
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


def check_tolerance(element: str, k: int, a_max: float, b_max: float) -> float:
    """1e-5 * sqrt(K) * max|A| * max|B|, inputs rounded identically on both sides;
    5e-5 for TF32 with K >= 4096 (the matrix unit's truncating accumulator)."""
    scale = 5e-5 if (element != "bf16" and k >= 4096) else 1e-5
    return scale * (k ** 0.5) * a_max * b_max


def sweep(m: int, n: int, k: int, element: str = "bf16", warmup: int = 3, repeat: int = 10,
          cooldown: float = 1.0, seed: int = 0, std: float = 1.0, rejected: list | None = None):
    """Returns (cublas_ms, [(label, ms, tflops, fraction_of_cublas)] best first).
    Candidates whose result is outside the tolerance are appended to `rejected`
    as (label, error, tolerance) and left out of the table."""
    dev = torch.device("cuda", torch.cuda.current_device())
    dtype = torch.bfloat16 if element == "bf16" else torch.float32
    a = torch.empty(m, k, device=dev, dtype=dtype)
    bt = torch.empty(n, k, device=dev, dtype=dtype)
    if element == "bf16":
        gemm.fill_normal(a, seed, std, 0)
        gemm.fill_normal(bt, seed, std, m * k)
    else:
        gemm.fill_uniform(a, seed, 0)
        gemm.fill_uniform(bt, seed, m * k)
    c = torch.empty(m, n, device=dev, dtype=torch.float32)
    c_ref = torch.empty(m, n, device=dev, dtype=dtype)
    l2 = torch.cuda.get_device_properties(dev).L2_cache_size
    slab = torch.empty(max(2 * l2, 128 << 20), dtype=torch.int8, device=dev)
    torch.backends.cuda.matmul.allow_tf32 = True
    run = gemm.gemm_bf16 if element == "bf16" else gemm.gemm_tf32
    flops = 2.0 * m * n * k
    cublas_ms = _median_ms(lambda: torch.matmul(a, bt.t(), out=c_ref), slab, warmup, repeat, cooldown)
    sample = torch.tensor(sorted({0, m // 2, m - 1}), device=dev)
    exact = gemm.gemm_exact(a[sample].contiguous(), bt, gemm.INPUT_BF16 if element == "bf16" else gemm.INPUT_TF32)
    tol = check_tolerance(element, k, float(a.float().abs().max()), float(bt.float().abs().max()))
    rows = []
    for label, spec in candidates(m, n, k, element):
        if isinstance(spec, str):
            tile, eb = catalog.kernel_tile(spec)
            el = "bf16" if eb == 2 else "f32"
            a_map = gemm.encode_tensor_map_2d(a.data_ptr(), k, m, k * eb, tile.bk, tile.bm, el)
            b_map = gemm.encode_tensor_map_2d(bt.data_ptr(), k, n, k * eb, tile.bk, tile.bn, el)
            da, db = gemm.alloc_device_tensor_map(a_map), gemm.alloc_device_tensor_map(b_map)
            fn = lambda spec=spec, da=da, db=db: gemm.launch_catalog(spec, da, db, c, m, n, k)
        else:
            flags = gemm.make_flags(**spec)
            fn = lambda flags=flags: run(a, bt, c, flags=flags)
        try:
            c.fill_(float("nan"))
            fn()
            err = float((c[sample] - exact).abs().max())
            if not err <= tol:     # NaN included
                print(f"REJECTED {label}: result off by {err} (tolerance {tol}); not timed", file=sys.stderr)
                if rejected is not None:
                    rejected.append((label, err, tol))
                continue
            ms = _median_ms(fn, slab, warmup, repeat, cooldown)
        except Exception as exc:  # a variant may refuse a shape; the sweep goes on
            print(f"skip {label}: {exc}", file=sys.stderr)
            continue
        rows.append((label, ms, flops / ms * 1e-9, cublas_ms / ms))
    gemm.device_status()
    rows.sort(key=lambda r: r[1])
    return cublas_ms, rows


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("m", type=int)
    ap.add_argument("n", type=int)
    ap.add_argument("k", type=int)
    ap.add_argument("--element", choices=["bf16", "f32"], default="bf16")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=10)
    ap.add_argument("--cooldown", type=float, default=1.0)
    ap.add_argument("--std", type=float, default=1.0)
    args = ap.parse_args()
    torch.cuda.set_device(0)
    cublas_ms, rows = sweep(args.m, args.n, args.k, args.element, args.warmup, args.repeat, args.cooldown,
                            std=args.std)
    flops = 2.0 * args.m * args.n * args.k
    print(f"gemm_autotune: problem {args.m}x{args.n}x{args.k} ({args.element}); "
          f"cuBLAS {cublas_ms:.4f} ms {flops / cublas_ms * 1e-9:.1f} TFLOPS")
    print(f"  {'candidate':44s} {'ms':>9s} {'TFLOPS':>9s} {'% cuBLAS':>9s}")
    for label, ms, tf, frac in rows:
        print(f"  {label:44s} {ms:9.4f} {tf:9.1f} {100 * frac:9.1f}")
    if rows:
        print(f"BEST {rows[0][0]}  TFLOPS={rows[0][2]:.1f}  %cuBLAS={100 * rows[0][3]:.1f}")


if __name__ == "__main__":
    main()
