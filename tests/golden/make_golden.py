"""Generate the committed fixtures under tests/golden/.

    python tests/golden/make_golden.py --reference /path/to/reference/checkout

1. Builds the reference's own host harness (test/hardware/run_gemm_h100.cu)
   against the fake CUDA driver (oracle/build.py) and runs both of its cases.
   The harness compares its CPU-computed expectation with the ORACLE's output;
   the fake driver reports every difference exactly.  The outcome is recorded
   in reference_pin.json -- zero differences means the oracle is bit-identical
   to the reference's host GEMM, so the vectors below are reference outputs.
2. Writes known-answer vectors produced by the oracle.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402
from oracle import build as obuild  # noqa: E402
from oxcamlgpu_b200 import synth  # noqa: E402


def gpu_header_rejections(reference: str) -> list[dict]:
    """The `.gpu` texts the reference's own tests require Gpu_metadata.parse to
    reject: the string literals handed to `parse_fails` in test/test_frontend.ml
    and the `malformed` literal of test/check_compiler_metadata.ml, read from the
    reference's test sources as text and unescaped as OCaml does."""
    import re
    out = []
    for rel, pattern in (("test/test_frontend.ml", r'parse_fails "((?:[^"\\]|\\.)*)";'),
                         ("test/check_compiler_metadata.ml", r'let malformed = "((?:[^"\\]|\\.)*)" in')):
        path = os.path.join(reference, rel)
        for no, line in enumerate(open(path, encoding="utf-8"), 1):
            for lit in re.findall(pattern, line):
                text = lit.replace("\\t", "\t").replace("\\n", "\n").replace('\\"', '"')
                out.append({"source": f"{rel}:{no}", "text": text})
    if len(out) < 5:
        raise SystemExit("expected at least five rejected .gpu vectors in the reference's tests")
    return out


def run_pin(reference: str) -> list[dict]:
    exe = obuild.build_reference_harness(reference, force=True)
    if exe is None:
        raise SystemExit("reference harness not found under " + reference)
    records = []
    for element, bk in (("f32", 32), ("bf16", 64)):
        out = subprocess.run([exe, "unused.cubin", "196768", "gemm_fast", element, str(bk), "288"],
                             capture_output=True, text=True, check=True).stdout
        lines = out.strip().splitlines()
        rec = json.loads([l for l in lines if l.startswith("{")][-1])
        rec["element"] = element
        rec["harness_stdout"] = [l for l in lines if not l.startswith("{")]
        records.append(rec)
    return records


def edge_floats() -> np.ndarray:
    bits = [0x00000000, 0x80000000, 0x3F800000, 0xBF800000, 0x3F808000, 0x3F818000, 0x3F807FFF,
            0x3F808001, 0x3F7FFFFF, 0x7F7FFFFF, 0x7F800000, 0xFF800000, 0x00000001, 0x007FFFFF,
            0x00800000, 0x33800000, 0x3DCCCCCD, 0x3C23D70A, 0x3D8F5C29, 0x477FE000, 0x477FF000,
            0x7F7F8000, 0x3F801000, 0x3F801FFF, 0x3F802000, 0xC2F6E979]
    rng = np.random.default_rng(1234)
    rnd = rng.integers(0, 2 ** 32, size=200, dtype=np.uint64).astype(np.uint32)
    # keep NaNs out of the random part (their payload handling is not pinned)
    rnd = rnd[((rnd >> 23) & 0xFF) != 0xFF]
    return np.concatenate([np.array(bits, dtype=np.uint32), rnd])


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()

    pin = run_pin(args.reference)
    for rec in pin:
        assert rec["launched"] == 1 and rec["operand_bytes_match"] == 1, rec
        assert rec["nonzero_diffs"] == 0 and rec["max_abs_diff"] == 0, rec
    with open(os.path.join(HERE, "reference_pin.json"), "w") as f:
        json.dump({"what": "reference host harness run against the oracle through a fake CUDA driver",
                   "cases": pin}, f, indent=1)

    # rounding helpers on edge values
    e = edge_floats()
    ef = e.view(np.float32)
    np.savez_compressed(os.path.join(HERE, "rounding_edges.npz"), bits=e,
                        bf16=np.array([oracle.to_bf16_scalar(float(x)) for x in ef], np.uint16),
                        tf32=np.array([oracle.round_tf32_scalar(float(x)) for x in ef],
                                      np.float32).view(np.uint32))

    # the harness's two pattern cases: M=N=256, K=16*BK
    for name, k, mode, narrow in (("pattern_f32_k512", 512, oracle.MODE_TF32, False),
                                  ("pattern_bf16_k1024", 1024, oracle.MODE_BF16, True)):
        a, b = oracle.pattern_inputs(256, 256, k)
        expect = oracle.gemm_rowmajor_b(a, b, mode)
        a_dev, bt_dev = oracle.prepare_operands(a, b, narrow)
        if narrow:
            again = oracle.gemm_kmajor_bf16(a_dev, bt_dev)
        else:
            again = oracle.gemm_kmajor(a_dev, bt_dev, mode)
        assert np.array_equal(expect.view(np.uint32), again.view(np.uint32))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), expect=expect)

    # 256^3, uniform[-1,1) seed 0, A row-major, B row-major
    a = synth.uniform_pm1(0, 256 * 256).reshape(256, 256)
    b = synth.uniform_pm1(0, 256 * 256, offset=256 * 256).reshape(256, 256)
    rows = np.arange(0, 256, 16, dtype=np.int32)
    bt = np.ascontiguousarray(b.T)
    np.savez_compressed(
        os.path.join(HERE, "uniform_seed0_256.npz"),
        a_head=a[:2, :8].copy(), b_head=b[:2, :8].copy(),
        expect_f32=oracle.gemm_rowmajor_b(a, b, oracle.MODE_NONE),
        rows=rows,
        expect_tf32_rows=oracle.gemm_kmajor(a, bt, oracle.MODE_TF32, rows=rows),
        expect_bf16_rows=oracle.gemm_kmajor(a, bt, oracle.MODE_BF16, rows=rows))

    # a ragged bf16 case with explicit operands
    rng = np.random.default_rng(7)
    m, n, k = 100, 72, 40
    a_bits = oracle.to_bf16(rng.standard_normal((m, k)).astype(np.float32))
    bt_bits = oracle.to_bf16(rng.standard_normal((n, k)).astype(np.float32))
    np.savez_compressed(os.path.join(HERE, "ragged_bf16_100x72x40.npz"), a_bits=a_bits,
                        bt_bits=bt_bits, expect=oracle.gemm_kmajor_bf16(a_bits, bt_bits))
    with open(os.path.join(HERE, "gpu_header_rejected.json"), "w") as f:
        json.dump(gpu_header_rejections(args.reference), f, indent=1)
        f.write("\n")
    for f in sorted(os.listdir(HERE)):
        print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
