"""The CPU oracle against the reference's own host check and the committed
known-answer vectors (no GPU)."""
import json
import os
import subprocess

import numpy as np
import pytest

import oracle
from oxcamlgpu_b200 import synth

REFERENCE_ROOT = os.environ.get("OXGPU_REFERENCE_ROOT", "/root/reference")


def test_reference_pin_record(golden_dir):
    """The committed outcome of running the reference harness against the oracle:
    identical operand bytes, zero differences over all 65536 outputs, both cases."""
    rec = json.load(open(os.path.join(golden_dir, "reference_pin.json")))
    cases = {c["element"]: c for c in rec["cases"]}
    assert set(cases) == {"f32", "bf16"}
    assert cases["f32"]["k"] == 512 and cases["bf16"]["k"] == 1024
    for c in cases.values():
        assert c["m"] == 256 and c["n"] == 256
        assert c["launched"] == 1 and c["operand_bytes_match"] == 1
        assert c["probes"] == 256 * 256 and c["nonzero_diffs"] == 0 and c["max_abs_diff"] == 0
        assert c["swizzle128_l2_128_nofill"] == 1
        assert c["grid"] == [1, 2, 1] and c["block"] == 288
    assert cases["f32"]["box_a"] == [32, 128] and cases["f32"]["box_b"] == [32, 256]
    assert cases["bf16"]["box_a"] == [64, 128] and cases["bf16"]["box_b"] == [64, 256]


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE_ROOT, "test/hardware/run_gemm_h100.cu")),
                    reason="no reference checkout on this machine")
def test_reference_pin_live():
    """Re-run the pin here: reference harness compiled in place + fake driver."""
    from oracle import build as obuild
    exe = obuild.build_reference_harness(REFERENCE_ROOT)
    for element, bk in (("f32", 32), ("bf16", 64)):
        out = subprocess.run([exe, "x.cubin", "196768", "gemm_fast", element, str(bk), "288"],
                             capture_output=True, text=True, check=True).stdout
        rec = json.loads([l for l in out.splitlines() if l.startswith("{")][-1])
        assert "passed" in out
        assert rec["operand_bytes_match"] == 1 and rec["nonzero_diffs"] == 0 and rec["probes"] == 65536


def test_rounding_edges(golden_dir):
    g = np.load(os.path.join(golden_dir, "rounding_edges.npz"))
    x = g["bits"].view(np.float32)
    assert np.array_equal(oracle.to_bf16(x), g["bf16"])
    assert np.array_equal(oracle.round_tf32(x).view(np.uint32), g["tf32"])
    # scalar C functions agree with the vectorised numpy forms
    for v, hb, tb in zip(x[:40], g["bf16"][:40], g["tf32"][:40]):
        assert oracle.to_bf16_scalar(float(v)) == int(hb)
        assert np.float32(oracle.round_tf32_scalar(float(v))).view(np.uint32) == tb


def test_bf16_rne_known_answers():
    f = lambda bits: float(np.array([bits], np.uint32).view(np.float32)[0])
    assert oracle.to_bf16_scalar(1.0) == 0x3F80
    assert oracle.to_bf16_scalar(f(0x3F808000)) == 0x3F80   # tie -> even (down)
    assert oracle.to_bf16_scalar(f(0x3F818000)) == 0x3F82   # tie -> even (up)
    assert oracle.to_bf16_scalar(f(0x3F808001)) == 0x3F81   # just above the tie
    assert oracle.to_bf16_scalar(f(0x3F807FFF)) == 0x3F80
    assert oracle.of_bf16_scalar(0x3F80) == 1.0 and oracle.of_bf16_scalar(0xC000) == -2.0
    assert oracle.round_tf32_scalar(f(0x3F801FFF)) == 1.0   # truncation, not rounding
    assert np.float32(oracle.round_tf32_scalar(f(0x3F802000))).view(np.uint32) == 0x3F802000


@pytest.mark.parametrize("name,k,mode,narrow", [("pattern_f32_k512", 512, oracle.MODE_TF32, False),
                                                ("pattern_bf16_k1024", 1024, oracle.MODE_BF16, True)])
def test_pattern_cases_match_golden(golden_dir, name, k, mode, narrow):
    """The harness's pattern case (run_gemm_h100.cu:113-118,129-130)."""
    expect = np.load(os.path.join(golden_dir, name + ".npz"))["expect"]
    a, b = oracle.pattern_inputs(256, 256, k)
    assert a[0, 0] == np.float32(0.01) and a[0, 6] == np.float32(7 * 0.01)
    got = oracle.gemm_rowmajor_b(a, b, mode)
    assert np.array_equal(got.view(np.uint32), expect.view(np.uint32))
    a_dev, bt_dev = oracle.prepare_operands(a, b, narrow)
    assert bt_dev.shape == (256, k)
    if narrow:
        assert np.array_equal(a_dev, oracle.to_bf16(a))
        km = oracle.gemm_kmajor_bf16(a_dev, bt_dev, threads=4)
    else:
        assert np.array_equal(bt_dev, b.T)
        km = oracle.gemm_kmajor(a_dev, bt_dev, mode, threads=4)
    assert np.array_equal(km.view(np.uint32), expect.view(np.uint32))
    first, worst = oracle.compare_abs(km, expect, oracle.REFERENCE_ABS_TOL["bf16" if narrow else "f32"])
    assert first == -1 and worst == 0.0


def test_uniform_256_matches_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "uniform_seed0_256.npz"))
    a = synth.uniform_pm1(0, 256 * 256).reshape(256, 256)
    b = synth.uniform_pm1(0, 256 * 256, offset=256 * 256).reshape(256, 256)
    assert np.array_equal(a[:2, :8], g["a_head"]) and np.array_equal(b[:2, :8], g["b_head"])
    assert a.min() >= -1.0 and a.max() < 1.0 and abs(float(a.mean())) < 0.02
    got = oracle.gemm_rowmajor_b(a, b, oracle.MODE_NONE)
    assert np.array_equal(got.view(np.uint32), g["expect_f32"].view(np.uint32))
    bt = np.ascontiguousarray(b.T)
    rows = g["rows"]
    assert np.array_equal(oracle.gemm_kmajor(a, bt, oracle.MODE_TF32, rows=rows, threads=2),
                          g["expect_tf32_rows"])
    assert np.array_equal(oracle.gemm_kmajor(a, bt, oracle.MODE_BF16, rows=rows), g["expect_bf16_rows"])
    # against float64: the f32 loop is within the strict bound of the true product
    exact = a.astype(np.float64) @ b.astype(np.float64)
    tol = oracle.tolerance(256, float(np.abs(a).max()), float(np.abs(b).max()))
    assert np.abs(got - exact).max() <= tol


def test_ragged_bf16_golden(golden_dir):
    g = np.load(os.path.join(golden_dir, "ragged_bf16_100x72x40.npz"))
    got = oracle.gemm_kmajor_bf16(g["a_bits"], g["bt_bits"])
    assert np.array_equal(got.view(np.uint32), g["expect"].view(np.uint32))
    wide = oracle.gemm_kmajor(oracle.of_bf16(g["a_bits"]), oracle.of_bf16(g["bt_bits"]), oracle.MODE_BF16)
    assert np.array_equal(wide, got)


def test_threads_and_row_subsets_do_not_change_bits():
    rng = np.random.default_rng(3)
    a = rng.standard_normal((37, 129)).astype(np.float32)
    bt = rng.standard_normal((53, 129)).astype(np.float32)
    full = oracle.gemm_kmajor(a, bt, oracle.MODE_TF32)
    assert np.array_equal(full, oracle.gemm_kmajor(a, bt, oracle.MODE_TF32, threads=oracle.max_threads()))
    rows = np.array([36, 0, 5, 5], np.int32)
    assert np.array_equal(oracle.gemm_kmajor(a, bt, oracle.MODE_TF32, rows=rows), full[rows])
    assert np.array_equal(full, oracle.gemm_rowmajor_b(a, np.ascontiguousarray(bt.T), oracle.MODE_TF32))


def test_edge_shapes():
    one = oracle.gemm_kmajor(np.array([[2.0]], np.float32), np.array([[3.0]], np.float32), 0)
    assert one.shape == (1, 1) and one[0, 0] == 6.0
    z = oracle.gemm_kmajor(np.zeros((3, 5), np.float32), np.ones((2, 5), np.float32), 0)
    assert np.array_equal(z, np.zeros((3, 2), np.float32))
    none = oracle.gemm_kmajor(np.ones((3, 5), np.float32), np.ones((2, 5), np.float32), 0,
                              rows=np.zeros(0, np.int32))
    assert none.shape == (0, 2)


def test_compare_abs_and_tolerance():
    e = np.zeros(10, np.float32)
    g = e.copy()
    g[7] = 0.3
    assert oracle.compare_abs(g, e, 0.2) == (7, pytest.approx(0.3))
    assert oracle.compare_abs(g, e, 0.5)[0] == -1
    g[2] = np.nan
    first, worst = oracle.compare_abs(g, e, 0.5)
    assert first == 2 and np.isnan(worst)
    assert oracle.tolerance(256, 1.0, 1.0) == pytest.approx(1.6e-4)


def test_synth_generators():
    u = synth.uniform_pm1(5, 1 << 16)
    assert u.dtype == np.float32 and u.min() >= -1 and u.max() < 1
    assert np.array_equal(u[100:200], synth.uniform_pm1(5, 100, offset=100))
    assert not np.array_equal(u[:100], synth.uniform_pm1(6, 100))
    z = synth.normal(2, 1 << 16)
    assert abs(float(z.mean())) < 0.02 and abs(float(z.std()) - 1.0) < 0.02
    z2 = synth.normal(3, 1 << 16, std=0.02)
    assert abs(float(z2.std()) - 0.02) < 1e-3
    big = synth.hash_u32(1, np.array([2 ** 32 + 5, 5], np.uint64))
    assert big[0] != big[1]
