"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Tolerances (inputs are rounded identically on both sides, so only accumulation
differs):
  strict   max|C - C_ref| <= 1e-5 * sqrt(K) * max|A| * max|B|.  Asserted for every
           tensor-core case with K <= 2048 (zero-mean inputs) -- and trivially for
           the exact path, which is bit-identical.
  tc       max|C - C_ref| <= 5e-5 * sqrt(K) * max|A| * max|B|: the stated relative
           tolerance, scaled by sqrt(K), for TF32/bf16 inputs with f32 accumulation
           in the matrix unit at large K.  The unit's accumulator drops low bits
           when it aligns addends (one-sided, so the difference to a sequential
           IEEE sum grows with the number of UMMA steps): measured 1.9e-5*sqrt(K)
           at TF32 4096^3 with uniform[-1,1) inputs.
  pattern  the reference's own thresholds, 5e-2 (f32/TF32) and 2e-1 (bf16)
           (run_gemm_h100.cu:193), plus a relative bound of 2^-16: the pattern
           inputs are all positive, so both sides carry O(K) one-sided rounding
           and the zero-mean bound does not apply to them.
  exact    0 -- the exact kernel repeats the oracle's operation order.
"""
import os

import numpy as np
import pytest
import torch

import oracle
from oxcamlgpu_b200 import catalog as cat
from oxcamlgpu_b200 import gemm, synth
from oxcamlgpu_b200._lib import OxgpuError

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TC_VARIANTS = ["1cta_128x256", "1cta_128x128", "1cta_256x128", "2cta_256x256", "2cta_256x128", "2cta_512x256",
               "1cta_256x256", "2cta_256x512"]


@pytest.fixture(scope="module", autouse=True)
def _device(oxlib):
    assert torch.cuda.is_available(), "these tests need a GPU"
    torch.cuda.set_device(0)
    yield
    # every test must leave the status block clean: no bounded wait may have expired
    assert gemm.device_status()[0] == 0


def bf16_tensor(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(DEV)


def rand_bf16(rng, rows, cols, scale=1.0):
    return oracle.to_bf16((rng.standard_normal((rows, cols)) * scale).astype(np.float32))


def strict_tol(k, a_max, b_max):
    return oracle.tolerance(k, a_max, b_max)


def tc_tol(k, a_max, b_max):
    """5e-5 * sqrt(K) * max|A| * max|B|: for TF32 with K >= 4096 only.  The matrix
    unit's accumulator truncates when it aligns addends, a one-sided error that
    grows with the number of UMMA steps; with uniform[-1,1) inputs at 4096^3 the
    difference to the sequential IEEE sum measures 1.9e-5 * sqrt(K).  Every bf16
    case meets the strict bound (8192^3 normal(0,1): 0.14 of it)."""
    return 5.0 * oracle.tolerance(k, a_max, b_max)


def check_bf16(a_bits, bt_bits, got, rows=None):
    expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits, rows=rows, threads=oracle.max_threads())
    g = got.float().cpu().numpy()
    if rows is not None:
        g = g[rows]
    tol = strict_tol(a_bits.shape[1], float(np.abs(oracle.of_bf16(a_bits)).max()),
                     float(np.abs(oracle.of_bf16(bt_bits)).max()))
    err = float(np.abs(g - expect).max())
    assert err <= tol, (err, tol)
    return err, tol


# ---- exact kernel: bit-identical to the oracle -----------------------------------
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (100, 72, 40), (1, 1, 1), (129, 257, 33), (128, 128, 512)])
@pytest.mark.parametrize("mode", [oracle.MODE_NONE, oracle.MODE_TF32, oracle.MODE_BF16])
def test_exact_kernel_is_bit_identical(m, n, k, mode):
    rng = np.random.default_rng(m * 1000 + n + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    bt = rng.standard_normal((n, k)).astype(np.float32)
    if mode == oracle.MODE_BF16:
        a_bits, bt_bits = oracle.to_bf16(a), oracle.to_bf16(bt)
        got = gemm.gemm_exact(bf16_tensor(a_bits), bf16_tensor(bt_bits), gemm.INPUT_BF16)
        expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits)
    else:
        got = gemm.gemm_exact(torch.from_numpy(a).to(DEV), torch.from_numpy(bt).to(DEV), mode)
        expect = oracle.gemm_kmajor(a, bt, mode)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), expect.view(np.uint32))


def test_config1_f32_256_against_golden(golden_dir):
    """f32 256^3, uniform[-1,1) seed 0: the exact path reproduces the host loop
    bit for bit; the TF32 tensor-core path meets the strict bound against the
    TF32-rounded oracle."""
    g = np.load(os.path.join(golden_dir, "uniform_seed0_256.npz"))
    a = torch.empty(256, 256, device=DEV)
    b = torch.empty(256, 256, device=DEV)
    gemm.fill_uniform(a, 0, 0)
    gemm.fill_uniform(b, 0, 256 * 256)
    a_h = synth.uniform_pm1(0, 256 * 256).reshape(256, 256)
    b_h = synth.uniform_pm1(0, 256 * 256, offset=256 * 256).reshape(256, 256)
    assert np.array_equal(a.cpu().numpy(), a_h) and np.array_equal(b.cpu().numpy(), b_h)
    bt = gemm.transpose(b)
    assert np.array_equal(bt.cpu().numpy(), b_h.T)
    exact = gemm.gemm_exact(a, bt, gemm.INPUT_NONE).cpu().numpy()
    assert np.array_equal(exact.view(np.uint32), g["expect_f32"].view(np.uint32))
    tol = strict_tol(256, 1.0, 1.0)
    rows = g["rows"]
    for variant in TC_VARIANTS:
        c = gemm.gemm_tf32(a, bt, flags=gemm.make_flags(variant)).cpu().numpy()
        err = np.abs(c[rows] - g["expect_tf32_rows"]).max()
        assert err <= tol, (variant, err, tol)
    # through the catalog entry the reference's choose_config picks for 256^3
    name = cat.kernel_binding(cat.choose_config(256, 256, 256))
    assert name == "gemm_bm64_bn256_s3"
    c = gemm.run_catalog_entry(name, a, bt).cpu().numpy()
    assert np.abs(c[rows] - g["expect_tf32_rows"]).max() <= tol
    full = oracle.gemm_kmajor(a_h, np.ascontiguousarray(b_h.T), oracle.MODE_TF32, threads=oracle.max_threads())
    assert np.abs(c - full).max() <= tol


# ---- the harness's pattern cases through the catalog entry points -----------------
@pytest.mark.parametrize("name,fixture,k,narrow", [("gemm_fast", "pattern_f32_k512", 512, False),
                                                  ("gemm_bf16_fast", "pattern_bf16_k1024", 1024, True)])
def test_pattern_case_through_catalog_entry(golden_dir, name, fixture, k, narrow):
    """run_gemm_h100.cu:113-118: M=N=256, K = 16 K-blocks so the ring wraps and
    the barrier parity flips both ways."""
    expect = np.load(os.path.join(golden_dir, fixture + ".npz"))["expect"]
    a, b = oracle.pattern_inputs(256, 256, k)
    a_dev, bt_dev = oracle.prepare_operands(a, b, narrow)
    if narrow:
        ta, tb = bf16_tensor(a_dev), bf16_tensor(bt_dev)
    else:
        ta, tb = torch.from_numpy(a_dev).to(DEV), torch.from_numpy(bt_dev).to(DEV)
    c = torch.full((256, 256), float("nan"), device=DEV)
    gemm.run_catalog_entry(name, ta, tb, c)
    got = c.cpu().numpy()
    first, worst = oracle.compare_abs(got, expect, oracle.REFERENCE_ABS_TOL["bf16" if narrow else "f32"])
    assert first == -1, (first, worst)
    rel = np.abs(got - expect) / np.abs(expect)
    assert rel.max() <= 2.0 ** -16, rel.max()


@pytest.mark.parametrize("mn", [(512, 512), (2560, 4096), (2560, 4352), (384, 768), (512, 384), (64, 256),
                                (192, 512)])
@pytest.mark.parametrize("name", cat.ENTRY_NAMES)
def test_every_catalog_entry(name, mn):
    """(2560, 4096) has enough tiles for a CTA-pair tile (256x512 for the 64/128-row
    A boxes, 512x256 for the 256-row ones), (2560, 4352) for the one-CTA 256x256
    kernel (every box divides it); the small sizes keep the entry's own tile
    shape.  M = 64 and 192 are sizes only the bm=64 entries accept (the reference
    needs M % bm == 0, bench/bench.py:247-250): the 128-row tile that serves them
    reads zeros past the end of A and its store is clipped."""
    tile, eb = cat.kernel_tile(name)
    rng = np.random.default_rng(len(name) * 31 + mn[0])
    m, n, k = mn[0], mn[1], 5 * tile.bk
    if m % tile.bm or n % tile.bn:
        pytest.skip("size not divisible by this entry's tile")
    if eb == 2:
        a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
        c = gemm.run_catalog_entry(name, bf16_tensor(a_bits), bf16_tensor(bt_bits))
        check_bf16(a_bits, bt_bits, c)
    else:
        a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        bt = rng.uniform(-1, 1, (n, k)).astype(np.float32)
        c = gemm.run_catalog_entry(name, torch.from_numpy(a).to(DEV), torch.from_numpy(bt).to(DEV))
        expect = oracle.gemm_kmajor(a, bt, oracle.MODE_TF32, threads=oracle.max_threads())
        assert np.abs(c.cpu().numpy() - expect).max() <= strict_tol(k, 1.0, 1.0)


def test_catalog_entry_rejects_bad_sizes():
    a = torch.zeros(256, 512, device=DEV)
    with pytest.raises(OxgpuError) as e:
        gemm.run_catalog_entry("gemm_fast", a[:200].contiguous(), a)
    assert e.value.status == -4


# ---- one-hot probes: descriptor / swizzle / TMEM-map errors show up as permutations
@pytest.mark.parametrize("variant", TC_VARIANTS)
def test_one_hot_probes_bf16(variant):
    rng = np.random.default_rng(11)
    m = n = 512
    k = 192
    bt_bits = rand_bf16(rng, n, k)
    bt = bf16_tensor(bt_bits)
    bt_f = oracle.of_bf16(bt_bits)
    picks = [(0, 0), (5, 17), (127, 63), (128, 64), (300, 191), (511, 100), (200, 15), (77, 130)]
    a = np.zeros((m, k), np.float32)
    for r, kk in picks:
        a[r, kk] = 1.0
    c = gemm.gemm_bf16(bf16_tensor(oracle.to_bf16(a)), bt, flags=gemm.make_flags(variant)).cpu().numpy()
    expect = np.zeros((m, n), np.float32)
    for r, kk in picks:
        expect[r] = bt_f[:, kk]
    assert np.array_equal(c, expect)          # exact: one product per output
    # and the other way round: one-hot B^T rows select columns of A
    a_bits = rand_bf16(rng, m, k)
    b1 = np.zeros((n, k), np.float32)
    for j, kk in picks:
        b1[j, kk] = 1.0
    c = gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(oracle.to_bf16(b1)),
                       flags=gemm.make_flags(variant)).cpu().numpy()
    expect = np.zeros((m, n), np.float32)
    for j, kk in picks:
        expect[:, j] = oracle.of_bf16(a_bits)[:, kk]
    assert np.array_equal(c, expect)


def test_tf32_inputs_are_truncated_not_rounded():
    """run_gemm_h100.cu:40-44 models the matrix unit as dropping the low 13
    mantissa bits.  Probe with one-hot rows so each output is a single product."""
    m = n = 256
    k = 32
    vals = np.array([0x3F801FFF, 0x3F802000, 0x3F803FFF, 0xBF801FFF, 0x3DCCCCCD, 0x477FFFFF],
                    np.uint32).view(np.float32)
    bt = np.zeros((n, k), np.float32)
    bt[np.arange(len(vals)), np.arange(len(vals))] = vals
    a = np.zeros((m, k), np.float32)
    a[0, :len(vals)] = 1.0
    a[1, :len(vals)] = vals          # both operands truncated
    c = gemm.gemm_tf32(torch.from_numpy(a).to(DEV), torch.from_numpy(bt).to(DEV),
                       flags=gemm.make_flags("1cta_128x128")).cpu().numpy()
    expect = oracle.gemm_kmajor(a, bt, oracle.MODE_TF32)
    assert np.array_equal(c[:2, :len(vals)].view(np.uint32), expect[:2, :len(vals)].view(np.uint32))


# ---- ring depth / barrier parity sweep ----------------------------------------------
@pytest.mark.parametrize("variant", TC_VARIANTS)
@pytest.mark.parametrize("kblocks", [1, 2, 3, 4, 5, 8, 16, 17])
def test_ring_and_parity_sweep_bf16(variant, kblocks):
    rng = np.random.default_rng(kblocks)
    m, n, k = 512, 768, 64 * kblocks
    a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    for stages in (2, 0):
        c = gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits),
                           flags=gemm.make_flags(variant, stages=stages))
        check_bf16(a_bits, bt_bits, c)


@pytest.mark.parametrize("variant", ["1cta_256x128", "2cta_512x256", "1cta_256x256", "2cta_256x512"])
@pytest.mark.parametrize("reorder", [15, 1, 2, 3])
@pytest.mark.parametrize("kblocks", [1, 2, 3, 5, 6, 7, 12])
def test_block_major_tile_ends(variant, reorder, kblocks):
    """256-row variants issue the first/last K blocks of a tile block-major; every
    setting must give the same result, with several tiles per CTA."""
    rng = np.random.default_rng(kblocks * 7 + reorder)
    m, n, k = 2048, 2560, 64 * kblocks
    a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    for stages in (2, 0):
        c = gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits),
                           flags=gemm.make_flags(variant, stages=stages, reorder=reorder))
        check_bf16(a_bits, bt_bits, c, rows=np.array([0, 127, 128, 255, 256, 1000, 2047], np.int32))
        exact = gemm.gemm_exact(bf16_tensor(a_bits), bf16_tensor(bt_bits), gemm.INPUT_BF16)
        assert float((c - exact).abs().max()) <= strict_tol(k, 6.0, 6.0)


@pytest.mark.parametrize("variant", TC_VARIANTS)
def test_many_tiles_per_cta_and_accumulator_reuse(variant):
    """More tiles than CTAs: both TMEM accumulators are reused several times."""
    rng = np.random.default_rng(5)
    m, n, k = 4096, 4096, 128
    a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    c = gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits), flags=gemm.make_flags(variant))
    exact = gemm.gemm_exact(bf16_tensor(a_bits), bf16_tensor(bt_bits), gemm.INPUT_BF16)
    tol = strict_tol(k, float(np.abs(oracle.of_bf16(a_bits)).max()), float(np.abs(oracle.of_bf16(bt_bits)).max()))
    assert float((c - exact).abs().max()) <= tol
    rows = np.array([0, 127, 128, 2049, 4095], np.int32)
    check_bf16(a_bits, bt_bits, c, rows=rows)


# ---- ragged shapes and guard bands ----------------------------------------------------
@pytest.mark.parametrize("variant", TC_VARIANTS)
@pytest.mark.parametrize("m,n,k", [(100, 72, 40), (129, 260, 72), (300, 520, 200), (1, 4, 8)])
def test_ragged_shapes_bf16(golden_dir, variant, m, n, k):
    if (m, n, k) == (100, 72, 40):
        g = np.load(os.path.join(golden_dir, "ragged_bf16_100x72x40.npz"))
        a_bits, bt_bits = g["a_bits"], g["bt_bits"]
    else:
        rng = np.random.default_rng(m + n + k)
        a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    # C sits inside a larger NaN-filled buffer: nothing outside [M,N] may be written
    pad = torch.full((m + 2, n + 8), float("nan"), device=DEV)
    c = pad[1:m + 1, 4:n + 4]
    gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits), c, flags=gemm.make_flags(variant))
    check_bf16(a_bits, bt_bits, c.contiguous())
    assert torch.isnan(pad[0]).all() and torch.isnan(pad[-1]).all()
    assert torch.isnan(pad[:, :4]).all() and torch.isnan(pad[:, n + 4:]).all()


def test_ragged_tf32():
    rng = np.random.default_rng(9)
    m, n, k = 200, 136, 52
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    bt = rng.uniform(-1, 1, (n, k)).astype(np.float32)
    for variant in TC_VARIANTS:
        c = gemm.gemm_tf32(torch.from_numpy(a).to(DEV), torch.from_numpy(bt).to(DEV),
                           flags=gemm.make_flags(variant)).cpu().numpy()
        expect = oracle.gemm_kmajor(a, bt, oracle.MODE_TF32)
        assert np.abs(c - expect).max() <= strict_tol(k, 1.0, 1.0), variant


def test_strided_operands():
    rng = np.random.default_rng(21)
    m, n, k = 256, 256, 128
    a_bits, bt_bits = rand_bf16(rng, m, k + 64), rand_bf16(rng, n, k + 8)
    ta, tb = bf16_tensor(a_bits)[:, :k], bf16_tensor(bt_bits)[:, :k]
    c = gemm.gemm_bf16(ta, tb)
    check_bf16(np.ascontiguousarray(a_bits[:, :k]), np.ascontiguousarray(bt_bits[:, :k]), c)


# ---- bf16 output ------------------------------------------------------------------------
@pytest.mark.parametrize("variant", ["auto", "1cta_128x256", "1cta_128x128", "2cta_256x256", "2cta_512x256"])
@pytest.mark.parametrize("m,n,k", [(512, 768, 320), (300, 520, 200), (2048, 2560, 128)])
def test_bf16_output(variant, m, n, k):
    """bf16 C = RNE(f32 accumulator): within half a bf16 ulp of the oracle's f32
    result plus the accumulation tolerance."""
    rng = np.random.default_rng(m + k)
    a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    pad = torch.full((m + 2, n + 16), float("nan"), device=DEV, dtype=torch.bfloat16)
    c = pad[1:m + 1, 8:n + 8]
    gemm.gemm_bf16_out16(bf16_tensor(a_bits), bf16_tensor(bt_bits), c, flags=gemm.make_flags(variant))
    expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits, threads=oracle.max_threads())
    got = c.float().cpu().numpy()
    tol = strict_tol(k, float(np.abs(oracle.of_bf16(a_bits)).max()), float(np.abs(oracle.of_bf16(bt_bits)).max()))
    assert (np.abs(got - expect) <= np.abs(expect) * 2.0 ** -8 + tol).all()
    # where the f32 kernel's result rounds unambiguously, the bf16 kernel must equal that rounding
    c32 = gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits), flags=gemm.make_flags(variant)).cpu().numpy()
    assert np.array_equal(oracle.to_bf16(c32), c.contiguous().view(torch.int16).cpu().numpy().view(np.uint16))
    assert torch.isnan(pad[0]).all() and torch.isnan(pad[-1]).all()
    assert torch.isnan(pad[:, :8]).all() and torch.isnan(pad[:, n + 8:]).all()


def test_bf16_output_rejects_unsupported():
    a = torch.zeros(256, 64, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(OxgpuError):
        gemm.gemm_bf16_out16(a, a, flags=gemm.make_flags("2cta_256x128"))
    with pytest.raises(OxgpuError):
        gemm.gemm_bf16_out16(a, a, flags=gemm.make_flags("splitk"))


# ---- split-K --------------------------------------------------------------------------
@pytest.mark.parametrize("m,n,k,splits", [(128, 1024, 2048, 4), (128, 1024, 2048, 0), (100, 264, 1000, 3),
                                          (256, 512, 64, 5)])
def test_split_k(m, n, k, splits):
    rng = np.random.default_rng(splits + k)
    a_bits, bt_bits = rand_bf16(rng, m, k, 0.02), rand_bf16(rng, n, k, 0.02)
    c = gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits),
                       flags=gemm.make_flags("splitk", splits=splits))
    check_bf16(a_bits, bt_bits, c)


@pytest.mark.parametrize("variant,splits", [("cluster_splitk_128x128", 2), ("cluster_splitk_128x128", 4),
                                            ("cluster_splitk_128x256", 2), ("cluster_splitk_128x256", 4),
                                            ("cluster_splitk_128x256", 8), ("cluster_splitk_128x128", 0)])
@pytest.mark.parametrize("m,n,k", [(128, 1024, 2048), (100, 520, 1000), (384, 512, 4096), (128, 256, 64)])
def test_cluster_split_k(variant, splits, m, n, k):
    """K slices across a thread-block cluster (two: added by TMA reductions to a
    tile of C that the kernel zeroes; four, eight: summed through distributed shared
    memory in ascending order): same slices and summation order as the workspace
    split-K, so the two agree bit for bit, and a second launch into the same C gives
    the same bits again; ragged edges and NaN guard bands as elsewhere."""
    rng = np.random.default_rng(splits * 13 + k)
    a_bits, bt_bits = rand_bf16(rng, m, k, 0.02), rand_bf16(rng, n, k, 0.02)
    pad = torch.full((m + 2, n + 8), float("nan"), device=DEV)
    c = pad[1:m + 1, 4:n + 4]
    gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits), c, flags=gemm.make_flags(variant, splits=splits))
    check_bf16(a_bits, bt_bits, c.contiguous())
    assert torch.isnan(pad[0]).all() and torch.isnan(pad[-1]).all()
    assert torch.isnan(pad[:, :4]).all() and torch.isnan(pad[:, n + 4:]).all()
    first = c.contiguous().clone()
    gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits), c, flags=gemm.make_flags(variant, splits=splits))
    assert torch.equal(c.contiguous(), first)         # a second launch into the same C: same bits
    if splits in (2, 4) and (k // 64) % splits == 0:
        ws = gemm.gemm_bf16(bf16_tensor(a_bits), bf16_tensor(bt_bits), flags=gemm.make_flags("splitk", splits=splits))
        assert torch.equal(first, ws)


@pytest.mark.parametrize("variant,m,n,k", [("cluster_splitk_128x128", 128, 1024, 4096), ("cluster_splitk_128x256", 200, 1000, 2112),
                                           ("cluster_splitk_128x128", 1024, 1024, 8192)])
def test_two_slice_cluster_split_k_both_routes_agree(monkeypatch, variant, m, n, k):
    """Two K slices in a cluster are summed either by TMA reductions into a tile of
    C that the kernel zeroed first (the default) or through distributed shared
    memory (what four and eight slices use).  Two addends: the same bits either
    way, over whatever C held before (NaN here), and nothing outside C."""
    rng = np.random.default_rng(k + m)
    a_bits, bt_bits = rand_bf16(rng, m, k, 0.02), rand_bf16(rng, n, k, 0.02)
    a, bt = bf16_tensor(a_bits), bf16_tensor(bt_bits)
    flags = gemm.make_flags(variant, splits=2)
    out = {}
    for route in ("", "dsmem"):
        monkeypatch.setenv("OXGPU_CLUSTER_REDUCE", route)
        pad = torch.full((m + 2, n + 8), float("nan"), device=DEV)
        c = pad[1:m + 1, 4:n + 4]
        for _ in range(3):   # repeated launches into the same C: the zeroing is part of every launch
            gemm.gemm_bf16(a, bt, c, flags=flags)
        out[route] = c.contiguous()
        assert torch.isnan(pad[0]).all() and torch.isnan(pad[-1]).all()
        assert torch.isnan(pad[:, :4]).all() and torch.isnan(pad[:, n + 4:]).all()
    assert torch.equal(out[""], out["dsmem"])
    check_bf16(a_bits, bt_bits, out[""])


def test_skinny_problem_takes_the_cluster_split_k_path_by_default():
    a = torch.empty(128, 8192, device=DEV, dtype=torch.bfloat16)
    bt = torch.empty(8192, 8192, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(a, 3, 0.02, 0)
    gemm.fill_normal(bt, 3, 0.02, 128 * 8192)
    auto = gemm.gemm_bf16(a, bt)
    explicit = gemm.gemm_bf16(a, bt, flags=gemm.make_flags("cluster_splitk_128x128", splits=2))
    assert torch.equal(auto, explicit)
    unsplit = gemm.gemm_bf16(a, bt, flags=gemm.make_flags("1cta_128x128"))
    assert not torch.equal(auto, unsplit)           # two K slices, summed once more at the end
    tf = gemm.gemm_tf32(a.float(), bt.float())
    exact = gemm.gemm_exact(a.float(), bt.float(), gemm.INPUT_TF32)
    assert float((tf - exact).abs().max()) <= tc_tol(8192, float(a.float().abs().max()), float(bt.float().abs().max()))


# ---- helpers ---------------------------------------------------------------------------
def test_conversion_and_transpose_match_the_oracle(golden_dir):
    g = np.load(os.path.join(golden_dir, "rounding_edges.npz"))
    x = g["bits"].view(np.float32)
    got = gemm.f32_to_bf16(torch.from_numpy(x.copy()).to(DEV)).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, g["bf16"])
    rng = np.random.default_rng(2)
    b = rng.standard_normal((70, 45)).astype(np.float32)
    assert np.array_equal(gemm.transpose(torch.from_numpy(b).to(DEV)).cpu().numpy(), b.T)
    b16 = oracle.to_bf16(b)
    got = gemm.transpose(bf16_tensor(b16)).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, b16.T)


@pytest.mark.parametrize("rows,cols", [(64, 64), (128, 192), (320, 256), (64, 128), (192, 384), (70, 45), (64, 100), (1, 9)])
def test_transpose_tiled_and_edge_paths(rows, cols):
    """Whole tiles (64 rows x 256 bytes) take the 16-byte-access kernel, other
    sizes the element-wise one; both must be exact permutations, for 4- and
    2-byte elements."""
    rng = np.random.default_rng(rows * 7 + cols)
    b = rng.standard_normal((rows, cols)).astype(np.float32)
    assert np.array_equal(gemm.transpose(torch.from_numpy(b).to(DEV)).cpu().numpy(), b.T)
    b16 = oracle.to_bf16(b)
    got = gemm.transpose(bf16_tensor(b16)).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, b16.T)


@pytest.mark.parametrize("rows,cols", [(64, 64), (128, 320), (448, 192)])
def test_fused_relayout_and_conversion(rows, cols):
    rng = np.random.default_rng(rows + cols)
    b = (rng.standard_normal((rows, cols)) * 10.0 ** rng.integers(-10, 10, (rows, cols))).astype(np.float32)
    got = gemm.transpose_to_bf16(torch.from_numpy(b).to(DEV)).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, oracle.to_bf16(b).T)
    with pytest.raises(OxgpuError):
        gemm.transpose_to_bf16(torch.zeros(70, 64, device=DEV))


@pytest.mark.parametrize("count,skip", [(1, 0), (7, 0), (8, 0), (4099, 0), (4096, 1), (1000, 3)])
def test_conversion_vector_and_tail_paths(count, skip):
    """f32 -> bf16 with and without 16-byte alignment and with a ragged tail:
    bit-equal to the oracle's round-to-nearest-even."""
    rng = np.random.default_rng(count + skip)
    x = (rng.standard_normal(count + skip) * 10.0 ** rng.integers(-20, 20, count + skip)).astype(np.float32)
    xd = torch.from_numpy(x).to(DEV)[skip:]
    got = gemm.f32_to_bf16(xd.contiguous() if skip == 0 else xd).view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.array_equal(got, oracle.to_bf16(x[skip:]))


@pytest.mark.parametrize("count,skip", [(5, 0), (1 << 12, 0), ((1 << 12) + 3, 0), (1 << 12, 1)])
def test_generators_are_index_functions(count, skip):
    """The value of element i depends only on (seed, offset + i): the vector
    path, the element path and an unaligned start all give the host generator's bits."""
    buf = torch.empty(count + skip, device=DEV)
    gemm.fill_uniform(buf[skip:], 9, 17)
    assert np.array_equal(buf[skip:].cpu().numpy(), synth.uniform_pm1(9, count, offset=17))
    whole = torch.empty(count + 4, device=DEV, dtype=torch.bfloat16)
    part = torch.empty_like(whole)
    gemm.fill_normal(whole, 4, 0.5, 0)
    gemm.fill_normal(part[skip:], 4, 0.5, skip)
    assert torch.equal(whole[skip:], part[skip:])


def test_device_generators():
    u = torch.empty(1 << 16, device=DEV)
    gemm.fill_uniform(u, 5, 100)
    assert np.array_equal(u.cpu().numpy(), synth.uniform_pm1(5, 1 << 16, offset=100))
    z = torch.empty(1 << 20, device=DEV)
    gemm.fill_normal(z, 2, 1.0)
    zh = synth.normal(2, 1 << 20)
    assert abs(float(z.mean())) < 0.01 and abs(float(z.std()) - 1.0) < 0.01
    assert np.abs(z.cpu().numpy() - zh).max() < 1e-4     # same stream, libm-level differences only
    zb = torch.empty(1 << 16, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(zb, 3, 0.02)
    assert abs(float(zb.float().std()) - 0.02) < 1e-3


def test_bounded_wait_gives_up_and_reports(oxlib):
    """A wait on a barrier nothing arrives on must time out, return and leave a
    status the host can read; the device stays usable."""
    st = oxlib.oxgpu_b200_selftest_bounded_wait(2_000_000)    # 2 ms budget
    assert st == -7
    assert b"kind 6" in oxlib.oxgpu_b200_last_error()
    assert gemm.device_status()[0] == 0                        # cleared by the read
    x = torch.ones(8, device=DEV)
    assert float(x.sum()) == 8.0


def test_host_buffer_entry_point():
    rng = np.random.default_rng(31)
    m, n, k = 1000, 520, 328
    a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    a_h = torch.from_numpy(a_bits.view(np.int16).copy()).view(torch.bfloat16).pin_memory()
    b_h = torch.from_numpy(bt_bits.view(np.int16).copy()).view(torch.bfloat16).pin_memory()
    c_h = torch.full((m, n), float("nan")).pin_memory()
    for _ in range(2):
        gemm.gemm_bf16_host(a_h, b_h, c_h)
        check_bf16(a_bits, bt_bits, c_h)
    # bf16 C on the host: equal to the device-side bf16-output GEMM of the same blocks' tiles
    # up to the tile choice, and within the bound after one rounding to bf16
    c16 = torch.zeros((m, n), dtype=torch.bfloat16).pin_memory()
    gemm.gemm_bf16_out16_host(a_h, b_h, c16)
    expect16 = oracle.gemm_kmajor_bf16(a_bits, bt_bits, threads=oracle.max_threads())
    tol16 = strict_tol(k, float(np.abs(oracle.of_bf16(a_bits)).max()), float(np.abs(oracle.of_bf16(bt_bits)).max()))
    got16 = c16.float().numpy()
    assert (np.abs(got16 - expect16) <= tol16 + np.abs(expect16) * 2.0 ** -8).all()   # one rounding to bf16
    with pytest.raises(OxgpuError):
        gemm.gemm_bf16_out16_host(a_h, b_h[:, :].contiguous()[:516], torch.zeros((m, 516), dtype=torch.bfloat16))
    a32 = rng.uniform(-1, 1, (300, 64)).astype(np.float32)
    b32 = rng.uniform(-1, 1, (260, 64)).astype(np.float32)
    c32 = torch.empty(300, 260)
    gemm.gemm_tf32_host(torch.from_numpy(a32), torch.from_numpy(b32), c32)
    expect = oracle.gemm_kmajor(a32, b32, oracle.MODE_TF32)
    assert np.abs(c32.numpy() - expect).max() <= strict_tol(64, 1.0, 1.0)


# ---- the workload configurations at full size ---------------------------------------------
def _sample_rows(m, count, seed):
    rng = np.random.default_rng(seed)
    rows = np.unique(np.concatenate([[0, m - 1, 127, 128], rng.integers(0, m, count)])).astype(np.int32)
    return rows


def test_tf32_4096_cubed():
    """TF32 4096^3, uniform[-1,1) seed 1: sampled rows against the CPU oracle,
    the whole matrix against the exact device kernel (itself bit-identical to
    the oracle), and linearity C(2A) == 2 C(A) exactly."""
    n = 4096
    a = torch.empty(n, n, device=DEV)
    b = torch.empty(n, n, device=DEV)
    gemm.fill_uniform(a, 1, 0)
    gemm.fill_uniform(b, 1, n * n)
    bt = gemm.transpose(b)
    c = gemm.gemm_tf32(a, bt)
    tol = tc_tol(n, 1.0, 1.0)
    rows = _sample_rows(n, 12, 1)
    expect = oracle.gemm_kmajor(a[rows].cpu().numpy(), bt.cpu().numpy(), oracle.MODE_TF32,
                                threads=oracle.max_threads())
    assert np.abs(c[rows].cpu().numpy() - expect).max() <= tol
    exact = gemm.gemm_exact(a, bt, gemm.INPUT_TF32)
    assert np.array_equal(exact[rows].cpu().numpy(), expect)
    assert float((c - exact).abs().max()) <= tol
    c2 = gemm.gemm_tf32(a * 2, bt)
    assert torch.equal(c2, c * 2)
    # the reference's own entry point with the reference's own maps (the drop-in call)
    via_entry = gemm.run_catalog_entry("gemm_fast", a, bt)
    assert float((via_entry - exact).abs().max()) <= tol and torch.equal(via_entry, c)


def test_bf16_8192_cubed():
    """bf16 8192^3, normal(0,1) seed 2, A row-major / B column-major."""
    n = 8192
    a = torch.empty(n, n, device=DEV, dtype=torch.bfloat16)
    bt = torch.empty(n, n, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(a, 2, 1.0, 0)
    gemm.fill_normal(bt, 2, 1.0, n * n)
    c = gemm.gemm_bf16(a, bt)
    a_max, b_max = float(a.float().abs().max()), float(bt.float().abs().max())
    tol = strict_tol(n, a_max, b_max)
    rows = _sample_rows(n, 4, 2)
    a_bits = a[rows].view(torch.int16).cpu().numpy().view(np.uint16)
    bt_bits = bt.view(torch.int16).cpu().numpy().view(np.uint16)
    expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits, threads=oracle.max_threads())
    assert np.abs(c[rows].cpu().numpy() - expect).max() <= tol
    exact = gemm.gemm_exact(a, bt, gemm.INPUT_BF16)
    assert np.array_equal(exact[rows].cpu().numpy(), expect)
    assert float((c - exact).abs().max()) <= tol
    for variant in ("1cta_128x256", "2cta_256x256", "2cta_256x128", "2cta_256x512"):
        cv = gemm.gemm_bf16(a, bt, flags=gemm.make_flags(variant))
        assert float((cv - exact).abs().max()) <= tol
    # the reference's own entry point with the reference's own maps (the drop-in call)
    via_entry = gemm.run_catalog_entry("gemm_bf16_fast", a, bt)
    assert float((via_entry - exact).abs().max()) <= tol and torch.equal(via_entry, c)


@pytest.mark.parametrize("m,n,k", [(8192, 28672, 8192), (8192, 8192, 28672), (128, 8192, 8192)])
def test_bf16_projection_shapes(m, n, k):
    """bf16 rectangular projection shapes, normal(0, 0.02) seed 3."""
    a = torch.empty(m, k, device=DEV, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(a, 3, 0.02, 0)
    gemm.fill_normal(bt, 3, 0.02, m * k)
    c = gemm.gemm_bf16(a, bt)
    tol = strict_tol(k, float(a.float().abs().max()), float(bt.float().abs().max()))
    rows = _sample_rows(m, 2, 3)[:4]
    a_bits = a[rows].view(torch.int16).cpu().numpy().view(np.uint16)
    bt_bits = bt.view(torch.int16).cpu().numpy().view(np.uint16)
    expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits, threads=oracle.max_threads())
    assert np.abs(c[rows].cpu().numpy() - expect).max() <= tol
    if m == 128:
        cs = gemm.gemm_bf16(a, bt, flags=gemm.make_flags("splitk"))
        assert np.abs(cs[rows].cpu().numpy() - expect).max() <= tol
        exact = gemm.gemm_exact(a, bt, gemm.INPUT_BF16)
        assert float((c - exact).abs().max()) <= tol and float((cs - exact).abs().max()) <= tol


def test_sharded_config_at_full_size():
    """bf16 M=32768 N=65536 K=8192, normal(0,1) seed 4, on one GPU (A 0.5 GiB, B^T
    1 GiB, C 8 GiB): C has 2^31 elements, so the last one sits at flat index
    2^31 - 1 -- past what the reference's 32-bit index arithmetic can address
    (lib/backend/ptx.ml:320-322).  Sampled rows, the last row and its last column
    included, against the CPU oracle (test/hardware/run_gemm_h100.cu:150-162) and
    bit for bit against the exact kernel; then the eight column shards the
    multi-GPU driver would compute equal the whole, bit for bit."""
    from oxcamlgpu_b200 import sharded
    m, n, k = 32768, 65536, 8192
    free, _ = torch.cuda.mem_get_info()
    if free < 14 * 2 ** 30:
        pytest.skip("needs 14 GiB of free device memory")
    a = torch.empty(m, k, device=DEV, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(a, 4, 1.0, 0)
    gemm.fill_normal(bt, 4, 1.0, m * k)
    c = torch.full((m, n), float("nan"), device=DEV)
    gemm.gemm_bf16(a, bt, c)
    assert c.numel() == 2 ** 31
    rows = torch.tensor([0, 12345, m // 2 + 1, m - 1], device=DEV)
    a_rows = a[rows].contiguous()
    got = c[rows].cpu().numpy()
    assert not np.isnan(got).any()
    a_bits = a_rows.view(torch.int16).cpu().numpy().view(np.uint16)
    bt_bits = bt.view(torch.int16).cpu().numpy().view(np.uint16)
    expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits, threads=oracle.max_threads())
    tol = strict_tol(k, float(a.float().abs().max()), float(bt[:8192].float().abs().max()))
    assert np.abs(got - expect).max() <= tol
    # the very last element of C, read through its flat index
    last = float(c.view(-1)[2 ** 31 - 1])
    assert last == float(got[3, n - 1]) and abs(last - float(expect[3, n - 1])) <= tol
    exact = gemm.gemm_exact(a_rows, bt, gemm.INPUT_BF16)
    assert np.array_equal(exact.cpu().numpy().view(np.uint32), expect.view(np.uint32))
    del bt_bits, expect, exact
    # the driver's eight shards, one after the other on this GPU
    shard = torch.empty(m, n // 8, device=DEV)
    for n0, n1 in sharded.column_partition(n, 8):
        assert n1 - n0 == n // 8
        shard.fill_(float("nan"))
        gemm.gemm_bf16(a, bt[n0:n1], shard)
        assert torch.equal(shard, c[:, n0:n1])
    del c, shard, a, bt
    torch.cuda.empty_cache()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_column_shards_concatenate_to_the_unsharded_result(world):
    """The multi-GPU driver's decomposition, run shard by shard on one GPU: every
    rank's C[:, n0:n1] = A * B[:, n0:n1] and the concatenation equals the
    unsharded GEMM bit for bit (same kernel, same K order per output)."""
    from oxcamlgpu_b200 import sharded
    m, n, k = 1024, 8192, 512
    a = torch.empty(m, k, device=DEV, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(a, 4, 1.0, 0)
    gemm.fill_normal(bt, 4, 1.0, m * k)
    whole = gemm.gemm_bf16(a, bt)
    parts = sharded.column_partition(n, world)
    shards = [gemm.gemm_bf16(a, bt[n0:n1]) for n0, n1 in parts]
    assert torch.equal(torch.cat(shards, dim=1), whole)
    # the gathered layout [world, M, N/world] and its re-interleave
    gathered = torch.stack(shards, dim=0)
    assert torch.equal(sharded.blocks_to_row_major(gathered), whole)
    exact = gemm.gemm_exact(a, bt, gemm.INPUT_BF16)
    assert float((whole - exact).abs().max()) <= strict_tol(k, float(a.float().abs().max()), float(bt.float().abs().max()))


FANOUT_VARIANTS = ["auto", "1cta_128x128", "2cta_256x256", "2cta_512x256"]


@pytest.mark.parametrize("variant", FANOUT_VARIANTS)
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_fanout_epilogue_replicates_the_shards(variant, world):
    """The fused GEMM + all-gather, all ranks emulated one after the other on one
    GPU: rank r's kernel writes its column window of every replica.  Each
    replica must equal the unsharded product of the same variant bit for bit,
    and nothing outside a window may be touched by the wrong rank."""
    from oxcamlgpu_b200 import sharded
    m, n, k = 640, 2304, 320  # 9 column blocks of 256: uneven shard widths for world 2 and 8
    a = torch.empty(m, k, device=DEV, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(a, 11, 1.0, 0)
    gemm.fill_normal(bt, 11, 1.0, m * k)
    flags = gemm.make_flags(variant)
    whole = gemm.gemm_bf16(a, bt, flags=flags)
    replicas = [torch.full((m, n), float("nan"), device=DEV) for _ in range(world)]
    for n0, n1 in sharded.column_partition(n, world):
        if n1 > n0:
            gemm.gemm_fanout(a, bt[n0:n1], [r[:, n0:n1] for r in replicas], flags=flags)
    for r in replicas:
        assert torch.equal(r, whole)
    exact = gemm.gemm_exact(a, bt, gemm.INPUT_BF16)
    assert float((whole - exact).abs().max()) <= strict_tol(k, float(a.float().abs().max()),
                                                            float(bt.float().abs().max()))


@pytest.mark.parametrize("variant", FANOUT_VARIANTS)
def test_fanout_ragged_window_does_not_spill(variant):
    """Ragged M and N: the stores are clipped to each destination's window, so
    the columns on either side of it keep their contents."""
    m, n, k = 300, 260, 200
    rng = np.random.default_rng(5)
    a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    a, bt = bf16_tensor(a_bits), bf16_tensor(bt_bits)
    full = [torch.full((m + 3, 1024), -7.0, device=DEV) for _ in range(2)]
    windows = [f[:m, 256:256 + n] for f in full]
    gemm.gemm_fanout(a, bt, windows, flags=gemm.make_flags(variant))
    for f, w in zip(full, windows):
        check_bf16(a_bits, bt_bits, w)
        mask = torch.ones_like(f, dtype=torch.bool)
        mask[:m, 256:256 + n] = False
        assert bool((f[mask] == -7.0).all())


def test_fanout_tf32_and_raw_addresses():
    m, n, k = 512, 768, 256
    a = torch.empty(m, k, device=DEV)
    bt = torch.empty(n, k, device=DEV)
    gemm.fill_uniform(a, 1, 0)
    gemm.fill_uniform(bt, 1, m * k)
    whole = gemm.gemm_tf32(a, bt)
    full = [torch.zeros(m, 2 * n, device=DEV) for _ in range(3)]
    gemm.gemm_fanout(a, bt, [f.data_ptr() + n * 4 for f in full], ldc=2 * n)
    for f in full:
        assert torch.equal(f[:, n:], whole) and bool((f[:, :n] == 0).all())


def test_fanout_rejects_bad_arguments():
    a = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    c = torch.zeros(128, 128, device=DEV)
    with pytest.raises(OxgpuError):
        gemm.gemm_fanout(a, a, [c] * 9)
    with pytest.raises(OxgpuError):
        gemm.gemm_fanout(a, a, [], ldc=128)
    with pytest.raises(OxgpuError):
        gemm.gemm_fanout(a, a, [c], flags=gemm.make_flags("1cta_256x128"))
    with pytest.raises(OxgpuError):
        gemm.gemm_fanout(a, a, [c.data_ptr() + 4], ldc=128)


def test_shared_buffer_is_a_tensor_view():
    buf = gemm.SharedBuffer(256 * 4)
    assert len(buf.handle) == 64
    t = buf.tensor((16, 16))
    t.fill_(3.0)
    torch.cuda.synchronize()
    assert t.data_ptr() == buf.ptr and float(t.sum()) == 768.0
    del t
    buf.free()


@pytest.mark.parametrize("variant", FANOUT_VARIANTS)
@pytest.mark.parametrize("alpha,beta,use_bias", [(1.0, 0.0, True), (0.5, 2.0, True), (-1.25, 1.0, False),
                                                 (2.0, 0.0, False)])
def test_affine_epilogue(variant, alpha, beta, use_bias):
    """C = (alpha * AB + beta * C_in) + bias in the GEMM's epilogue equals, bit for
    bit, the same three f32 operations applied to the plain GEMM's output (which
    the other tests hold against the oracle); ragged M and N."""
    m, n, k = 300, 1284, 320
    rng = np.random.default_rng(17)
    a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    a, bt = bf16_tensor(a_bits), bf16_tensor(bt_bits)
    flags = gemm.make_flags(variant)
    plain = gemm.gemm_bf16(a, bt, flags=flags)
    check_bf16(a_bits, bt_bits, plain)
    c_in = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(DEV)
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(DEV) if use_bias else None
    expect = alpha * plain + beta * c_in
    if use_bias:
        expect = expect + bias
    got = gemm.gemm_affine(a, bt, None, alpha, beta, bias, c_in, flags=flags)
    assert torch.equal(got, expect)
    # in place: C_in is C
    c = c_in.clone()
    gemm.gemm_affine(a, bt, c, alpha, beta, bias, flags=flags)
    assert torch.equal(c, expect)


@pytest.mark.parametrize("variant", FANOUT_VARIANTS)
def test_affine_epilogue_with_bf16_output(variant):
    """bias (and alpha, beta * C_in) applied in f32, then ONE rounding to bf16:
    equal to rounding the f32 affine kernel's result."""
    m, n, k = 300, 1288, 320
    rng = np.random.default_rng(19)
    a_bits, bt_bits = rand_bf16(rng, m, k), rand_bf16(rng, n, k)
    a, bt = bf16_tensor(a_bits), bf16_tensor(bt_bits)
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).to(DEV)
    c_in = torch.from_numpy(rng.standard_normal((m, n)).astype(np.float32)).to(DEV)
    flags = gemm.make_flags(variant)
    for alpha, beta in ((1.0, 0.0), (0.5, -2.0)):
        f32 = gemm.gemm_affine(a, bt, None, alpha, beta, bias, c_in, flags=flags)
        pad = torch.full((m + 2, n + 16), float("nan"), device=DEV, dtype=torch.bfloat16)
        c16 = pad[1:m + 1, 8:n + 8]
        gemm.gemm_affine(a, bt, c16, alpha, beta, bias, c_in, flags=flags)
        assert torch.equal(c16, f32.to(torch.bfloat16))
        assert torch.isnan(pad[0]).all() and torch.isnan(pad[-1]).all()
        assert torch.isnan(pad[:, :8]).all() and torch.isnan(pad[:, n + 8:]).all()


def test_affine_epilogue_tf32_and_beta_zero_ignores_c_in():
    m, n, k = 512, 768, 256
    a = torch.empty(m, k, device=DEV)
    bt = torch.empty(n, k, device=DEV)
    gemm.fill_uniform(a, 1, 0)
    gemm.fill_uniform(bt, 1, m * k)
    plain = gemm.gemm_tf32(a, bt)
    bias = torch.arange(n, device=DEV, dtype=torch.float32) * 0.25
    poisoned = torch.full((m, n), float("nan"), device=DEV)
    got = gemm.gemm_affine(a, bt, None, 3.0, 0.0, bias, poisoned)
    assert torch.equal(got, 3.0 * plain + bias)
    with pytest.raises(OxgpuError):
        gemm.gemm_affine(a, bt, None, 1.0, 0.0, flags=gemm.make_flags("1cta_256x128"))
    with pytest.raises(OxgpuError):
        gemm.gemm_affine(a, bt, None, 1.0, 0.0, torch.empty(n + 1, device=DEV)[1:])  # misaligned bias


def test_concurrent_host_threads_on_their_own_streams():
    """The entry points are reentrant per stream: two host threads launch
    different problems on their own streams at the same time; every result must
    equal the one computed alone."""
    import threading
    shapes = [(640, 768, 512), (300, 520, 200)]
    data, alone = [], []
    for i, (m, n, k) in enumerate(shapes):
        a = torch.empty(m, k, device=DEV, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=DEV, dtype=torch.bfloat16)
        gemm.fill_normal(a, 30 + i, 1.0, 0)
        gemm.fill_normal(bt, 30 + i, 1.0, m * k)
        data.append((a, bt))
        alone.append(gemm.gemm_bf16(a, bt))
    torch.cuda.synchronize()
    failures = []

    def worker(i):
        try:
            stream = torch.cuda.Stream()
            a, bt = data[i]
            with torch.cuda.stream(stream):
                for _ in range(20):
                    c = gemm.gemm_bf16(a, bt)
                    bias = torch.zeros(bt.shape[0], device=DEV)
                    c2 = gemm.gemm_affine(a, bt, None, 1.0, 0.0, bias)
                stream.synchronize()
            if not (torch.equal(c, alone[i]) and torch.equal(c2, alone[i])):
                failures.append(i)
        except Exception as e:  # noqa: BLE001
            failures.append(repr(e))

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures


@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (300, 520, 200), (1024, 768, 1024), (128, 264, 2048)])
def test_f32_split_meets_the_strict_bound_on_unrounded_inputs(m, n, k):
    """f32 operands as given (no TF32 rounding on the oracle's side): the
    three-piece TF32 split stays inside 1e-5 * sqrt(K) * max|A| * max|B|, the
    bound stated for f32-in cases, where the plain TF32 path misses it."""
    rng = np.random.default_rng(m + n + k)
    a = rng.uniform(-1, 1, (m, k)).astype(np.float32)
    bt = rng.uniform(-1, 1, (n, k)).astype(np.float32)
    expect = oracle.gemm_kmajor(a, bt, oracle.MODE_NONE, threads=oracle.max_threads())
    ta, tb = torch.from_numpy(a).to(DEV), torch.from_numpy(bt).to(DEV)
    tol = strict_tol(k, float(np.abs(a).max()), float(np.abs(bt).max()))
    got = gemm.gemm_f32_split(ta, tb).cpu().numpy()
    err = float(np.abs(got - expect).max())
    assert err <= tol, (err, tol)
    plain = gemm.gemm_tf32(ta, tb).cpu().numpy()
    assert float(np.abs(plain - expect).max()) > tol          # why the split exists
    exact = gemm.gemm_exact(ta, tb, gemm.INPUT_NONE).cpu().numpy()
    assert np.array_equal(exact.view(np.uint32), expect.view(np.uint32))
    print(f"split err {err:.3e} plain TF32 err {float(np.abs(plain - expect).max()):.3e} tol {tol:.3e}")


def test_f32_split_contract():
    a = torch.zeros(128, 64, device=DEV)
    with pytest.raises(OxgpuError):
        gemm.gemm_f32_split(a, a, workspace=torch.empty(16, dtype=torch.uint8, device=DEV))
    with pytest.raises(OxgpuError):
        gemm.gemm_f32_split(torch.zeros(128, 66, device=DEV)[:, :62], torch.zeros(128, 66, device=DEV)[:, :62])


def test_launches_can_be_captured_in_a_cuda_graph():
    """After one eager call (attributes, occupancy query), the buffer entry
    points only encode maps on the host and launch: a loop of them captures into
    a CUDA graph, and replays give the eager result.  Covers a CTA-pair kernel, the
    in-cluster split-K, the affine epilogue, and a problem large enough for the
    queue-driven tile schedule (the queue slot is part of the captured launch; every
    replay must find it clean, i.e. the previous replay's last cluster reset it)."""
    cases = []
    for (m, n, k) in [(1024, 5120, 256), (128, 1024, 2048), (4096, 8192, 256)]:
        a = torch.empty(m, k, device=DEV, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=DEV, dtype=torch.bfloat16)
        gemm.fill_normal(a, 40, 0.5, 0)
        gemm.fill_normal(bt, 40, 0.5, m * k)
        bias = torch.arange(n, device=DEV, dtype=torch.float32)
        eager = gemm.gemm_bf16(a, bt)
        eager_affine = gemm.gemm_affine(a, bt, None, 2.0, 0.0, bias)
        outs = [torch.zeros(m, n, device=DEV) for _ in range(3)]
        cases.append((a, bt, bias, eager, eager_affine, outs))
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for a, bt, bias, _, _, outs in cases:
            gemm.gemm_bf16(a, bt, outs[0])
            gemm.gemm_bf16(a, bt, outs[1])
            gemm.gemm_affine(a, bt, outs[2], 2.0, 0.0, bias)
    for _ in range(3):
        for *_, outs in cases:
            for o in outs:
                o.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        for _, _, _, eager, eager_affine, outs in cases:
            assert torch.equal(outs[0], eager) and torch.equal(outs[1], eager)
            assert torch.equal(outs[2], eager_affine)


@pytest.mark.parametrize("size", [256, 1024])
def test_back_to_back_launches_see_each_others_results(monkeypatch, size):
    """The GEMM kernels are launched so that each may start its set-up while the
    kernel before it is still running; everything that touches global memory waits
    for that kernel first.  A chain in which every GEMM reads the one before it
    (bf16 C of one is the A of the next), and a C that consecutive launches
    overwrite, must give what the same calls give as ordinary launches with a
    synchronisation after each.  Small problems: a few CTAs each, so the next
    kernel's CTAs really do start on idle SMs while the previous one runs."""
    n = size
    x0 = torch.empty(n, n, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(x0, 41, 1.0, 0)
    ws = []
    for i in range(6):
        w = torch.empty(n, n, device=DEV, dtype=torch.bfloat16)
        gemm.fill_normal(w, 42 + i, 1.0 / n ** 0.5, 0)
        ws.append(w)

    def chain(sync):
        x = x0
        for w in ws:                      # x <- x W^T, six times, each reading the last
            x = gemm.gemm_bf16_out16(x, w)
            if sync:
                torch.cuda.synchronize()
        out = torch.full((n, n), float("nan"), device=DEV)
        for w in ws:                      # the same C written six times: the last one stays
            gemm.gemm_bf16(x, w, out)
            if sync:
                torch.cuda.synchronize()
        torch.cuda.synchronize()
        return x, out

    monkeypatch.setenv("OXGPU_DEPENDENT_LAUNCH", "0")
    want_x, want_out = chain(True)
    monkeypatch.setenv("OXGPU_DEPENDENT_LAUNCH", "1")
    for _ in range(5):
        got_x, got_out = chain(False)
        assert torch.equal(got_x.view(torch.int16), want_x.view(torch.int16))
        assert torch.equal(got_out, want_out)


def test_single_tile_row_problems_do_not_take_tall_tiles():
    """M = 128 against a wide N: a 512-row pair tile would be three quarters
    padding; the library must pick a 128-row tile (same bits as asking for it)."""
    a = torch.empty(128, 512, device=DEV, dtype=torch.bfloat16)
    bt = torch.empty(28672, 512, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(a, 6, 1.0, 0)
    gemm.fill_normal(bt, 6, 1.0, 128 * 512)
    before = gemm.launch_count()
    auto = gemm.gemm_bf16(a, bt)
    assert gemm.launch_count() == before + 1
    assert torch.equal(auto, gemm.gemm_bf16(a, bt, flags=gemm.make_flags("1cta_128x128")))
    exact = gemm.gemm_exact(a, bt, gemm.INPUT_BF16)
    assert float((auto - exact).abs().max()) <= strict_tol(512, float(a.float().abs().max()), float(bt.float().abs().max()))


def test_launch_count_increases():
    before = gemm.launch_count()
    a = torch.zeros(128, 64, device=DEV, dtype=torch.bfloat16)
    gemm.gemm_bf16(a, a)
    assert gemm.launch_count() == before + 1


def test_autotune_sweep_checks_before_it_times():
    """The sweep verifies every candidate against the exact kernel before timing
    it (as the reference's sweep does through its bench, bench/bench.py:294-305),
    nothing is rejected on a healthy build, and the library's own choice is
    close to the best candidate."""
    from oxcamlgpu_b200 import autotune
    rejected = []
    cublas_ms, rows = autotune.sweep(512, 768, 320, repeat=2, warmup=1, cooldown=0, rejected=rejected)
    assert rejected == [] and cublas_ms > 0 and len(rows) >= 8
    labels = [r[0] for r in rows]
    assert "auto (library default)" in labels
    best_ms = rows[0][1]
    auto_ms = next(r[1] for r in rows if r[0] == "auto (library default)")
    # a 6 us kernel timed twice: allow launch jitter on top of the 5 %
    assert auto_ms <= 1.05 * best_ms + 0.004, (auto_ms, best_ms)
    # the check itself: a candidate that produces a wrong result is dropped, not timed
    real = gemm.gemm_bf16
    try:
        def broken(a, bt, c=None, flags=0, **kw):
            out = real(a, bt, c, flags=flags, **kw)
            if (flags & 0xFF) == gemm.V_1CTA_128x128:
                out[0, 0] += 1000.0
            return out
        gemm.gemm_bf16 = broken
        rejected = []
        _, rows2 = autotune.sweep(512, 768, 320, repeat=1, warmup=1, cooldown=0, rejected=rejected)
    finally:
        gemm.gemm_bf16 = real
    assert rejected and all("1cta_128x128" in r[0] for r in rejected)
    assert not any(r[0].startswith("1cta_128x128") for r in rows2)


@pytest.mark.parametrize("variant", TC_VARIANTS)
def test_dynamic_tile_schedule_matches_the_static_walk(variant, monkeypatch):
    """Problems with several tiles per cluster hand their tiles out from a queue
    in walk order (whichever cluster is free takes the next one); which cluster
    computes a tile does not change its value, so the result is bit-equal to the
    static walk's.  Back-to-back launches reuse queue slots (each launch must
    leave its slot clean), and launches on two streams at once use different
    slots."""
    m, n, k = 2048, 4096, 192          # 512 tiles of 128 x 128, 32 of 512 x 256: several per cluster for the small tiles
    if variant in ("2cta_512x256", "2cta_256x512"):
        m, n = 8192, 8192              # 512 pair tiles on 74 pairs
    a = torch.empty(m, k, device=DEV, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=DEV, dtype=torch.bfloat16)
    gemm.fill_normal(a, 31, 1.0, 0)
    gemm.fill_normal(bt, 31, 1.0, m * k)
    flags = gemm.make_flags(variant)
    monkeypatch.setenv("OXGPU_TILE_SCHEDULE", "static")
    static = gemm.gemm_bf16(a, bt, flags=flags)
    torch.cuda.synchronize()
    monkeypatch.delenv("OXGPU_TILE_SCHEDULE")
    outs = [torch.full((m, n), float("nan"), device=DEV) for _ in range(4)]
    for c in outs[:2]:
        gemm.gemm_bf16(a, bt, c, flags=flags)          # back to back on one stream
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    gemm.gemm_bf16(a, bt, outs[2], flags=flags, stream=s1)   # and two at once
    gemm.gemm_bf16(a, bt, outs[3], flags=flags, stream=s2)
    torch.cuda.synchronize()
    for c in outs:
        assert torch.equal(c, static)
    rows = torch.from_numpy(_sample_rows(m, 2, 5)[:3]).long().to(DEV)
    check_bf16(a[rows].contiguous().view(torch.int16).cpu().numpy().view(np.uint16),
               bt.view(torch.int16).cpu().numpy().view(np.uint16), static[rows])
