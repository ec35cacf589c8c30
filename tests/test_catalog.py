"""Catalog parity with the reference's Gemm_catalog (test/gemm_catalog.ml) and
the answers its emitter CLI is pinned to (test/check_oxcaml_signature.sh:234-251).
Host logic only: no GPU."""
import os

import pytest

from oxcamlgpu_b200 import catalog as cat
from oxcamlgpu_b200.catalog import TileConfig


def test_print_choose_answers_pinned_by_the_reference(oxlib):
    # test/check_oxcaml_signature.sh:234-251
    assert cat.print_choose(4096, 4096, 4096) == "gemm_fast 128 256 32 288"
    assert cat.print_choose(8192, 8192, 8192) == "gemm_fast 128 256 32 288"
    assert cat.print_config("bm=64,bn=256,bk=32,stages=2,producers=32,threads=160") == \
        "gemm_bm64_bn256_s2 64 256 32 160"


def test_choose_config_branches(oxlib):
    # test/gemm_catalog.ml:131-136
    assert cat.choose_config(8192, 4096, 64) == TileConfig(256, 128, 32, 3, 32)       # m >= 2n
    assert cat.choose_config(8192, 4097, 64) == TileConfig(128, 256, 32, 4, 32)
    assert cat.choose_config(256, 256, 256) == TileConfig(64, 256, 32, 3, 32)         # small, square-ish
    assert cat.choose_config(1024, 1024, 1) == TileConfig(64, 256, 32, 3, 32)
    assert cat.choose_config(1024, 512, 1) == TileConfig(256, 128, 32, 3, 32)         # m >= 2n wins first
    assert cat.choose_config(512, 1024, 1) == TileConfig(128, 256, 32, 4, 32)         # n >= 2m
    assert cat.choose_config(1025, 1024, 1) == TileConfig(128, 256, 32, 4, 32)
    assert cat.choose_config() == TileConfig(128, 256, 32, 4, 32)                     # defaults 4096
    # the workload shapes: rectangular projections, skinny M, sharded
    assert cat.kernel_binding(cat.choose_config(8192, 28672, 8192)) == "gemm_fast"
    assert cat.kernel_binding(cat.choose_config(128, 8192, 8192)) == "gemm_fast"
    assert cat.kernel_binding(cat.choose_config(32768, 8192, 8192)) == "gemm_bm256_bn128_s3"


def test_tile_catalog_and_bindings(oxlib):
    tiles = cat.tile_catalog()
    assert tiles == [TileConfig(128, 256, 32, 4, 32), TileConfig(128, 256, 32, 3, 32),
                     TileConfig(128, 256, 32, 2, 32), TileConfig(128, 128, 32, 3, 32),
                     TileConfig(128, 128, 32, 2, 32), TileConfig(64, 256, 32, 3, 32),
                     TileConfig(256, 128, 32, 3, 32)]
    assert cat.hopper_f32() == tiles[0]
    assert [cat.kernel_binding(t) for t in tiles] == [
        "gemm_fast", "gemm_bm128_bn256_s3", "gemm_bm128_bn256_s2", "gemm_bm128_bn128_s3",
        "gemm_bm128_bn128_s2", "gemm_bm64_bn256_s3", "gemm_bm256_bn128_s3"]
    assert cat.kernel_binding(TileConfig(64, 256, 32, 2, 32)) == "gemm_bm64_bn256_s2"
    assert cat.kernel_binding(TileConfig(256, 128, 32, 2, 32)) == "gemm_bm256_bn128_s2"
    with pytest.raises(ValueError, match="no OxCaml kernel for bm=128,bn=64,bk=32,stages=3,producers=32,threads=288"):
        cat.kernel_binding(TileConfig(128, 64, 32, 3, 32))
    assert cat.list_catalog()[0] == "bm=128,bn=256,bk=32,stages=4,producers=32,threads=288"
    assert cat.list_catalog()[5] == "bm=64,bn=256,bk=32,stages=3,producers=32,threads=160"
    assert cat.list_catalog()[6] == "bm=256,bn=128,bk=32,stages=3,producers=32,threads=544"


def test_threads(oxlib):
    # consumers = 128 * (bm / 64), threads = consumers + producers
    assert cat.threads(TileConfig(128, 256, 32, 4, 32)) == 288
    assert cat.threads(TileConfig(64, 256, 32, 3, 32)) == 160
    assert cat.threads(TileConfig(256, 128, 32, 3, 32)) == 544
    assert cat.consumers(TileConfig(256, 128, 32, 3, 64)) == 512 and cat.warp_groups(TileConfig(192, 8, 32, 2, 32)) == 3


@pytest.mark.parametrize("cfg,msg", [
    (TileConfig(96, 256, 32, 3, 32), "BM must be a positive multiple of 64"),
    (TileConfig(0, 256, 32, 3, 32), "BM must be a positive multiple of 64"),
    (TileConfig(128, 260, 32, 3, 32), "BN must be in"),
    (TileConfig(128, 0, 32, 3, 32), "BN must be in"),
    (TileConfig(128, 264, 32, 3, 32), "BN must be in"),
    (TileConfig(128, 256, 64, 3, 32), "BK must be 32"),
    (TileConfig(128, 256, 16, 3, 32), "BK must be 32"),
    (TileConfig(128, 256, 32, 1, 32), "pipeline stages must be"),
    (TileConfig(128, 256, 32, 3, 0), "producers must be a positive multiple"),
    (TileConfig(128, 256, 32, 3, 48), "producers must be a positive multiple"),
    (TileConfig(512, 256, 32, 3, 32), "CTA threads"),
])
def test_validate_rejections(oxlib, cfg, msg):
    with pytest.raises(ValueError, match=msg):
        cat.validate(cfg)


def test_validate_accepts(oxlib):
    for t in cat.tile_catalog():
        assert cat.validate(t) == t
    assert cat.validate(TileConfig(448, 8, 32, 2, 128)) == TileConfig(448, 8, 32, 2, 128)  # 1024 threads


def test_parse_config(oxlib):
    assert cat.parse_config("bm=128,bn=256,bk=32,stages=4,producers=32") == TileConfig(128, 256, 32, 4, 32)
    # stages defaults to 3; unknown keys (legacy tm/tn, threads) ignored; whitespace trimmed
    assert cat.parse_config(" bm = 128 , bn=128,bk=32, producers=32 ,tm=8,tn=8") == TileConfig(128, 128, 32, 3, 32)
    assert cat.parse_config(cat.string_of_config(TileConfig(64, 256, 32, 2, 32))) == TileConfig(64, 256, 32, 2, 32)
    with pytest.raises(ValueError, match="bad config fragment: bm"):
        cat.parse_config("bm,bn=1")
    with pytest.raises(ValueError, match="bad config fragment: bm=1=2"):
        cat.parse_config("bm=1=2")
    with pytest.raises(ValueError, match="config key bm is not an integer: oops"):
        cat.parse_config("bm=oops,bn=256,bk=32,producers=32")
    with pytest.raises(ValueError, match="missing config key: producers"):
        cat.parse_config("bm=128,bn=256,bk=32")
    with pytest.raises(ValueError, match="missing config key: bn"):
        cat.parse_config("bm=128,bk=32,producers=32")
    with pytest.raises(ValueError, match="BK must be 32"):
        cat.parse_config("bm=128,bn=256,bk=64,producers=32")
    with pytest.raises(ValueError, match="bad config fragment: $"):
        cat.parse_config("")


def test_kernel_info_and_tiles(oxlib):
    for name in cat.ENTRY_NAMES:
        threads, dyn, total = cat.kernel_info(name)
        assert threads == 320                       # 10 warps: TMA, UMMA, 8 epilogue
        assert 118784 <= dyn <= 232448 and total == dyn
        tile, eb = cat.kernel_tile(name)
        assert eb == (2 if name == "gemm_bf16_fast" else 4)
        assert tile.bk * eb == 128                  # one 128-byte swizzle row per K block
    assert cat.kernel_tile("gemm_fast")[0] == TileConfig(128, 256, 32, 4, 32)
    assert cat.kernel_tile("gemm_bf16_fast")[0] == TileConfig(128, 256, 64, 4, 32)
    # deeper rings need more shared memory
    assert cat.kernel_info("gemm_fast")[1] > cat.kernel_info("gemm_bm128_bn256_s3")[1] > \
        cat.kernel_info("gemm_bm128_bn256_s2")[1]
    with pytest.raises(ValueError, match="no kernel named gemm_slow"):
        cat.kernel_info("gemm_slow")


@pytest.mark.parametrize("tiles_m,tiles_n,group", [(64, 32, 16), (5, 3, 16), (17, 4, 16), (33, 1, 16),
                                                   (1, 9, 16), (20, 7, 8), (16, 16, 16), (31, 2, 4)])
def test_grouped_tile_is_a_bijection(oxlib, tiles_m, tiles_n, group):
    """tools/exporter/export_prims_index.ml:33-39: every tile exactly once,
    including a short last group."""
    seen = set()
    for pid in range(tiles_m * tiles_n):
        tm, tn = cat.grouped_tile(pid, group, tiles_m, tiles_n)
        assert 0 <= tm < tiles_m and 0 <= tn < tiles_n
        # independent restatement of the formula
        per_group = group * tiles_n
        first = (pid // per_group) * group
        rows = min(tiles_m - first, group)
        assert (tm, tn) == (first + pid % rows, (pid % per_group) // rows)
        seen.add((tm, tn))
    assert len(seen) == tiles_m * tiles_n
    # a group walks `group` tile-rows before moving along N
    if tiles_m >= group and tiles_n > 1:
        assert [cat.grouped_tile(p, group, tiles_m, tiles_n) for p in range(group + 1)] == \
            [(i, 0) for i in range(group)] + [(0, 1)]
    with pytest.raises(ValueError):
        cat.grouped_tile(tiles_m * tiles_n, group, tiles_m, tiles_n)


# ---- .gpu metadata header (lib/frontend/gpu_metadata.ml, format 3) -----------------
def _gpu_text(kernel="gemm_fast", threads=288, args=None, fmt="3", result=True, body=True):
    span = '"examples/kernels/gemm.ml"\t50\t6\t50\t12'
    if args is None:
        args = [("tensor_map", "aliased", "global", "nonportable", "read"),
                ("tensor_map", "aliased", "global", "nonportable", "read"),
                ("buffer_f32", "unique", "global", "nonportable", "read_write"),
                ("scalar_i32", "aliased", "global", "portable", "read"),
                ("scalar_i32", "aliased", "global", "portable", "read"),
                ("scalar_i32", "aliased", "global", "portable", "read")]
    rows = [f"format\t{fmt}", f"kernel\t{kernel}"]
    if threads is not None:
        rows.append(f"threads\t{threads}")
    for i, a in enumerate(args):
        rows.append("\t".join(["arg", str(i), *a, span]))
    if result:
        rows.append("\t".join(["result", "unit", "aliased", "global", "portable", "read", span]))
    if body:
        rows += ['loc\t"examples/kernels/gemm.ml"\t54\t4\t54\t60', "body\tconst_i32\t0\t128", "yield\t-"]
    return "\n".join(rows) + "\n"


@pytest.mark.parametrize("tiles_m,tiles_n,group", [(1, 1, 16), (16, 32, 4), (17, 5, 4), (3, 700, 8), (64, 256, 4), (7, 3, 16),
                                                    (1, 2048, 16), (2048, 2047, 16)])
def test_tile_walk_is_grouped_tile_with_every_other_group_reversed(oxlib, tiles_m, tiles_n, group):
    """The kernels' walk goes through multiply-by-reciprocal arithmetic (magic
    numbers for the launch's divisors, plain division for the last, shorter group
    of tile rows, and for tile counts too large for the reciprocal to be exact --
    the 2048 x 2047 case): it must agree with the reference's grouped order,
    columns reversed in odd groups, for every tile."""
    total = tiles_m * tiles_n
    pids = range(total) if total <= 20000 else list(range(0, total, 997)) + [total - 1, total - 2]
    seen = set()
    for pid in pids:
        tm, tn = cat.grouped_tile(pid, group, tiles_m, tiles_n)
        if (tm // group) & 1:
            tn = tiles_n - 1 - tn
        assert cat.tile_walk(pid, group, tiles_m, tiles_n) == (tm, tn)
        seen.add((tm, tn))
    if total <= 20000:
        assert len(seen) == total
    with pytest.raises(Exception):
        cat.tile_walk(total, group, tiles_m, tiles_n)



def test_gpu_header_round_trip_and_check(oxlib):
    h = cat.parse_gpu_header(_gpu_text())
    assert h.kernel == "gemm_fast" and h.threads == 288 and len(h.args) == 6
    assert h.args[0] == cat.GpuArg("tensor_map", "aliased", "read")
    assert h.args[2] == cat.GpuArg("buffer_f32", "unique", "read_write")
    assert h.args[5].type == "scalar_i32"
    cat.check_gpu_header(h)
    # every f32 entry with its Hopper CTA width (gemm.ml:165-199)
    for name in cat.ENTRY_NAMES:
        tile, _ = cat.kernel_tile(name)
        cat.check_gpu_header(cat.parse_gpu_header(_gpu_text(kernel=name, threads=128 * (tile.bm // 64) + 32)))
    # blank lines are dropped, a file without `threads` parses
    assert cat.parse_gpu_header("\n" + _gpu_text(threads=None)).threads is None


@pytest.mark.parametrize("text,msg", [
    (_gpu_text(fmt="2"), "malformed region/header"),
    ("kernel\tgemm_fast\n", "malformed region/header"),
    ("format\t3\nthreads\t288\n", "missing kernel"),
    (_gpu_text(threads=0), "CTA thread count must be in 1..1024"),
    (_gpu_text(threads=2048), "CTA thread count must be in 1..1024"),
    (_gpu_text(threads="many"), "invalid integer many"),
    (_gpu_text(result=False, body=False), "missing result"),
    (_gpu_text(args=[("tensor_map", "shared", "global", "nonportable", "read")]), "invalid ownership"),
    (_gpu_text(args=[("tensor_map", "aliased", "global", "nonportable", "execute")]), "invalid permission"),
    (_gpu_text(args=[("tensor_map", "aliased", "remote", "nonportable", "read")]), "invalid locality"),
    (_gpu_text(args=[("matrix", "aliased", "global", "nonportable", "read")]), "unsupported frontend type"),
    (_gpu_text(args=[("tensor_map", "aliased", "global", "nonportable")]), "missing or extra mode fields"),
])
def test_gpu_header_parse_errors(oxlib, text, msg):
    with pytest.raises(ValueError, match=msg):
        cat.parse_gpu_header(text)


def test_gpu_header_rejects_the_reference_tests_own_vectors(oxlib, golden_dir):
    """Every `.gpu` text the reference's tests require its parser to refuse
    (test/test_frontend.ml:25-28, test/check_compiler_metadata.ml:8; extracted by
    tests/golden/make_golden.py) is refused here too."""
    import json
    vectors = json.load(open(os.path.join(golden_dir, "gpu_header_rejected.json")))
    assert len(vectors) >= 5
    for v in vectors:
        with pytest.raises(ValueError):
            cat.parse_gpu_header(v["text"])


def test_gpu_header_noncontiguous_args(oxlib):
    text = _gpu_text().replace("arg\t1\t", "arg\t4\t", 1)
    with pytest.raises(ValueError, match="argument ids must be contiguous"):
        cat.parse_gpu_header(text)


def test_gpu_header_check_rejections(oxlib):
    with pytest.raises(ValueError, match="no kernel named saxpy"):
        cat.check_gpu_header(cat.parse_gpu_header(_gpu_text(kernel="saxpy")))
    with pytest.raises(ValueError, match="specialised for 288 threads per CTA, the metadata says 160"):
        cat.check_gpu_header(cat.parse_gpu_header(_gpu_text(threads=160)))
    with pytest.raises(ValueError, match="specialised for 160 threads"):
        cat.check_gpu_header(cat.parse_gpu_header(_gpu_text(kernel="gemm_bm64_bn256_s3", threads=288)))
    saxpy_args = [("buffer_f32", "aliased", "global", "nonportable", "read"),
                  ("buffer_f32", "unique", "global", "nonportable", "read_write")]
    with pytest.raises(ValueError, match="six arguments"):
        cat.check_gpu_header(cat.parse_gpu_header(_gpu_text(args=saxpy_args)))
    bad = [("tensor_map", "unique", "global", "nonportable", "read")] + [None] * 5
    full = cat.parse_gpu_header(_gpu_text())
    args = [("tensor_map", "unique", "global", "nonportable", "read"),
            ("tensor_map", "aliased", "global", "nonportable", "read"),
            ("buffer_f32", "unique", "global", "nonportable", "read_write")] + \
           [("scalar_i32", "aliased", "global", "portable", "read")] * 3
    with pytest.raises(ValueError, match="tensor maps, aliased and read-only"):
        cat.check_gpu_header(cat.parse_gpu_header(_gpu_text(args=args)))
    args[0] = ("tensor_map", "aliased", "global", "nonportable", "read")
    args[2] = ("buffer_f32", "aliased", "global", "nonportable", "read_write")
    with pytest.raises(ValueError, match="unique and read_write"):
        cat.check_gpu_header(cat.parse_gpu_header(_gpu_text(args=args)))
    args[2] = ("buffer_f32", "unique", "global", "nonportable", "read_write")
    args[4] = ("scalar_f32", "aliased", "global", "portable", "read")
    with pytest.raises(ValueError, match="i32 scalars"):
        cat.check_gpu_header(cat.parse_gpu_header(_gpu_text(args=args)))
    del bad, full
