"""Host mirror of the reference's ``Gemm_catalog`` (test/gemm_catalog.ml) and of
the queries ``emit_gemm_ptx`` answers (test/emit_gemm_ptx.ml:39-68).

Same names, same argument meaning, same error text; ``invalid_arg`` becomes
``ValueError``.  The logic lives in the C++ library (csrc/catalog.cpp); this
module only marshals.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from ._lib import OxgpuError, TileConfigStruct, check, lib


@dataclass(frozen=True)
class TileConfig:
    """type tile_config (test/gemm_catalog.ml:9-15)."""
    bm: int
    bn: int
    bk: int
    stages: int
    producers: int

    def _struct(self) -> TileConfigStruct:
        return TileConfigStruct(self.bm, self.bn, self.bk, self.stages, self.producers)

    @staticmethod
    def _from(s: TileConfigStruct) -> "TileConfig":
        return TileConfig(s.bm, s.bn, s.bk, s.stages, s.producers)


def _invalid(fn, *args):
    try:
        return check(fn(*args))
    except OxgpuError as e:
        if e.status < 0:
            raise ValueError(e.message) from None
        raise


def warp_groups(c: TileConfig) -> int:
    """test/gemm_catalog.ml:17."""
    return c.bm // 64


def consumers(c: TileConfig) -> int:
    """test/gemm_catalog.ml:18."""
    return 128 * warp_groups(c)


def threads(c: TileConfig) -> int:
    """test/gemm_catalog.ml:19 (the Hopper CTA width of the reference kernel)."""
    s = c._struct()
    return lib().oxgpu_b200_config_threads(ctypes.byref(s))


def validate(c: TileConfig) -> TileConfig:
    """test/gemm_catalog.ml:21-35; raises ValueError with the reference's text."""
    s = c._struct()
    _invalid(lib().oxgpu_b200_validate_config, ctypes.byref(s))
    return c


def string_of_config(c: TileConfig) -> str:
    """test/gemm_catalog.ml:37-40."""
    s = c._struct()
    buf = ctypes.create_string_buffer(160)
    _invalid(lib().oxgpu_b200_string_of_config, ctypes.byref(s), buf, len(buf))
    return buf.value.decode()


def parse_config(spec: str) -> TileConfig:
    """test/gemm_catalog.ml:42-73."""
    out = TileConfigStruct()
    _invalid(lib().oxgpu_b200_parse_config, spec.encode(), ctypes.byref(out))
    return TileConfig._from(out)


def tile_catalog() -> list[TileConfig]:
    """test/gemm_catalog.ml:80-89."""
    out = []
    for i in range(lib().oxgpu_b200_catalog_size()):
        s = TileConfigStruct()
        check(lib().oxgpu_b200_catalog_get(i, ctypes.byref(s)))
        out.append(TileConfig._from(s))
    return out


def hopper_f32() -> TileConfig:
    """test/gemm_catalog.ml:92-95: the fallback tile, first catalog entry."""
    return tile_catalog()[0]


def kernel_binding(c: TileConfig) -> str:
    """test/gemm_catalog.ml:101-112."""
    s = c._struct()
    name = ctypes.c_char_p()
    _invalid(lib().oxgpu_b200_kernel_binding, ctypes.byref(s), ctypes.byref(name))
    return name.value.decode()


def choose_config(m: int = 4096, n: int = 4096, k: int = 4096) -> TileConfig:
    """test/gemm_catalog.ml:114-137."""
    out = TileConfigStruct()
    _invalid(lib().oxgpu_b200_choose_config, m, n, k, ctypes.byref(out))
    return TileConfig._from(out)


def print_choose(m: int, n: int, k: int) -> str:
    """`emit_gemm_ptx --print-choose M N K` (test/emit_gemm_ptx.ml:44-58)."""
    c = choose_config(m, n, k)
    return f"{kernel_binding(c)} {c.bm} {c.bn} {c.bk} {threads(c)}"


def print_config(spec: str) -> str:
    """`emit_gemm_ptx --print-config SPEC` (test/emit_gemm_ptx.ml:59-64)."""
    c = parse_config(spec)
    return f"{kernel_binding(c)} {c.bm} {c.bn} {c.bk} {threads(c)}"


def list_catalog() -> list[str]:
    """`emit_gemm_ptx --list-catalog` (test/emit_gemm_ptx.ml:65-68)."""
    return [string_of_config(c) for c in tile_catalog()]


def kernel_info(name: str) -> tuple[int, int, int]:
    """`emit_gemm_ptx --info` (test/emit_gemm_ptx.ml:39-43): (threads,
    dynamic shared bytes, total shared bytes) of the B200 kernel serving `name`."""
    t, d, tot = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
    _invalid(lib().oxgpu_b200_kernel_info, name.encode(), ctypes.byref(t), ctypes.byref(d),
             ctypes.byref(tot))
    return t.value, d.value, tot.value


def kernel_tile(name: str) -> tuple[TileConfig, int]:
    """Tile and input element size (bytes) a catalog entry was specialised for
    (examples/kernels/gemm.ml:165-199, gemm_bf16.ml:130-132)."""
    s = TileConfigStruct()
    eb = ctypes.c_int()
    _invalid(lib().oxgpu_b200_kernel_tile, name.encode(), ctypes.byref(s), ctypes.byref(eb))
    return TileConfig._from(s), eb.value


def grouped_tile(pid: int, group: int, tiles_m: int, tiles_n: int) -> tuple[int, int]:
    """Gpu.grouped_tile_m / grouped_tile_n (tools/exporter/export_prims_index.ml:40-61)."""
    tm, tn = ctypes.c_int(), ctypes.c_int()
    _invalid(lib().oxgpu_b200_grouped_tile, pid, group, tiles_m, tiles_n, ctypes.byref(tm),
             ctypes.byref(tn))
    return tm.value, tn.value


def tile_walk(pid: int, group: int, tiles_m: int, tiles_n: int) -> tuple[int, int]:
    """Tile `pid` of the order the library's kernels visit tiles in: grouped_tile
    with the columns of every other group of tile rows reversed."""
    tm, tn = ctypes.c_int(), ctypes.c_int()
    _invalid(lib().oxgpu_b200_tile_walk, pid, group, tiles_m, tiles_n, ctypes.byref(tm), ctypes.byref(tn))
    return tm.value, tn.value


TYPE_NAMES = {1: "scalar_i32", 2: "scalar_f32", 3: "bool", 4: "unit", 5: "buffer_f32", 6: "buffer_bf16",
              7: "buffer_f16", 8: "tensor_map", 9: "scalar_u64"}
OWNERSHIP_NAMES = {1: "unique", 2: "aliased"}
PERMISSION_NAMES = {1: "read", 2: "write", 3: "read_write", 4: "immutable"}


@dataclass(frozen=True)
class GpuArg:
    type: str
    ownership: str
    permission: str


@dataclass(frozen=True)
class GpuHeader:
    """Header of a `.gpu` metadata file (lib/frontend/gpu_metadata.ml, format 3)."""
    kernel: str
    threads: int | None
    args: tuple
    _raw: object = None


def parse_gpu_header(text: str) -> GpuHeader:
    """The header part of Gpu_metadata.parse (gpu_metadata.ml:289-343); raises
    ValueError with the reference's Parse_error text."""
    from ._lib import GpuHeaderStruct
    raw = GpuHeaderStruct()
    data = text.encode()
    _invalid(lib().oxgpu_b200_parse_gpu_header, data, len(data), ctypes.byref(raw))
    args = tuple(GpuArg(TYPE_NAMES[a.type], OWNERSHIP_NAMES[a.ownership], PERMISSION_NAMES[a.permission])
                 for a in list(raw.args)[:raw.nargs])
    return GpuHeader(raw.kernel.decode(), raw.threads or None, args, raw)


def check_gpu_header(header: GpuHeader) -> None:
    """Raises ValueError unless the header describes a GEMM catalog entry this
    library serves (name, CTA width, argument types and modes)."""
    _invalid(lib().oxgpu_b200_check_gpu_header, ctypes.byref(header._raw))


ENTRY_NAMES = (
    "gemm_fast", "gemm_bm128_bn256_s3", "gemm_bm128_bn256_s2", "gemm_bm128_bn128_s3",
    "gemm_bm128_bn128_s2", "gemm_bm64_bn256_s3", "gemm_bm64_bn256_s2", "gemm_bm256_bn128_s3",
    "gemm_bm256_bn128_s2", "gemm_bf16_fast",
)
