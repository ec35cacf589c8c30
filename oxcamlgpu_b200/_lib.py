"""ctypes loader for liboxgpu_b200.so.  Fails loudly when the library is absent:
there is no Python or CPU fallback for any compute entry point."""
from __future__ import annotations

import ctypes
import os

from . import build as _build

_LIB = None


class OxgpuError(RuntimeError):
    """A non-zero status from the C ABI (status < 0: contract violation,
    status > 0: CUDA error), carrying the library's message."""

    def __init__(self, status: int, message: str):
        super().__init__(f"oxgpu_b200 status {status}: {message}")
        self.status = status
        self.message = message


class GpuSlotStruct(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("type", "ownership", "locality", "portability", "permission",
                                            "start_line", "start_col", "end_line", "end_col")]


class GpuHeaderStruct(ctypes.Structure):
    _fields_ = [("kernel", ctypes.c_char * 64), ("threads", ctypes.c_int), ("nargs", ctypes.c_int),
                ("args", GpuSlotStruct * 16), ("result", GpuSlotStruct)]


class EpilogueStruct(ctypes.Structure):
    _fields_ = [("alpha", ctypes.c_float), ("beta", ctypes.c_float), ("bias", ctypes.c_void_p),
                ("c_in", ctypes.c_void_p), ("ldc_in", ctypes.c_int64)]


class TileConfigStruct(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("bm", "bn", "bk", "stages", "producers")]


def lib() -> ctypes.CDLL:
    global _LIB
    if _LIB is not None:
        return _LIB
    path = _build.LIB
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python -m oxcamlgpu_b200.build` "
            "(nvcc, sm_100a).  There is no fallback implementation.")
    L = ctypes.CDLL(path)
    c_int, c_void_p, c_char_p = ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p
    i64, u64, u32, sz = ctypes.c_int64, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_size_t
    cfgp = ctypes.POINTER(TileConfigStruct)
    intp = ctypes.POINTER(c_int)
    sig = {
        "oxgpu_b200_last_error": ([], c_char_p),
        "oxgpu_b200_strerror": ([c_int], c_char_p),
        "oxgpu_b200_config_threads": ([cfgp], c_int),
        "oxgpu_b200_validate_config": ([cfgp], c_int),
        "oxgpu_b200_string_of_config": ([cfgp, c_char_p, sz], c_int),
        "oxgpu_b200_parse_config": ([c_char_p, cfgp], c_int),
        "oxgpu_b200_catalog_size": ([], c_int),
        "oxgpu_b200_catalog_get": ([c_int, cfgp], c_int),
        "oxgpu_b200_kernel_binding": ([cfgp, ctypes.POINTER(c_char_p)], c_int),
        "oxgpu_b200_choose_config": ([c_int, c_int, c_int, cfgp], c_int),
        "oxgpu_b200_kernel_info": ([c_char_p, intp, intp, intp], c_int),
        "oxgpu_b200_kernel_tile": ([c_char_p, cfgp, intp], c_int),
        "oxgpu_b200_parse_gpu_header": ([c_char_p, sz, ctypes.POINTER(GpuHeaderStruct)], c_int),
        "oxgpu_b200_check_gpu_header": ([ctypes.POINTER(GpuHeaderStruct)], c_int),
        "oxgpu_b200_grouped_tile": ([c_int, c_int, c_int, c_int, intp, intp], c_int),
        "oxgpu_b200_tile_walk": ([c_int, c_int, c_int, c_int, intp, intp], c_int),
        "oxgpu_b200_encode_tmap_2d": ([c_void_p, c_void_p, c_int, u64, u64, u64, u32, u32], c_int),
        "oxgpu_b200_gemm_tmap": ([c_char_p, u64, u64, u64, c_int, c_int, c_int, c_void_p], c_int),
        "oxgpu_b200_gemm_tf32": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                  ctypes.c_uint, c_void_p], c_int),
        "oxgpu_b200_gemm_bf16": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                  ctypes.c_uint, c_void_p], c_int),
        "oxgpu_b200_gemm_bf16_out16": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                        ctypes.c_uint, c_void_p], c_int),
        "oxgpu_b200_splitk_workspace_bytes": ([c_int, c_int, c_int], sz),
        "oxgpu_b200_gemm_bf16_ws": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                     ctypes.c_uint, c_void_p, sz, c_void_p], c_int),
        "oxgpu_b200_gemm_bf16_fanout": ([c_void_p, c_void_p, ctypes.POINTER(c_void_p), c_int, c_int, c_int,
                                         c_int, i64, i64, i64, ctypes.c_uint, c_void_p], c_int),
        "oxgpu_b200_gemm_tf32_fanout": ([c_void_p, c_void_p, ctypes.POINTER(c_void_p), c_int, c_int, c_int,
                                         c_int, i64, i64, i64, ctypes.c_uint, c_void_p], c_int),
        "oxgpu_b200_f32_split_workspace_bytes": ([c_int, c_int, c_int], sz),
        "oxgpu_b200_gemm_f32_split": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                       ctypes.c_uint, c_void_p, sz, c_void_p], c_int),
        "oxgpu_b200_gemm_bf16_affine": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                         ctypes.POINTER(EpilogueStruct), ctypes.c_uint, c_void_p], c_int),
        "oxgpu_b200_gemm_bf16_out16_affine": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                               ctypes.POINTER(EpilogueStruct), ctypes.c_uint, c_void_p], c_int),
        "oxgpu_b200_gemm_tf32_affine": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                         ctypes.POINTER(EpilogueStruct), ctypes.c_uint, c_void_p], c_int),
        "oxgpu_b200_shared_alloc": ([sz, ctypes.POINTER(c_void_p), ctypes.c_char_p], c_int),
        "oxgpu_b200_shared_open": ([ctypes.c_char_p, ctypes.POINTER(c_void_p)], c_int),
        "oxgpu_b200_shared_close": ([c_void_p], c_int),
        "oxgpu_b200_shared_free": ([c_void_p], c_int),
        "oxgpu_b200_gemm_bf16_splitk_static": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64,
                                                i64, i64, c_int, c_void_p], c_int),
        "oxgpu_b200_mg_column_partition": ([c_int, c_int, c_int, intp, intp], c_int),
        "oxgpu_b200_mg_create": ([c_int, intp, ctypes.POINTER(c_void_p)], c_int),
        "oxgpu_b200_mg_destroy": ([c_void_p], c_int),
        "oxgpu_b200_mg_device_count": ([c_void_p], c_int),
        "oxgpu_b200_mg_device": ([c_void_p, c_int], c_int),
        "oxgpu_b200_mg_peer_access": ([c_void_p], c_int),
        "oxgpu_b200_mg_gemm_bf16": ([c_void_p, ctypes.POINTER(c_void_p), ctypes.POINTER(c_void_p),
                                     ctypes.POINTER(c_void_p), c_int, c_int, c_int, c_int,
                                     ctypes.POINTER(c_void_p), ctypes.c_uint], c_int),
        "oxgpu_b200_mg_sync": ([c_void_p], c_int),
        "oxgpu_b200_mg_elapsed_ms": ([c_void_p, ctypes.POINTER(ctypes.c_float),
                                      ctypes.POINTER(ctypes.c_float)], c_int),
        "oxgpu_b200_mg_gemm_bf16_host": ([c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                          ctypes.c_uint], c_int),
        "oxgpu_b200_mg_alloc": ([c_void_p, c_int, sz, ctypes.POINTER(c_void_p)], c_int),
        "oxgpu_b200_mg_free": ([c_void_p, c_int, c_void_p], c_int),
        "oxgpu_b200_mg_copy": ([c_void_p, c_int, c_void_p, c_void_p, sz, c_int], c_int),
        "oxgpu_b200_host_alloc": ([sz, c_int, ctypes.POINTER(c_void_p)], c_int),
        "oxgpu_b200_host_free": ([c_void_p, sz], c_int),
        "oxgpu_b200_gemm_exact": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, i64, i64, i64,
                                   c_int, c_void_p], c_int),
        "oxgpu_b200_transpose": ([c_void_p, c_void_p, c_int, c_int, c_int, c_void_p], c_int),
        "oxgpu_b200_f32_to_bf16": ([c_void_p, c_void_p, sz, c_void_p], c_int),
        "oxgpu_b200_transpose_f32_to_bf16": ([c_void_p, c_void_p, c_int, c_int, c_void_p], c_int),
        "oxgpu_b200_gemm_bf16_host": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                       ctypes.c_uint], c_int),
        "oxgpu_b200_gemm_tf32_host": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                       ctypes.c_uint], c_int),
        "oxgpu_b200_gemm_bf16_out16_host": ([c_void_p, c_void_p, c_void_p, c_int, c_int, c_int,
                                             ctypes.c_uint], c_int),
        "oxgpu_b200_release_staging": ([], c_int),
        "oxgpu_b200_fill_uniform": ([c_void_p, sz, c_int, u32, u64, c_void_p], c_int),
        "oxgpu_b200_fill_normal": ([c_void_p, sz, c_int, u32, ctypes.c_float, u64, c_void_p], c_int),
        "oxgpu_b200_device_status": ([ctypes.POINTER(u32)], c_int),
        "oxgpu_b200_selftest_bounded_wait": ([u64], c_int),
        "oxgpu_b200_launch_count": ([], u64),
        "oxgpu_b200_build_info": ([], c_char_p),
    }
    for name, (argtypes, restype) in sig.items():
        fn = getattr(L, name)  # AttributeError if the library lacks a declared symbol
        fn.argtypes = argtypes
        fn.restype = restype
    L._oxgpu_signatures = sig
    _LIB = L
    return L


def check(status: int) -> int:
    if status != 0:
        msg = lib().oxgpu_b200_last_error()
        raise OxgpuError(status, msg.decode("utf-8", "replace") if msg else "")
    return status
