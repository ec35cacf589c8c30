"""ctypes front end of the CPU oracle (``gemm_ref.c``).  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference
arm of ``bench.py`` may import this package.  The product package
(``oxcamlgpu_b200``) never does.

The functions follow the reference's host check,
``test/hardware/run_gemm_h100.cu`` (bf16 RNE 26-30, bf16->f32 32-36, TF32
truncation 40-44, operand preparation 137-148, triple loop 150-162, tolerance
191-197); ``tests/golden/make_golden.py`` pins them bit-for-bit against that
file (record: ``tests/golden/reference_pin.json``).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

from . import build as _build

MODE_NONE, MODE_TF32, MODE_BF16 = 0, 1, 2
# The reference's own acceptance thresholds (run_gemm_h100.cu:193).
REFERENCE_ABS_TOL = {"f32": 5e-2, "bf16": 2e-1}

_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = _build.LIB
        if not os.path.exists(path):
            path = _build.build_oracle()
        L = ctypes.CDLL(path)
        i64, f32p, u16p, intp = ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p
        L.oxref_to_bf16.argtypes = [ctypes.c_float]
        L.oxref_to_bf16.restype = ctypes.c_uint16
        L.oxref_of_bf16.argtypes = [ctypes.c_uint16]
        L.oxref_of_bf16.restype = ctypes.c_float
        L.oxref_round_tf32.argtypes = [ctypes.c_float]
        L.oxref_round_tf32.restype = ctypes.c_float
        L.oxref_pattern_a.argtypes = [f32p, ctypes.c_size_t]
        L.oxref_pattern_b.argtypes = [f32p, ctypes.c_size_t]
        L.oxref_prepare_a.argtypes = [f32p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.oxref_prepare_bt.argtypes = [f32p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.oxref_gemm_rowmajor_b.argtypes = [f32p, f32p, f32p] + [ctypes.c_int] * 4
        L.oxref_gemm_kmajor.argtypes = [f32p, i64, f32p, i64, f32p, i64] + [ctypes.c_int] * 4 + [
            intp, ctypes.c_int, ctypes.c_int]
        L.oxref_gemm_kmajor_bf16.argtypes = [u16p, i64, u16p, i64, f32p, i64] + [ctypes.c_int] * 3 + [
            intp, ctypes.c_int, ctypes.c_int]
        L.oxref_compare_abs.argtypes = [f32p, f32p, ctypes.c_size_t, ctypes.c_float,
                                        ctypes.POINTER(ctypes.c_float)]
        L.oxref_compare_abs.restype = ctypes.c_int64
        L.oxref_tolerance.argtypes = [ctypes.c_int, ctypes.c_float, ctypes.c_float]
        L.oxref_tolerance.restype = ctypes.c_float
        L.oxref_max_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def _ptr(a: np.ndarray) -> int:
    return a.ctypes.data


def _c(a, dtype) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=dtype)


# ---- scalar helpers (direct calls into the C restatement) -------------------
def to_bf16_scalar(x: float) -> int:
    return int(lib().oxref_to_bf16(ctypes.c_float(x)))


def of_bf16_scalar(h: int) -> float:
    return float(lib().oxref_of_bf16(ctypes.c_uint16(h)))


def round_tf32_scalar(x: float) -> float:
    return float(lib().oxref_round_tf32(ctypes.c_float(x)))


# ---- vectorised equivalents (numpy; checked against the scalars in tests) ---
def to_bf16(x) -> np.ndarray:
    """bf16 bits (uint16) of an f32 array, RNE as run_gemm_h100.cu:26-30."""
    u = _c(x, np.float32).view(np.uint32)
    lsb = (u >> np.uint32(16)) & np.uint32(1)
    return ((u + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


def of_bf16(h) -> np.ndarray:
    return (_c(h, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_tf32(x) -> np.ndarray:
    u = _c(x, np.float32).view(np.uint32) & np.uint32(0xFFFFE000)
    return u.view(np.float32)


def pattern_inputs(m: int, n: int, k: int):
    """The harness's pattern case (run_gemm_h100.cu:129-130): A[M,K], B[K,N] f32."""
    a = np.empty(m * k, np.float32)
    b = np.empty(k * n, np.float32)
    lib().oxref_pattern_a(_ptr(a), a.size)
    lib().oxref_pattern_b(_ptr(b), b.size)
    return a.reshape(m, k), b.reshape(k, n)


def prepare_operands(a: np.ndarray, b: np.ndarray, narrow: bool):
    """Device operands as the harness builds them (137-148): A[M,K] and B^T[N,K],
    bf16 bits when ``narrow`` else f32."""
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    m, k = a.shape
    k2, n = b.shape
    assert k == k2
    dt = np.uint16 if narrow else np.float32
    a_dev = np.empty((m, k), dt)
    bt_dev = np.empty((n, k), dt)
    lib().oxref_prepare_a(_ptr(a), _ptr(a_dev), m, k, int(narrow))
    lib().oxref_prepare_bt(_ptr(b), _ptr(bt_dev), k, n, int(narrow))
    return a_dev, bt_dev


def gemm_rowmajor_b(a: np.ndarray, b: np.ndarray, mode: int) -> np.ndarray:
    """The triple loop exactly as written (150-162): A[M,K], B[K,N] row-major."""
    a = _c(a, np.float32)
    b = _c(b, np.float32)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), np.float32)
    lib().oxref_gemm_rowmajor_b(_ptr(a), _ptr(b), _ptr(c), m, n, k, mode)
    return c


def _rows_arg(rows):
    if rows is None:
        return None, 0, None
    r = _c(rows, np.int32)
    return _ptr(r), int(r.size), r


def gemm_kmajor(a: np.ndarray, bt: np.ndarray, mode: int, rows=None, threads: int = 1) -> np.ndarray:
    """Same loop on K-major operands A[M,K], B^T[N,K] (f32 values)."""
    a = _c(a, np.float32)
    bt = _c(bt, np.float32)
    m, k = a.shape
    n = bt.shape[0]
    assert bt.shape[1] == k
    rp, nr, keep = _rows_arg(rows)
    out_rows = nr if rows is not None else m
    c = np.empty((out_rows, n), np.float32)
    lib().oxref_gemm_kmajor(_ptr(a), k, _ptr(bt), k, _ptr(c), n, m, n, k, mode, rp, nr, threads)
    del keep
    return c


def gemm_kmajor_bf16(a_bits: np.ndarray, bt_bits: np.ndarray, rows=None, threads: int = 1) -> np.ndarray:
    """Same loop on bf16-bit operands A[M,K], B^T[N,K] (uint16)."""
    a = _c(a_bits, np.uint16)
    bt = _c(bt_bits, np.uint16)
    m, k = a.shape
    n = bt.shape[0]
    assert bt.shape[1] == k
    rp, nr, keep = _rows_arg(rows)
    out_rows = nr if rows is not None else m
    c = np.empty((out_rows, n), np.float32)
    lib().oxref_gemm_kmajor_bf16(_ptr(a), k, _ptr(bt), k, _ptr(c), n, m, n, k, rp, nr, threads)
    del keep
    return c


def compare_abs(got: np.ndarray, expect: np.ndarray, tol: float):
    """(first mismatching flat index or -1, max abs difference) as lines 191-197."""
    g = _c(got, np.float32).ravel()
    e = _c(expect, np.float32).ravel()
    assert g.size == e.size
    worst = ctypes.c_float(0)
    first = lib().oxref_compare_abs(_ptr(g), _ptr(e), g.size, tol, ctypes.byref(worst))
    return int(first), float(worst.value)


def tolerance(k: int, max_a: float, max_b: float) -> float:
    """1e-5 * sqrt(K) * max|A| * max|B| -- the bound for same-rounded inputs."""
    return float(lib().oxref_tolerance(k, max_a, max_b))


def max_threads() -> int:
    return int(lib().oxref_max_threads())
