"""Seeded synthetic operands: a counter-based generator (seed, index) -> value.

The same integer hash is implemented on the device (``csrc/synth.cuh``), so a
matrix of any size can be produced in place in HBM and any row of it can be
regenerated on the host.  Uniform values are bit-identical between host and
device (integer arithmetic plus exact float conversions).  Normal values use
Box-Muller through the platform's log/cos, so host and device agree only to a
few ulp; anything that needs the exact device values reads them back.

There is no dataset behind the reference's benchmark (it draws random
matrices, ``bench/bench.py:255-259``); these generators supply the
distributions the workload configurations name.
"""
from __future__ import annotations

import numpy as np

_M32 = np.uint64(0xFFFFFFFF)


def hash_u32(seed: int, index: np.ndarray, stream: int = 0) -> np.ndarray:
    """lowbias32-style finaliser over (seed, stream, 64-bit index) -> uint32."""
    idx = np.asarray(index, dtype=np.uint64)
    lo = idx & _M32
    hi = idx >> np.uint64(32)
    s = np.uint64((int(seed) * 0x9E3779B9 + int(stream) * 0x7F4A7C15 + 0x632BE5AB) & 0xFFFFFFFF)
    x = (lo ^ s ^ ((hi * np.uint64(0x85EBCA6B)) & _M32)) & _M32
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x7FEB352D)) & _M32
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(0x846CA68B)) & _M32
    x ^= x >> np.uint64(16)
    return x.astype(np.uint32)


def uniform_pm1(seed: int, count: int, offset: int = 0) -> np.ndarray:
    """i.i.d. uniform on [-1, 1): multiples of 2^-23, exact in f32."""
    idx = np.arange(offset, offset + count, dtype=np.uint64)
    h = hash_u32(seed, idx, 0)
    return ((h >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -23) - np.float32(1.0)).astype(np.float32)


def normal(seed: int, count: int, std: float = 1.0, offset: int = 0) -> np.ndarray:
    """i.i.d. normal(0, std) by Box-Muller on two hashed uniforms (f32 math)."""
    idx = np.arange(offset, offset + count, dtype=np.uint64)
    h1 = hash_u32(seed, idx, 1)
    h2 = hash_u32(seed, idx, 2)
    u1 = ((h1 >> np.uint32(8)).astype(np.float32) + np.float32(1.0)) * np.float32(2.0 ** -24)
    u2 = (h2 >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)
    r = np.sqrt(np.float32(-2.0) * np.log(u1, dtype=np.float32), dtype=np.float32)
    z = r * np.cos(np.float32(2.0 * np.pi) * u2, dtype=np.float32)
    return (z * np.float32(std)).astype(np.float32)
