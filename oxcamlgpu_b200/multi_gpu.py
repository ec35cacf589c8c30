"""One process, several GPUs: the thin Python side of the multi-GPU driver in
liboxgpu_b200.so (oxgpu_b200_mg_*).  The driver itself -- one host thread and
one stream per device, the column partition, peer access, the NCCL all-gather
and the fused peer-store gather -- is C++ behind the C ABI; this file only
marshals pointers.  torch supplies device memory and nothing else.

The reference has no multi-GPU path; its launcher drives one device from one
host thread (test/hardware/run_gemm_h100.cu:100-108,183-186).
"""
from __future__ import annotations

import ctypes

from ._lib import check, lib

GATHER_NONE, GATHER_NCCL, GATHER_FUSED, GATHER_NCCL_BLOCKS = 0, 1, 2, 3
GATHER_NAMES = {"none": GATHER_NONE, "nccl": GATHER_NCCL, "fused": GATHER_FUSED, "nccl_blocks": GATHER_NCCL_BLOCKS}
HOST_C_ROW_MAJOR, HOST_C_BLOCKS = 0, 1
COLUMN_ALIGN = 256


def column_partition(n: int, parts: int, align: int = COLUMN_ALIGN) -> list[tuple[int, int]]:
    """oxgpu_b200_mg_column_partition: the contiguous column ranges the driver
    gives its devices.  Pure host code; works without a GPU."""
    if n <= 0 or parts <= 0 or align <= 0:
        raise ValueError("n, parts and align must be positive")
    lo = (ctypes.c_int * parts)()
    hi = (ctypes.c_int * parts)()
    check(lib().oxgpu_b200_mg_column_partition(n, parts, align, lo, hi))
    return [(int(lo[i]), int(hi[i])) for i in range(parts)]


def _ptr_array(tensors_or_ints, count):
    if tensors_or_ints is None:
        return None
    if len(tensors_or_ints) != count:
        raise ValueError(f"expected {count} entries, one per device")
    vals = [(t if isinstance(t, int) else (0 if t is None else t.data_ptr())) for t in tensors_or_ints]
    return (ctypes.c_void_p * count)(*vals)


class MultiGpu:
    """A driver handle over `devices` (CUDA ordinals; default: the first `ngpu`)."""

    def __init__(self, ngpu: int | None = None, devices: list[int] | None = None):
        if devices is None:
            if ngpu is None:
                raise ValueError("give ngpu or devices")
            devices = list(range(ngpu))
        self.devices = list(devices)
        arr = (ctypes.c_int * len(self.devices))(*self.devices)
        h = ctypes.c_void_p()
        check(lib().oxgpu_b200_mg_create(len(self.devices), arr, ctypes.byref(h)))
        self._h = h

    @property
    def count(self) -> int:
        return len(self.devices)

    @property
    def peer_access(self) -> bool:
        return bool(lib().oxgpu_b200_mg_peer_access(self._h))

    def partition(self, n: int) -> list[tuple[int, int]]:
        return column_partition(n, self.count)

    def gemm_bf16(self, a_repl, bt_shard, c_shard, m: int, n: int, k: int, gather: int | str = GATHER_NONE,
                  c_full=None, flags: int = 0) -> None:
        """Enqueue C[:, shard_d] = A * B[:, shard_d] on every device (lists of
        tensors or raw device addresses, one per device).  Returns when the work
        is enqueued; sync() waits for it."""
        if isinstance(gather, str):
            gather = GATHER_NAMES[gather]
        g = self.count
        check(lib().oxgpu_b200_mg_gemm_bf16(self._h, _ptr_array(a_repl, g), _ptr_array(bt_shard, g),
                                            _ptr_array(c_shard, g), m, n, k, gather, _ptr_array(c_full, g),
                                            flags))

    def sync(self) -> None:
        check(lib().oxgpu_b200_mg_sync(self._h))

    def elapsed_ms(self) -> tuple[list[float], list[float]]:
        """(total, gemm-only) device milliseconds of the last call, per device."""
        tot = (ctypes.c_float * self.count)()
        gem = (ctypes.c_float * self.count)()
        check(lib().oxgpu_b200_mg_elapsed_ms(self._h, tot, gem))
        return list(tot), list(gem)

    def gemm_bf16_host(self, a_host, bt_host, c_host, m: int, n: int, k: int, c_layout: int = HOST_C_ROW_MAJOR,
                       flags: int = 0) -> None:
        """Operands and result in host memory (CPU tensors or raw addresses)."""
        p = lambda t: t if isinstance(t, int) else t.data_ptr()
        check(lib().oxgpu_b200_mg_gemm_bf16_host(self._h, p(a_host), p(bt_host), p(c_host), m, n, k, c_layout,
                                                 flags))

    def alloc(self, index: int, nbytes: int) -> int:
        ptr = ctypes.c_void_p()
        check(lib().oxgpu_b200_mg_alloc(self._h, index, nbytes, ctypes.byref(ptr)))
        return ptr.value

    def free(self, index: int, ptr: int) -> None:
        check(lib().oxgpu_b200_mg_free(self._h, index, ctypes.c_void_p(ptr)))

    def copy(self, index: int, dst: int, src: int, nbytes: int, to_host: bool) -> None:
        check(lib().oxgpu_b200_mg_copy(self._h, index, ctypes.c_void_p(dst), ctypes.c_void_p(src), nbytes,
                                       1 if to_host else 0))

    def close(self) -> None:
        if self._h:
            check(lib().oxgpu_b200_mg_destroy(self._h))
            self._h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class PinnedHostBuffer:
    """oxgpu_b200_host_alloc: pinned host memory placed on the NUMA node of
    `device`, viewable as a torch CPU tensor without a copy."""

    def __init__(self, nbytes: int, device: int = -1):
        ptr = ctypes.c_void_p()
        check(lib().oxgpu_b200_host_alloc(nbytes, device, ctypes.byref(ptr)))
        self.ptr, self.nbytes = ptr.value, nbytes

    def tensor(self, shape, dtype):
        import numpy as np
        import torch
        raw = (ctypes.c_uint8 * self.nbytes).from_address(self.ptr)
        t = torch.from_numpy(np.frombuffer(raw, dtype=np.uint8)).view(dtype).view(*shape)
        t._oxgpu_keepalive = self
        return t

    def free(self) -> None:
        if self.ptr:
            check(lib().oxgpu_b200_host_free(ctypes.c_void_p(self.ptr), self.nbytes))
            self.ptr = 0
