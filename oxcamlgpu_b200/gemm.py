"""Host launcher above the C ABI, mirroring the reference's two launchers:
the C harness test/hardware/run_gemm_h100.cu (encode_tiled_2d 46-72, launch
164-186) and bench/bench.py (encode_tensor_map_2d 126-147,
alloc_device_tensor_map 150-156, launch_mm 281-292).

torch is used for device memory and streams only; every GEMM below is a call
into liboxgpu_b200.so.
"""
from __future__ import annotations

import ctypes

import torch

from . import catalog
from ._lib import EpilogueStruct, check, lib

(VARIANT_AUTO, V_1CTA_128x256, V_1CTA_128x128, V_1CTA_256x128, V_2CTA_256x256, V_2CTA_256x128, V_SPLITK,
 V_2CTA_512x256, V_1CTA_256x256, V_CSPLITK_128x256, V_CSPLITK_128x128, V_2CTA_256x512) = range(12)
VARIANT_NAMES = {
    "auto": VARIANT_AUTO, "1cta_128x256": V_1CTA_128x256, "1cta_128x128": V_1CTA_128x128,
    "1cta_256x128": V_1CTA_256x128, "2cta_256x256": V_2CTA_256x256, "2cta_256x128": V_2CTA_256x128,
    "splitk": V_SPLITK, "2cta_512x256": V_2CTA_512x256, "1cta_256x256": V_1CTA_256x256,
    "cluster_splitk_128x256": V_CSPLITK_128x256, "cluster_splitk_128x128": V_CSPLITK_128x128,
    "2cta_256x512": V_2CTA_256x512,
}
ELEMENT_BYTES = {"f32": 4, "bf16": 2}
INPUT_NONE, INPUT_TF32, INPUT_BF16 = 0, 1, 2


def make_flags(variant: int | str = VARIANT_AUTO, stages: int = 0, group_m: int = 0, splits: int = 0,
               reorder: int = 0) -> int:
    """reorder: K blocks issued block-major at tile ends (256-row variants);
    0 = library default, 15 = never."""
    if isinstance(variant, str):
        variant = VARIANT_NAMES[variant]
    return ((variant & 0xFF) | ((stages & 0xF) << 8) | ((group_m & 0xFF) << 12) | ((splits & 0xFF) << 20) |
            ((reorder & 0xF) << 28))


def _stream(stream=None) -> int:
    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


class TensorMap(ctypes.Structure):
    """A 128-byte CUtensorMap in host memory (64-byte aligned)."""
    _fields_ = [("opaque", ctypes.c_uint64 * 16)]
    _align_ = 64


def encode_tensor_map_2d(device_ptr: int, dim0: int, dim1: int, stride1_bytes: int, box0: int,
                         box1: int, element: str = "f32") -> ctypes.Array:
    """bench/bench.py:126-147 / run_gemm_h100.cu:46-72: 2-D tiled, 128-byte
    swizzle, L2 promotion 128 B, zero fill."""
    raw = (ctypes.c_uint8 * 192)()
    base = ctypes.addressof(raw)
    off = (-base) % 64
    check(lib().oxgpu_b200_encode_tmap_2d(ctypes.c_void_p(base + off), ctypes.c_void_p(device_ptr),
                                          ELEMENT_BYTES[element], dim0, dim1, stride1_bytes, box0,
                                          box1))
    out = (ctypes.c_uint8 * 128)()
    ctypes.memmove(out, base + off, 128)
    return out


def alloc_device_tensor_map(host_map) -> torch.Tensor:
    """bench/bench.py:150-156: copy a host CUtensorMap into device memory."""
    cpu = torch.empty(128, dtype=torch.uint8)
    ctypes.memmove(cpu.data_ptr(), host_map, 128)
    return cpu.cuda()


def launch_catalog(name: str, d_a_map: torch.Tensor, d_b_map: torch.Tensor, c: torch.Tensor, m: int,
                   n: int, k: int, stream=None) -> None:
    """Launch a catalog entry point with reference-style arguments (device
    pointers to the A and B^T maps, C, m, n, k): run_gemm_h100.cu:183-185."""
    check(lib().oxgpu_b200_gemm_tmap(name.encode(), d_a_map.data_ptr(), d_b_map.data_ptr(),
                                     c.data_ptr(), m, n, k, ctypes.c_void_p(_stream(stream))))


def run_catalog_entry(name: str, a: torch.Tensor, bt: torch.Tensor, c: torch.Tensor | None = None):
    """Everything the reference's harness does around one launch: encode the
    maps with the entry's boxes, put them in device memory, launch."""
    tile, ebytes = catalog.kernel_tile(name)
    element = "bf16" if ebytes == 2 else "f32"
    m, k = a.shape
    n = bt.shape[0]
    if c is None:
        c = torch.empty(m, n, device=a.device, dtype=torch.float32)
    a_map = encode_tensor_map_2d(a.data_ptr(), k, m, k * ebytes, tile.bk, tile.bm, element)
    b_map = encode_tensor_map_2d(bt.data_ptr(), k, n, k * ebytes, tile.bk, tile.bn, element)
    da, db = alloc_device_tensor_map(a_map), alloc_device_tensor_map(b_map)
    launch_catalog(name, da, db, c, m, n, k)
    c._oxgpu_keepalive = (da, db)
    return c


def _check_operands(a: torch.Tensor, bt: torch.Tensor, dtype) -> tuple[int, int, int]:
    if not (a.is_cuda and bt.is_cuda):
        raise ValueError("operands must be CUDA tensors")
    if a.dtype != dtype or bt.dtype != dtype:
        raise ValueError(f"operands must be {dtype}")
    if a.dim() != 2 or bt.dim() != 2 or a.shape[1] != bt.shape[1]:
        raise ValueError("expected A[M,K] and B^T[N,K]")
    if a.stride(1) != 1 or bt.stride(1) != 1:
        raise ValueError("operands must be K-contiguous")
    return a.shape[0], bt.shape[0], a.shape[1]


def _out(c, m, n, device):
    if c is None:
        c = torch.empty(m, n, device=device, dtype=torch.float32)
    if c.dtype != torch.float32 or c.stride(1) != 1 or tuple(c.shape) != (m, n):
        raise ValueError("C must be f32 [M,N] with unit column stride")
    return c


def gemm_bf16(a: torch.Tensor, bt: torch.Tensor, c: torch.Tensor | None = None, flags: int = 0,
              workspace: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """C = A * B with bf16 A[M,K], B^T[N,K]; f32 out (gemm_bf16.ml:33-128)."""
    m, n, k = _check_operands(a, bt, torch.bfloat16)
    c = _out(c, m, n, a.device)
    s = ctypes.c_void_p(_stream(stream))
    if (flags & 0xFF) == V_SPLITK:
        if workspace is None:
            need = lib().oxgpu_b200_splitk_workspace_bytes(m, n, (flags >> 20) & 0xFF)
            workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
        check(lib().oxgpu_b200_gemm_bf16_ws(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k,
                                            a.stride(0), bt.stride(0), c.stride(0), flags,
                                            workspace.data_ptr(), workspace.numel() * workspace.element_size(), s))
        c._oxgpu_keepalive = workspace
    else:
        check(lib().oxgpu_b200_gemm_bf16(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k,
                                         a.stride(0), bt.stride(0), c.stride(0), flags, s))
    return c


def gemm_f32_split(a: torch.Tensor, bt: torch.Tensor, c: torch.Tensor | None = None, flags: int = 0,
                   workspace: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """f32 A[M,K], B^T[N,K] -> f32 C at close to f32 accuracy on the tensor cores:
    operands split into TF32 part + remainder, one TF32 GEMM over 3K."""
    m, n, k = _check_operands(a, bt, torch.float32)
    c = _out(c, m, n, a.device)
    need = lib().oxgpu_b200_f32_split_workspace_bytes(m, n, k)
    if workspace is None:
        workspace = torch.empty(need, dtype=torch.uint8, device=a.device)
    check(lib().oxgpu_b200_gemm_f32_split(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k, a.stride(0),
                                          bt.stride(0), c.stride(0), flags, workspace.data_ptr(),
                                          workspace.numel() * workspace.element_size(),
                                          ctypes.c_void_p(_stream(stream))))
    c._oxgpu_keepalive = workspace
    return c


def gemm_affine(a: torch.Tensor, bt: torch.Tensor, c: torch.Tensor | None = None, alpha: float = 1.0,
                beta: float = 0.0, bias: torch.Tensor | None = None, c_in: torch.Tensor | None = None,
                flags: int = 0, stream=None) -> torch.Tensor:
    """C = (alpha * (A B) + beta * C_in) + bias in the GEMM's epilogue (bf16 or
    f32/TF32 operands by dtype).  c_in defaults to c (in-place) when beta != 0."""
    kind = {torch.bfloat16: "bf16", torch.float32: "tf32"}.get(a.dtype)
    if kind is None:
        raise ValueError("operands must be bf16 or f32")
    m, n, k = _check_operands(a, bt, a.dtype)
    out16 = c is not None and c.dtype == torch.bfloat16      # bf16 C: pass a bf16 tensor to write into
    if out16:
        if kind != "bf16" or c.stride(1) != 1 or tuple(c.shape) != (m, n):
            raise ValueError("bf16 C needs bf16 operands and a [M,N] tensor with unit column stride")
        if beta != 0.0 and c_in is None:
            raise ValueError("with bf16 C, c_in (f32) must be given when beta != 0")
    else:
        c = _out(c, m, n, a.device)
    if beta != 0.0 and c_in is None:
        c_in = c
    if bias is not None and (bias.dtype != torch.float32 or tuple(bias.shape) != (n,) or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous f32 vector of length N")
    if c_in is not None and (c_in.dtype != torch.float32 or tuple(c_in.shape) != (m, n) or c_in.stride(1) != 1):
        raise ValueError("c_in must be f32 [M,N] with unit column stride")
    ep = EpilogueStruct(alpha, beta, bias.data_ptr() if bias is not None else None,
                        c_in.data_ptr() if c_in is not None else None,
                        c_in.stride(0) if c_in is not None else 0)
    fn = (lib().oxgpu_b200_gemm_bf16_out16_affine if out16 else
          lib().oxgpu_b200_gemm_bf16_affine if kind == "bf16" else lib().oxgpu_b200_gemm_tf32_affine)
    check(fn(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k, a.stride(0), bt.stride(0), c.stride(0),
             ctypes.byref(ep), flags, ctypes.c_void_p(_stream(stream))))
    return c


def gemm_fanout(a: torch.Tensor, bt: torch.Tensor, dests, ldc: int | None = None, flags: int = 0,
                stream=None) -> None:
    """C = A * B written to every destination in `dests` by one kernel (bf16 or
    f32/TF32 operands by dtype).  A destination is either an f32 tensor view
    [M,N] with unit column stride (its row stride must equal `ldc` of the
    others) or a raw device address (int) of the window's first element, in
    which case `ldc` is required -- the form used for windows inside another
    process's memory."""
    kind = {torch.bfloat16: "bf16", torch.float32: "tf32"}.get(a.dtype)
    if kind is None:
        raise ValueError("operands must be bf16 or f32")
    m, n, k = _check_operands(a, bt, a.dtype)
    ptrs = []
    for d in dests:
        if isinstance(d, int):
            ptrs.append(d)
            continue
        if d.dtype != torch.float32 or d.stride(1) != 1 or tuple(d.shape) != (m, n):
            raise ValueError("a destination must be f32 [M,N] with unit column stride")
        if ldc is None:
            ldc = d.stride(0)
        if d.stride(0) != ldc:
            raise ValueError("all destinations share one leading dimension")
        ptrs.append(d.data_ptr())
    if ldc is None:
        raise ValueError("ldc is required when destinations are raw addresses")
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    fn = lib().oxgpu_b200_gemm_bf16_fanout if kind == "bf16" else lib().oxgpu_b200_gemm_tf32_fanout
    check(fn(a.data_ptr(), bt.data_ptr(), arr, len(ptrs), m, n, k, a.stride(0), bt.stride(0), ldc, flags,
             ctypes.c_void_p(_stream(stream))))


class SharedBuffer:
    """Device memory of this process that other processes can map
    (oxgpu_b200_shared_alloc), viewable as a torch tensor without a copy."""

    def __init__(self, nbytes: int, device: torch.device | int | None = None):
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None else
                                   (device if isinstance(device, int) else device.index))
        self.nbytes = nbytes
        ptr = ctypes.c_void_p()
        handle = ctypes.create_string_buffer(64)
        with torch.cuda.device(self.device):
            check(lib().oxgpu_b200_shared_alloc(nbytes, ctypes.byref(ptr), handle))
        self.ptr = ptr.value
        self.handle = handle.raw

    def tensor(self, shape, dtype=torch.float32) -> torch.Tensor:
        holder = type("_CudaArray", (), {})()
        holder.__cuda_array_interface__ = {
            "shape": tuple(shape), "typestr": {torch.float32: "<f4", torch.uint8: "|u1"}[dtype],
            "data": (self.ptr, False), "version": 2}
        t = torch.as_tensor(holder, device=self.device)
        t._oxgpu_keepalive = self
        return t

    def free(self) -> None:
        if self.ptr:
            check(lib().oxgpu_b200_shared_free(ctypes.c_void_p(self.ptr)))
            self.ptr = 0


def shared_open(handle: bytes) -> int:
    """Map another process's SharedBuffer; returns the address in this process."""
    ptr = ctypes.c_void_p()
    check(lib().oxgpu_b200_shared_open(handle, ctypes.byref(ptr)))
    return ptr.value


def shared_close(ptr: int) -> None:
    check(lib().oxgpu_b200_shared_close(ctypes.c_void_p(ptr)))


def gemm_bf16_out16(a: torch.Tensor, bt: torch.Tensor, c: torch.Tensor | None = None, flags: int = 0,
                    stream=None) -> torch.Tensor:
    """bf16 A[M,K], B^T[N,K] -> bf16 C[M,N] (f32 accumulation, one RNE rounding at
    the store): the narrow-output epilogue of docs/roadmap.md:67-71."""
    m, n, k = _check_operands(a, bt, torch.bfloat16)
    if c is None:
        c = torch.empty(m, n, device=a.device, dtype=torch.bfloat16)
    if c.dtype != torch.bfloat16 or c.stride(1) != 1 or tuple(c.shape) != (m, n):
        raise ValueError("C must be bf16 [M,N] with unit column stride")
    check(lib().oxgpu_b200_gemm_bf16_out16(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k, a.stride(0),
                                           bt.stride(0), c.stride(0), flags,
                                           ctypes.c_void_p(_stream(stream))))
    return c


STATIC_SCRATCH_BYTES = 32 << 20


def gemm_bf16_splitk_static(a: torch.Tensor, bt: torch.Tensor, c: torch.Tensor, splits: int = 0,
                            stream=None) -> torch.Tensor:
    """Split-K bf16 GEMM for callers that cannot allocate device memory at call
    time (memory handed out up front by an arena or a fixed budget, or a loop
    that cannot tolerate an allocation's device-wide synchronisation): the K
    slices' partial tiles go to a fixed 32 MiB array inside the library instead
    of a workspace, so the caller passes only A, B^T and C.  Raises OxgpuError
    (status -6) when the slices would not fit.  Calls that overlap on one GPU
    race on that array; keep them on one stream."""
    m, n, k = _check_operands(a, bt, torch.bfloat16)
    c = _out(c, m, n, a.device)
    check(lib().oxgpu_b200_gemm_bf16_splitk_static(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k,
                                                   a.stride(0), bt.stride(0), c.stride(0), splits,
                                                   ctypes.c_void_p(_stream(stream))))
    return c


def gemm_tf32(a: torch.Tensor, bt: torch.Tensor, c: torch.Tensor | None = None, flags: int = 0,
              stream=None) -> torch.Tensor:
    """C = A * B with f32 A[M,K], B^T[N,K] rounded to TF32 by the matrix unit
    (gemm.ml:47-163)."""
    m, n, k = _check_operands(a, bt, torch.float32)
    c = _out(c, m, n, a.device)
    check(lib().oxgpu_b200_gemm_tf32(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k, a.stride(0),
                                     bt.stride(0), c.stride(0), flags, ctypes.c_void_p(_stream(stream))))
    return c


def gemm_exact(a: torch.Tensor, bt: torch.Tensor, input_mode: int, c: torch.Tensor | None = None,
               stream=None) -> torch.Tensor:
    """Bit-exact device restatement of the host reference loop
    (run_gemm_h100.cu:150-162) -- see oxgpu_b200_gemm_exact."""
    dtype = torch.bfloat16 if input_mode == INPUT_BF16 else torch.float32
    m, n, k = _check_operands(a, bt, dtype)
    c = _out(c, m, n, a.device)
    check(lib().oxgpu_b200_gemm_exact(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k, a.stride(0),
                                      bt.stride(0), c.stride(0), input_mode,
                                      ctypes.c_void_p(_stream(stream))))
    return c


def transpose(b: torch.Tensor, stream=None) -> torch.Tensor:
    """B[K,N] -> B^T[N,K] on the device (run_gemm_h100.cu:142-148, bench.py:268)."""
    if not b.is_cuda or b.dim() != 2 or not b.is_contiguous() or b.element_size() not in (2, 4):
        raise ValueError("expected a contiguous 2-D CUDA tensor of 2- or 4-byte elements")
    k, n = b.shape
    bt = torch.empty(n, k, device=b.device, dtype=b.dtype)
    check(lib().oxgpu_b200_transpose(b.data_ptr(), bt.data_ptr(), k, n, b.element_size(),
                                     ctypes.c_void_p(_stream(stream))))
    return bt


def f32_to_bf16(x: torch.Tensor, stream=None) -> torch.Tensor:
    """Round-to-nearest-even f32 -> bf16 (run_gemm_h100.cu:26-30)."""
    if not x.is_cuda or x.dtype != torch.float32 or not x.is_contiguous():
        raise ValueError("expected a contiguous f32 CUDA tensor")
    out = torch.empty(x.shape, device=x.device, dtype=torch.bfloat16)
    check(lib().oxgpu_b200_f32_to_bf16(x.data_ptr(), out.data_ptr(), x.numel(),
                                       ctypes.c_void_p(_stream(stream))))
    return out


def transpose_to_bf16(b: torch.Tensor, stream=None) -> torch.Tensor:
    """f32 B[K,N] -> bf16 B^T[N,K] in one pass (K and N multiples of 64)."""
    if not b.is_cuda or b.dim() != 2 or not b.is_contiguous() or b.dtype != torch.float32:
        raise ValueError("expected a contiguous 2-D f32 CUDA tensor")
    k, n = b.shape
    bt = torch.empty(n, k, device=b.device, dtype=torch.bfloat16)
    check(lib().oxgpu_b200_transpose_f32_to_bf16(b.data_ptr(), bt.data_ptr(), k, n,
                                                 ctypes.c_void_p(_stream(stream))))
    return bt


def matmul(a: torch.Tensor, b: torch.Tensor, element: str = "f32", flags: int = 0) -> torch.Tensor:
    """A[M,K] @ B[K,N] the way the reference's bench drives its kernel
    (bench.py:255-271): convert to the input width, re-lay B K-major, launch."""
    if element == "bf16":
        a16 = a if a.dtype == torch.bfloat16 else f32_to_bf16(a.contiguous())
        if b.dtype == torch.float32 and b.shape[0] % 64 == 0 and b.shape[1] % 64 == 0:
            return gemm_bf16(a16, transpose_to_bf16(b.contiguous()), flags=flags)
        b16 = b if b.dtype == torch.bfloat16 else f32_to_bf16(b.contiguous())
        return gemm_bf16(a16, transpose(b16.contiguous()), flags=flags)
    return gemm_tf32(a.contiguous(), transpose(b.contiguous()), flags=flags)


def gemm_bf16_host(a_host: torch.Tensor, bt_host: torch.Tensor, c_host: torch.Tensor, flags: int = 0) -> torch.Tensor:
    """Host-buffer entry point: operands and result in (pinned) host memory."""
    if a_host.is_cuda or bt_host.is_cuda or c_host.is_cuda:
        raise ValueError("host entry point takes CPU tensors")
    m, k = a_host.shape
    n = bt_host.shape[0]
    check(lib().oxgpu_b200_gemm_bf16_host(a_host.data_ptr(), bt_host.data_ptr(), c_host.data_ptr(),
                                          m, n, k, flags))
    return c_host


def gemm_bf16_out16_host(a_host: torch.Tensor, bt_host: torch.Tensor, c_host: torch.Tensor,
                         flags: int = 0) -> torch.Tensor:
    """Host-buffer entry point with bf16 C: half the bytes come back over PCIe."""
    if a_host.is_cuda or bt_host.is_cuda or c_host.is_cuda:
        raise ValueError("host entry point takes CPU tensors")
    if c_host.dtype != torch.bfloat16:
        raise ValueError("C must be a bf16 CPU tensor")
    m, k = a_host.shape
    n = bt_host.shape[0]
    check(lib().oxgpu_b200_gemm_bf16_out16_host(a_host.data_ptr(), bt_host.data_ptr(), c_host.data_ptr(),
                                                m, n, k, flags))
    return c_host


def gemm_tf32_host(a_host: torch.Tensor, bt_host: torch.Tensor, c_host: torch.Tensor, flags: int = 0) -> torch.Tensor:
    if a_host.is_cuda or bt_host.is_cuda or c_host.is_cuda:
        raise ValueError("host entry point takes CPU tensors")
    m, k = a_host.shape
    n = bt_host.shape[0]
    check(lib().oxgpu_b200_gemm_tf32_host(a_host.data_ptr(), bt_host.data_ptr(), c_host.data_ptr(),
                                          m, n, k, flags))
    return c_host


def fill_uniform(t: torch.Tensor, seed: int, offset: int = 0, stream=None) -> torch.Tensor:
    """uniform[-1,1) from the counter-based generator, in place."""
    check(lib().oxgpu_b200_fill_uniform(t.data_ptr(), t.numel(), t.element_size(), seed, offset,
                                        ctypes.c_void_p(_stream(stream))))
    return t


def fill_normal(t: torch.Tensor, seed: int, std: float = 1.0, offset: int = 0, stream=None) -> torch.Tensor:
    """normal(0, std) from the counter-based generator, in place (f32 or bf16)."""
    check(lib().oxgpu_b200_fill_normal(t.data_ptr(), t.numel(), t.element_size(), seed, std, offset,
                                       ctypes.c_void_p(_stream(stream))))
    return t


def device_status() -> list[int]:
    """Synchronise and read the device status block; raises OxgpuError
    (status -7) if a bounded device wait timed out."""
    words = (ctypes.c_uint32 * 8)()
    check(lib().oxgpu_b200_device_status(words))
    return list(words)


def launch_count() -> int:
    return int(lib().oxgpu_b200_launch_count())
