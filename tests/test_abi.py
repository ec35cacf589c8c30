"""The C-ABI library loads without a GPU, exports every symbol the public
header declares, and rejects contract violations before touching a device."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "oxgpu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"OXGPU_API\s+[^;(]*?\b(oxgpu_b200_\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    assert len(names) >= 30
    for must in ("oxgpu_b200_gemm_tmap", "oxgpu_b200_gemm_bf16", "oxgpu_b200_gemm_tf32",
                 "oxgpu_b200_gemm_exact", "oxgpu_b200_choose_config", "oxgpu_b200_kernel_binding",
                 "oxgpu_b200_kernel_info", "oxgpu_b200_encode_tmap_2d", "oxgpu_b200_gemm_bf16_host"):
        assert must in names


def test_library_exports_every_declared_symbol(oxlib):
    raw = ctypes.CDLL(oxlib._name)
    missing = [n for n in declared_symbols() if not hasattr(raw, n)]
    assert not missing, missing
    # and the Python binding table covers the same surface
    assert sorted(oxlib._oxgpu_signatures) == declared_symbols()


def test_library_has_no_link_time_driver_dependency(oxlib):
    """libcuda is resolved at run time, so the library loads on a CPU-only box."""
    import subprocess
    out = subprocess.run(["readelf", "-d", oxlib._name], capture_output=True, text=True).stdout
    assert "libcuda.so" not in out
    assert b"sm_100a" in oxlib.oxgpu_b200_build_info()


def test_strerror_and_status_codes(oxlib):
    assert oxlib.oxgpu_b200_strerror(0) == b"ok"
    assert b"divisible" in oxlib.oxgpu_b200_strerror(-4)
    assert oxlib.oxgpu_b200_strerror(700) == b"CUDA error"


def test_tmap_entry_contract_checks_need_no_device(oxlib):
    """bench/bench.py:247-250 refuses sizes the tile does not divide; so do we,
    before any CUDA call."""
    f = oxlib.oxgpu_b200_gemm_tmap
    ok_ptr = 0x1000
    assert f(b"gemm_nope", ok_ptr, ok_ptr, ok_ptr, 256, 256, 512, None) == -3
    assert f(b"gemm_fast", 0, ok_ptr, ok_ptr, 256, 256, 512, None) == -1
    assert f(b"gemm_fast", ok_ptr, ok_ptr, ok_ptr, 0, 256, 512, None) == -1
    assert f(b"gemm_fast", ok_ptr + 8, ok_ptr, ok_ptr, 256, 256, 512, None) == -5
    assert f(b"gemm_fast", ok_ptr, ok_ptr, ok_ptr + 4, 256, 256, 512, None) == -5
    assert f(b"gemm_fast", ok_ptr, ok_ptr, ok_ptr, 200, 256, 512, None) == -4       # M % 128
    assert b"must be divisible by CTA 128x256 and BK 32" in oxlib.oxgpu_b200_last_error()
    assert f(b"gemm_fast", ok_ptr, ok_ptr, ok_ptr, 256, 128, 512, None) == -4       # N % 256
    assert f(b"gemm_fast", ok_ptr, ok_ptr, ok_ptr, 256, 256, 500, None) == -4       # K % 32
    assert f(b"gemm_bf16_fast", ok_ptr, ok_ptr, ok_ptr, 256, 256, 96, None) == -4   # K % 64
    assert f(b"gemm_bm64_bn256_s3", ok_ptr, ok_ptr, ok_ptr, 96, 256, 64, None) == -4  # M % bm
    assert f(b"gemm_bm256_bn128_s3", ok_ptr, ok_ptr, ok_ptr, 128, 128, 64, None) == -4


def test_buffer_entry_contract_checks_need_no_device(oxlib):
    g = oxlib.oxgpu_b200_gemm_bf16
    p = 0x10000
    assert g(None, p, p, 128, 128, 64, 64, 64, 128, 0, None) == -1
    assert g(p, p, p, 128, 128, 0, 64, 64, 128, 0, None) == -1
    assert g(p, p, p, 128, 128, 64, 32, 64, 128, 0, None) == -1     # lda < K
    assert g(p + 2, p, p, 128, 128, 64, 64, 64, 128, 0, None) == -5  # misaligned A
    assert g(p, p, p, 128, 128, 64, 68, 64, 128, 0, None) == -5      # lda*2 % 16
    assert g(p, p, p, 128, 126, 64, 64, 64, 126, 0, None) == -5      # ldc*4 % 16
    assert g(p, p, p, 128, 128, 60, 64, 64, 128, 0, None) == -4      # K*2 % 16
    assert g(p, p, p, 128, 128, 64, 64, 64, 128, 6, None) == -1      # split-K without workspace
    t = oxlib.oxgpu_b200_gemm_tf32
    assert t(p, p, p, 128, 128, 30, 32, 32, 128, 0, None) == -4      # K*4 % 16
    e = oxlib.oxgpu_b200_gemm_exact
    assert e(p, p, p, 4, 4, 4, 4, 4, 4, 3, None) == -1
    assert oxlib.oxgpu_b200_transpose(p, p, 4, 4, 3, None) == -1
    assert oxlib.oxgpu_b200_splitk_workspace_bytes(128, 8192, 4) == 4 * 128 * 8192 * 4
    assert oxlib.oxgpu_b200_splitk_workspace_bytes(100, 8, 2) == 2 * 128 * 8 * 4


def test_compute_without_a_device_fails_loudly(oxlib):
    """No CPU fallback: on a machine without a GPU a well-formed call returns a
    CUDA error instead of computing anything."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    p = 0x10000
    st = oxlib.oxgpu_b200_gemm_bf16(p, p, p, 128, 128, 64, 64, 64, 128, 0, None)
    assert st > 0 or st == -8
    assert oxlib.oxgpu_b200_gemm_exact(p, p, p, 4, 4, 4, 4, 4, 4, 0, None) > 0
