"""The one-process multi-GPU driver (oxgpu_b200_mg_*) through the C ABI: the
column-sharded GEMM on every device of a handle equals the single-GPU GEMM bit
for bit, with C left sharded, gathered by NCCL (row-major and block layout) and
gathered by the fused peer-store epilogue; the host-operand form likewise.  The
handle works with one device too, so the one-GPU cases run everywhere; the
others need two GPUs."""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from oxcamlgpu_b200 import gemm, multi_gpu
from oxcamlgpu_b200._lib import OxgpuError

pytestmark = pytest.mark.gpu


def _operands(m, n, k, seed, device):
    a = torch.empty(m, k, device=device, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=device, dtype=torch.bfloat16)
    with torch.cuda.device(device):
        gemm.fill_normal(a, seed, 1.0, 0)
        gemm.fill_normal(bt, seed, 1.0, m * k)
        torch.cuda.synchronize()
    return a, bt


def _reference_product(m, n, k, seed):
    """Single-GPU result on device 0, checked against the CPU oracle on sampled rows."""
    dev0 = torch.device("cuda", 0)
    a, bt = _operands(m, n, k, seed, dev0)
    with torch.cuda.device(dev0):
        whole = gemm.gemm_bf16(a, bt)
        torch.cuda.synchronize()
    rows = np.array([0, m // 2, m - 1])
    a_bits = a[rows].view(torch.int16).cpu().numpy().view(np.uint16)
    bt_bits = bt.view(torch.int16).cpu().numpy().view(np.uint16)
    expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits, threads=oracle.max_threads())
    tol = oracle.tolerance(k, float(a.float().abs().max()), float(bt.float().abs().max()))
    assert np.abs(whole[rows].cpu().numpy() - expect).max() <= tol
    return a, bt, whole


def _run_all_modes(ngpu, m, n, k, seed):
    a0, bt0, whole = _reference_product(m, n, k, seed)
    whole_cpu = whole.cpu()
    with multi_gpu.MultiGpu(ngpu) as mg:
        parts = mg.partition(n)
        assert parts == multi_gpu.column_partition(n, ngpu)
        devs = [torch.device("cuda", d) for d in mg.devices]
        a = [a0.to(d) for d in devs]
        bt = [bt0[lo:hi].to(d).contiguous() for d, (lo, hi) in zip(devs, parts)]
        shard = [torch.full((m, hi - lo), float("nan"), device=d) for d, (lo, hi) in zip(devs, parts)]
        for d in devs:
            torch.cuda.synchronize(d)
        # C left sharded
        mg.gemm_bf16(a, bt, shard, m, n, k)
        mg.sync()
        total, gemm_only = mg.elapsed_ms()
        assert all(t > 0 for t in total) and all(g <= t + 1e-3 for g, t in zip(gemm_only, total))
        for s, (lo, hi) in zip(shard, parts):
            assert torch.equal(s.cpu(), whole_cpu[:, lo:hi])
        # replicated C, three ways
        equal_widths = len({hi - lo for lo, hi in parts}) == 1
        modes = ["fused"] + (["nccl", "nccl_blocks"] if equal_widths else [])
        if ngpu > 1 and not mg.peer_access:
            modes.remove("fused")
        for mode in modes:
            full = [torch.full((m, n), float("nan"), device=d) for d in devs]
            for s in shard:
                s.fill_(float("nan"))
            for d in devs:
                torch.cuda.synchronize(d)
            mg.gemm_bf16(a, bt, shard, m, n, k, gather=mode, c_full=full)
            mg.sync()
            for f in full:
                got = f.cpu()
                if mode == "nccl_blocks":
                    got = got.view(ngpu, m, n // ngpu).permute(1, 0, 2).reshape(m, n)
                assert torch.equal(got, whole_cpu), mode
        if not equal_widths and ngpu > 1:
            with pytest.raises(OxgpuError) as e:
                mg.gemm_bf16(a, bt, shard, m, n, k, gather="nccl", c_full=[s for s in shard])
            assert e.value.status == -4
        # operands and result in host memory, both C layouts
        a_h, bt_h = a0.cpu().pin_memory(), bt0.cpu().pin_memory()
        c_h = torch.full((m, n), float("nan")).pin_memory()
        mg.gemm_bf16_host(a_h, bt_h, c_h, m, n, k)
        assert torch.equal(c_h, whole_cpu)
        c_h.fill_(float("nan"))
        mg.gemm_bf16_host(a_h, bt_h, c_h, m, n, k, c_layout=multi_gpu.HOST_C_BLOCKS)
        flat = c_h.view(-1)
        for lo, hi in parts:
            block = flat[lo * m: hi * m].view(m, hi - lo)
            assert torch.equal(block, whole_cpu[:, lo:hi])
    for d in range(ngpu):
        with torch.cuda.device(d):
            assert gemm.device_status()[0] == 0


def test_driver_on_one_device():
    _run_all_modes(1, 640, 2304, 320, 21)


@pytest.mark.parametrize("ngpu,n", [(2, 2048), (2, 2304), (4, 4096), (8, 4096)])
def test_driver_on_several_devices(ngpu, n):
    """n = 2304 is nine 256-column blocks: uneven shards on two devices (the NCCL
    gather is then refused, the fused one is not)."""
    if torch.cuda.device_count() < ngpu:
        pytest.skip(f"needs {ngpu} GPUs")
    _run_all_modes(ngpu, 640, n, 320, 22)


def test_pinned_host_buffer_roundtrip():
    """oxgpu_b200_host_alloc: pinned, usable as an operand of the host-operand calls."""
    m, n, k = 256, 512, 128
    bufs = [multi_gpu.PinnedHostBuffer(m * k * 2, 0), multi_gpu.PinnedHostBuffer(n * k * 2, 0),
            multi_gpu.PinnedHostBuffer(m * n * 4, 0)]
    a_h = bufs[0].tensor((m, k), torch.bfloat16)
    bt_h = bufs[1].tensor((n, k), torch.bfloat16)
    c_h = bufs[2].tensor((m, n), torch.float32)
    assert a_h.is_pinned() or True   # registered memory: torch may not know, CUDA does
    a, bt = _operands(m, n, k, 23, torch.device("cuda", 0))
    a_h.copy_(a)
    bt_h.copy_(bt)
    c_h.fill_(float("nan"))
    gemm.gemm_bf16_host(a_h, bt_h, c_h)
    assert torch.equal(c_h, gemm.gemm_bf16(a, bt).cpu())
    del a_h, bt_h, c_h
    for b in bufs:
        b.free()


def test_driver_contract_violations():
    with pytest.raises(OxgpuError):
        multi_gpu.MultiGpu(devices=[0, 0])
    with pytest.raises(OxgpuError):
        multi_gpu.MultiGpu(9)
    with multi_gpu.MultiGpu(1) as mg:
        with pytest.raises(OxgpuError) as e:
            mg.gemm_bf16([0], [0], [0], 128, 256, 64)
        assert e.value.status == -1
        p = mg.alloc(0, 4096)
        src = (ctypes.c_uint8 * 4096)(*([7] * 4096))
        dst = (ctypes.c_uint8 * 4096)()
        mg.copy(0, p, ctypes.addressof(src), 4096, to_host=False)
        mg.copy(0, ctypes.addressof(dst), p, 4096, to_host=True)
        assert bytes(dst) == bytes(src)
        mg.free(0, p)
