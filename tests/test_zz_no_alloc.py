"""The allocation-free split-K entry point (collected last on purpose).

Some users of the library cannot ask for device memory when they call it: their
memory is carved up in advance by an arena or a fixed budget, or they sit in a
loop where an allocation's device-wide synchronisation is unacceptable.
oxgpu_b200_gemm_bf16_splitk_static keeps the split-K partial tiles in a fixed
32 MiB array inside the library instead.  Here it is called straight through the
C ABI, twice in a row with different problems (the second one finds the first
one's leftovers in the array), and each result must equal the workspace entry
point's -- same kernels, same slice count, so equal to the last bit, which is
also inside the strict tolerance the other tests use against the oracle.
"""
import ctypes

import numpy as np
import pytest
import torch

import oracle
from oxcamlgpu_b200 import gemm
from oxcamlgpu_b200._lib import lib


def _operands(seed, m, n, k):
    rng = np.random.default_rng(seed)
    a_bits = oracle.to_bf16((rng.standard_normal((m, k)) * 0.02).astype(np.float32))
    bt_bits = oracle.to_bf16((rng.standard_normal((n, k)) * 0.02).astype(np.float32))
    dev = lambda bits: torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to("cuda:0")
    return a_bits, bt_bits, dev(a_bits), dev(bt_bits)


@pytest.mark.gpu
def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row(oxlib):
    torch.cuda.set_device(0)
    L = lib()
    for seed, (m, n, k, splits) in enumerate([(128, 8192, 4096, 4), (100, 520, 1000, 3)]):
        a_bits, bt_bits, a, bt = _operands(seed, m, n, k)
        c_static = torch.full((m, n), float("nan"), device="cuda:0")
        st = L.oxgpu_b200_gemm_bf16_splitk_static(a.data_ptr(), bt.data_ptr(), c_static.data_ptr(), m, n,
                                                  k, k, k, n, splits, ctypes.c_void_p(0))
        assert st == 0, L.oxgpu_b200_last_error()
        c_ws = gemm.gemm_bf16(a, bt, flags=gemm.make_flags("splitk", splits=splits))
        torch.cuda.synchronize()
        assert torch.equal(c_static, c_ws)
        expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits, threads=oracle.max_threads())
        tol = oracle.tolerance(k, float(np.abs(oracle.of_bf16(a_bits)).max()),
                               float(np.abs(oracle.of_bf16(bt_bits)).max()))
        assert float(np.abs(c_static.cpu().numpy() - expect).max()) <= tol
    assert gemm.device_status()[0] == 0


@pytest.mark.gpu
def test_static_scratch_entry_refuses_what_does_not_fit(oxlib):
    torch.cuda.set_device(0)
    L = lib()
    m, n, k = 128, 8192, 8192
    _, _, a, bt = _operands(5, m, n, k)
    c = torch.zeros(m, n, device="cuda:0")
    before = gemm.launch_count()
    # 16 slices x 128 x 8192 x 4 bytes = 64 MiB > 32 MiB
    st = L.oxgpu_b200_gemm_bf16_splitk_static(a.data_ptr(), bt.data_ptr(), c.data_ptr(), m, n, k, k, k, n,
                                              16, ctypes.c_void_p(0))
    assert st == -6 and b"built-in scratch holds" in L.oxgpu_b200_last_error()
    assert gemm.launch_count() == before and float(c.abs().max()) == 0.0
    # 8 slices fit exactly
    gemm.gemm_bf16_splitk_static(a, bt, c, splits=8)
    ref = gemm.gemm_bf16(a, bt, flags=gemm.make_flags("splitk", splits=8))
    assert torch.equal(c, ref)
