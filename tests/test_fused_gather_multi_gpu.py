"""The fused GEMM + all-gather across real GPUs: one process per GPU, every
rank's kernel stores its tiles into all ranks' row-major C over NVLink.  Needs
at least two GPUs; skipped otherwise.  (The same kernel with all destinations
on one GPU is covered by test_gemm_gpu.py.)"""
import datetime
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, results):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=120))
    ok, detail = False, ""
    try:
        from oxcamlgpu_b200 import gemm, sharded
        m, n, k = 1024, 4096, 512
        dev = torch.device("cuda", rank)
        a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
        gemm.fill_normal(a, 21, 1.0, 0)          # counter-based: identical on every rank
        gemm.fill_normal(bt, 21, 1.0, m * k)
        fused = sharded.FusedGatherGemm(m, n, k)
        fused.c.fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(2):                         # twice: the second run overwrites in place
            fused.run(a, sharded.shard_rows_of_bt(bt, rank, world))
            c = fused.finish()
        whole = gemm.gemm_bf16(a, bt)
        exact = gemm.gemm_exact(a, bt, gemm.INPUT_BF16)
        tol = 1e-5 * (k ** 0.5) * float(a.float().abs().max()) * float(bt.float().abs().max())
        err = float((c - exact).abs().max())
        ok = bool(torch.equal(c, whole)) and err <= tol and gemm.device_status()[0] == 0
        detail = f"err {err:.3e} tol {tol:.3e} equal {bool(torch.equal(c, whole))}"
        dist.barrier()
        fused.close()
    except Exception as e:  # noqa: BLE001 - reported to the parent
        detail = repr(e)
    results.put((rank, ok, detail))
    results.close()
    results.join_thread()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_gather_matches_the_unsharded_gemm(world, oxlib):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    got = [results.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(60)
    assert all(ok for _, ok, _ in got), got
