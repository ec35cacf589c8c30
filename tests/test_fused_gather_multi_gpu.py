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


def _departing_worker(rank, world, port, results):
    """Step 1 completes on both ranks; rank 1 then leaves between steps (nothing
    of it in flight, its mappings closed).  Rank 0 learns of it on the host
    before its next launch and launches nothing; its GPU stays usable."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    outcome = "?"
    try:
        from oxcamlgpu_b200 import gemm, sharded
        m, n, k = 512, 1024, 256
        dev = torch.device("cuda", rank)
        a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
        gemm.fill_normal(a, 5, 1.0, 0)
        gemm.fill_normal(bt, 5, 1.0, m * k)
        fused = sharded.FusedGatherGemm(m, n, k)
        shard = sharded.shard_rows_of_bt(bt, rank, world)
        fused.run(a, shard, check_peers_s=10.0)
        c = fused.finish().clone()           # the shared buffer is freed by close()
        step1_ok = bool(torch.equal(c, gemm.gemm_bf16(a, bt)))
        if rank == 1:
            # leave with nothing in flight: unmap the peer's buffer, but do not free this
            # rank's own, which rank 0 may still have mapped (process exit releases it)
            fused.close(barrier=False, free_own=False)
            results.put((rank, step1_ok, "left"))
            results.close()
            results.join_thread()
            os._exit(0)
        launches = gemm.launch_count()
        try:
            fused.run(a, shard, check_peers_s=3.0)
            outcome = "launched"
        except RuntimeError:
            outcome = "refused" if gemm.launch_count() == launches else "launched anyway"
        fused.close(barrier=False)
        still_fine = bool(torch.equal(gemm.gemm_bf16(a, bt), c)) and gemm.device_status()[0] == 0
        results.put((rank, step1_ok and still_fine, outcome))
    except Exception as e:  # noqa: BLE001 - reported to the parent
        results.put((rank, False, repr(e)))
    results.close()
    results.join_thread()
    os._exit(0)


def test_a_departed_rank_is_noticed_before_the_next_launch(oxlib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_departing_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in range(2):
        r, ok, what = results.get(timeout=300)
        got[r] = (ok, what)
    for p in procs:
        p.join(60)
    assert got[1] == (True, "left") and got[0] == (True, "refused"), got
