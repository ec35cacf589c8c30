"""Host-side logic of the column-sharded multi-GPU driver, on CPU: partitioning,
and a world_size-2 gloo run in which each rank computes its shard with the
oracle, the shards are all-gathered and re-interleaved, and the result equals
the unsharded oracle bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oxcamlgpu_b200 import sharded

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("n,world", [(65536, 1), (65536, 2), (65536, 4), (65536, 8), (8192, 8), (2048, 8),
                                     (1000, 3), (256, 4), (28672, 8)])
def test_column_partition(n, world):
    parts = sharded.column_partition(n, world)
    assert len(parts) == world and parts[0][0] == 0 and parts[-1][1] == n
    covered = 0
    for lo, hi in parts:
        assert lo == covered and hi >= lo
        assert lo % 256 == 0
        covered = hi
    assert covered == n
    widths = [hi - lo for lo, hi in parts]
    # at most one aligned block apart (the ragged tail may shorten the last one further)
    assert max(widths) - min(widths) < 2 * 256
    if n % (256 * world) == 0:
        assert len(set(widths)) == 1 and widths[0] == n // world


def _partition_rule(n, world, align=256):
    """The rule stated in the header, restated here: whole `align`-column blocks,
    counts differing by at most one, the first ranges take the extra blocks."""
    blocks = (n + align - 1) // align
    base, extra = divmod(blocks, world)
    out, start = [], 0
    for r in range(world):
        w = base + (1 if r < extra else 0)
        out.append((min(start * align, n), min((start + w) * align, n)))
        start += w
    return out


@pytest.mark.parametrize("n,world,align", [(65536, 8, 256), (65536, 7, 256), (1000, 3, 256), (100, 8, 256),
                                           (28672, 8, 256), (4096, 3, 128), (2 ** 31 - 1, 8, 256), (5, 5, 1)])
def test_c_partition_function(oxlib, n, world, align):
    """oxgpu_b200_mg_column_partition is what both the one-process driver and the
    one-process-per-GPU wrapper use."""
    import ctypes
    lo, hi = (ctypes.c_int * world)(), (ctypes.c_int * world)()
    assert oxlib.oxgpu_b200_mg_column_partition(n, world, align, lo, hi) == 0
    assert [(lo[i], hi[i]) for i in range(world)] == _partition_rule(n, world, align)
    assert oxlib.oxgpu_b200_mg_column_partition(0, world, align, lo, hi) == -1
    assert oxlib.oxgpu_b200_mg_column_partition(n, world, align, None, hi) == -1


def test_peers_alive_refuses_a_group_that_would_wait_on_the_device(monkeypatch):
    """The liveness check must stay on the host: with any backend but gloo it
    raises instead of issuing a barrier that would run as a kernel."""
    monkeypatch.setattr(dist, "is_initialized", lambda: True)
    monkeypatch.setattr(dist, "get_world_size", lambda group=None: 2)
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "nccl")
    called = []
    monkeypatch.setattr(dist, "barrier", lambda *a, **k: called.append("barrier"))
    monkeypatch.setattr(dist, "monitored_barrier", lambda *a, **k: called.append("monitored"))
    with pytest.raises(ValueError, match="gloo"):
        sharded.peers_alive(timeout_s=1.0)
    assert called == []
    # and a non-gloo default group gets a gloo side group over the same ranks
    made = {}
    monkeypatch.setattr(dist, "get_process_group_ranks", lambda g: [0, 1])
    monkeypatch.setattr(dist, "new_group", lambda ranks, backend: made.update(ranks=ranks, backend=backend) or "side")
    assert sharded.host_group(None) == "side" and made == {"ranks": [0, 1], "backend": "gloo"}
    monkeypatch.setattr(dist, "get_backend", lambda group=None: "gloo")
    assert sharded.host_group("g") == "g"


def test_partition_rejects_nonsense():
    with pytest.raises(ValueError):
        sharded.column_partition(0, 2)
    with pytest.raises(ValueError):
        sharded.column_partition(10, 0)


def test_blocks_to_row_major():
    g = torch.arange(2 * 3 * 4).reshape(2, 3, 4)
    c = sharded.blocks_to_row_major(g)
    assert c.shape == (3, 8)
    assert torch.equal(c[:, :4], g[0]) and torch.equal(c[:, 4:], g[1])


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, failures):
    try:
        sys.path.insert(0, ROOT)
        import oracle
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        m, n, k = 48, 512, 96
        rng = np.random.default_rng(0)                       # same operands on every rank
        a_bits = oracle.to_bf16(rng.standard_normal((m, k)).astype(np.float32))
        bt_bits = oracle.to_bf16(rng.standard_normal((n, k)).astype(np.float32))
        bt_shard = sharded.shard_rows_of_bt(torch.from_numpy(bt_bits.view(np.int16)), rank, world)
        n0, n1 = sharded.column_partition(n, world)[rank]
        assert bt_shard.shape[0] == n1 - n0 == n // world
        c_shard = oracle.gemm_kmajor_bf16(a_bits, bt_shard.numpy().view(np.uint16))
        gathered = sharded.all_gather_c(torch.from_numpy(c_shard))
        assert gathered.shape == (world, m, n // world)
        full = sharded.blocks_to_row_major(gathered).numpy()
        expect = oracle.gemm_kmajor_bf16(a_bits, bt_bits)
        assert np.array_equal(full.view(np.uint32), expect.view(np.uint32))
        # max-over-ranks timing reduction used by the bench
        t = torch.tensor([1.0 + rank])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert float(t) == float(world)
        dist.barrier()
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover - reported through the queue
        failures.put(f"rank {rank}: {e!r}")
        raise


def test_two_ranks_gloo_shard_gather_reassemble():
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, failures)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    assert not msgs, msgs
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


def _failing_worker(rank, world, port, results):
    """Rank 1 fails on the host before the exchange step; rank 0 must get an error
    from the gather (short process-group timeout), not hang."""
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    dist.barrier()
    if rank == 1:
        results.put((rank, "failed before the gather"))
        results.close()
        results.join_thread()
        os._exit(3)                      # the rank is gone: no kernels, no collectives in flight
    try:
        sharded.all_gather_c(torch.ones(4, 8))
        results.put((rank, "gather returned"))
    except Exception as e:               # noqa: BLE001 - any transport / timeout error is the expected outcome
        results.put((rank, "error: " + type(e).__name__))
    results.close()
    results.join_thread()
    os._exit(0)


def test_rank_failure_surfaces_as_an_error_not_a_hang():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert all(not p.is_alive() for p in procs), "a rank hung"
    got = {}
    while not results.empty():
        r, msg = results.get()
        got[r] = msg
    assert got.get(1) == "failed before the gather" and procs[1].exitcode == 3
    assert got.get(0, "").startswith("error: ") and procs[0].exitcode == 0


def _liveness_worker(rank, world, port, results):
    import datetime
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    side = sharded.host_group(None)                     # gloo default group: used as it is
    assert side is None
    first = sharded.peers_alive(side, timeout_s=5.0)    # everybody is here
    if rank == 1:
        results.put((rank, first, None))
        results.close()
        results.join_thread()
        os._exit(0)                                     # leaves between steps
    second = sharded.peers_alive(side, timeout_s=2.0)   # rank 1 is gone
    results.put((rank, first, second))
    results.close()
    results.join_thread()
    os._exit(0)


def test_peers_alive_reports_a_departed_rank():
    ctx = mp.get_context("spawn")
    results = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_liveness_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert all(not p.is_alive() for p in procs), "a rank hung"
    got = {}
    while not results.empty():
        r, first, second = results.get()
        got[r] = (first, second)
    assert got[1][0] is True and got[0] == (True, False), got


def test_fanout_destination_windows():
    bases = [0x7000_0000_0000, 0x7100_0000_0000, 0x7200_0000_0000]
    n = 2304
    for rank, (n0, n1) in enumerate(sharded.column_partition(n, 3)):
        d = sharded.fanout_destinations(bases, n0)
        assert d == [b + 4 * n0 for b in bases] and all(x % 16 == 0 for x in d)
    with pytest.raises(ValueError):
        sharded.fanout_destinations(bases, 3)       # 12 bytes into a row: not 16-byte aligned
