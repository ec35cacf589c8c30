"""Column-sharded GEMM over several GPUs: one process per GPU.

C[:, n0:n1] = A @ B[:, n0:n1] needs no exchange: with B held K-major as
B^T[N,K], a column block of B is a contiguous row block of B^T.  Rank r owns
rows [n0, n1) of B^T, a replica of A, and produces the [M, n1-n0] shard of C.
The reference has no multi-GPU code; the single-GPU call each rank makes is the
same C-ABI entry point as everywhere else.

A replicated C is optional and comes two ways.  all_gather_c is the plain one:
a separate NCCL all-gather after the GEMM; NCCL gathers contiguous chunks, so
the gathered buffer is block-column-major [world][M][N/world] and
blocks_to_row_major re-interleaves it into C[M,N] when a row-major replica is
wanted.  FusedGatherGemm is the fused one: every rank holds a full row-major
C[M,N] that the other ranks have mapped, and each rank's GEMM kernel stores
its tiles into all replicas as they are produced (fan-out epilogue), so the
transfer over NVLink overlaps the main loop and no re-interleave pass exists.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

COLUMN_ALIGN = 256  # shard widths are multiples of the widest tile


def column_partition(n: int, world: int, align: int = COLUMN_ALIGN) -> list[tuple[int, int]]:
    """Contiguous column ranges [n0, n1) per rank: widths are multiples of
    `align` except possibly the last non-empty one (the ragged tail), and block
    counts differ by at most one.  The rule lives in the C library
    (oxgpu_b200_mg_column_partition), shared with the one-process driver."""
    from .multi_gpu import column_partition as c_partition
    return c_partition(n, world, align)


def shard_rows_of_bt(bt_full: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank's rows of B^T[N,K] (= its columns of B); a view, no copy."""
    n0, n1 = column_partition(bt_full.shape[0], world)[rank]
    return bt_full[n0:n1]


def all_gather_c(c_shard: torch.Tensor, group=None) -> torch.Tensor:
    """Gather equal-width shards [M, N/world] into [world, M, N/world].  Works on
    any backend (NCCL on GPUs, gloo on CPU tensors)."""
    world = dist.get_world_size(group)
    c_shard = c_shard.contiguous()
    m, w = c_shard.shape
    out = torch.empty((world * m, w), dtype=c_shard.dtype, device=c_shard.device)
    dist.all_gather_into_tensor(out, c_shard, group=group)  # concatenation along dim 0
    return out.view(world, m, w)


def blocks_to_row_major(gathered: torch.Tensor) -> torch.Tensor:
    """[world, M, W] block-column-major -> row-major C[M, world*W]."""
    world, m, w = gathered.shape
    return gathered.permute(1, 0, 2).reshape(m, world * w).contiguous()


def fanout_destinations(bases: list[int], n0: int, element_bytes: int = 4) -> list[int]:
    """Device addresses the fan-out GEMM of the rank owning columns [n0, ...)
    writes to: the first element of its column window in every rank's row-major
    C (`bases[i]` = address of rank i's C in this process)."""
    if n0 < 0 or (n0 * element_bytes) % 16:
        raise ValueError("a column window must start on a 16-byte boundary")
    return [b + n0 * element_bytes for b in bases]


def host_group(group=None):
    """A gloo group over the same ranks as `group`, for waits that must stay on
    the host.  `group` itself when it already is gloo; otherwise a new gloo group
    (a collective call: every rank of `group` must make it, in the same order)."""
    if dist.get_backend(group) == "gloo":
        return group
    ranks = dist.get_process_group_ranks(group if group is not None else dist.group.WORLD)
    return dist.new_group(ranks=ranks, backend="gloo")


def peers_alive(group=None, timeout_s: float = 5.0) -> bool:
    """Host-side liveness check before a launch that writes into other ranks'
    memory: True if every rank of the group reached this call within the
    time-out.  A rank that has left (between steps, nothing in flight) shows up
    here as False on the others instead of as stores into memory nobody owns.

    `group` must be a gloo group (see host_group): the check is a monitored
    barrier on the host with its own time-out and puts no work on any GPU.  A
    barrier on an NCCL group would enqueue a kernel that waits on the device for
    the absent rank, so any other backend is refused."""
    import datetime
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return True
    if dist.get_backend(group) != "gloo":
        raise ValueError("peers_alive needs a gloo group (sharded.host_group makes one); "
                         "a barrier on another backend would wait on the device")
    try:
        dist.monitored_barrier(group=group, timeout=datetime.timedelta(seconds=timeout_s))
        return True
    except Exception:                        # noqa: BLE001 - any transport or time-out error means "not all here"
        return False


class ColumnShardedGemm:
    """bf16 GEMM with B and C column-sharded across the ranks of a process
    group and A replicated.  Each rank launches the single-GPU kernel on its
    shard; nothing crosses NVLink unless gather() is called."""

    def __init__(self, m: int, n: int, k: int, group=None, flags: int = 0):
        from . import gemm  # needs the CUDA library
        self._gemm = gemm
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.m, self.n, self.k = m, n, k
        self.flags = flags
        self.n0, self.n1 = column_partition(n, self.world)[self.rank]
        self.width = self.n1 - self.n0

    def run(self, a: torch.Tensor, bt_shard: torch.Tensor, c_shard: torch.Tensor | None = None) -> torch.Tensor:
        if tuple(bt_shard.shape) != (self.width, self.k) or tuple(a.shape) != (self.m, self.k):
            raise ValueError("operand shapes do not match this rank's shard")
        return self._gemm.gemm_bf16(a, bt_shard, c_shard, flags=self.flags)

    def gather(self, c_shard: torch.Tensor, row_major: bool = False) -> torch.Tensor:
        widths = {hi - lo for lo, hi in column_partition(self.n, self.world)}
        if len(widths) != 1:
            raise ValueError("all_gather needs equal shard widths")
        g = all_gather_c(c_shard, self.group)
        return blocks_to_row_major(g) if row_major else g


class FusedGatherGemm:
    """Column-sharded GEMM whose result is replicated on every rank by the GEMM
    kernel itself: rank r computes C[:, n0:n1] and its epilogue writes each tile
    to column window [n0, n1) of every rank's row-major C[M,N] (its own by local
    stores, the others' over NVLink by plain TMA tile stores into memory mapped
    from the owning process).  No collective runs on the data path; the only
    exchange is of 64-byte memory handles at construction (any backend).

    run() launches and returns immediately; finish() waits for this rank's
    kernel and then for every other rank's (a host barrier), after which
    self.c holds the complete product on every rank."""

    def __init__(self, m: int, n: int, k: int, group=None, flags: int = 0, device=None):
        from . import gemm
        self._gemm = gemm
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > 8:
            raise ValueError("at most 8 destinations per kernel")
        self.m, self.n, self.k, self.flags = m, n, k, flags
        # liveness checks and the completion barrier stay on the host
        self.host_group = host_group(group) if self.world > 1 else None
        self.parts = column_partition(n, self.world)
        self.n0, self.n1 = self.parts[self.rank]
        self.width = self.n1 - self.n0
        if n % 4:
            raise ValueError("N must be a multiple of 4 (16-byte aligned column windows)")
        self._buf = gemm.SharedBuffer(m * n * 4, device)
        self.c = self._buf.tensor((m, n))
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, self._buf.handle, group=group)
        self._opened = []
        self._dest_base = []
        for r in range(self.world):
            if r == self.rank:
                self._dest_base.append(self._buf.ptr)
            else:
                ptr = gemm.shared_open(handles[r])
                self._opened.append(ptr)
                self._dest_base.append(ptr)

    def run(self, a: torch.Tensor, bt_shard: torch.Tensor, check_peers_s: float | None = None) -> None:
        """Launch this rank's GEMM.  With check_peers_s, first make sure on the
        host that every rank is still there (peers_alive) and raise RuntimeError
        without launching if not."""
        if tuple(bt_shard.shape) != (self.width, self.k) or tuple(a.shape) != (self.m, self.k):
            raise ValueError("operand shapes do not match this rank's shard")
        if check_peers_s is not None and not peers_alive(self.host_group, check_peers_s):
            raise RuntimeError("a rank of the group did not answer: nothing was launched")
        if self.width == 0:
            return
        dests = fanout_destinations(self._dest_base, self.n0)
        self._gemm.gemm_fanout(a, bt_shard, dests, ldc=self.n, flags=self.flags)

    def finish(self) -> torch.Tensor:
        torch.cuda.current_stream().synchronize()
        if self.world > 1:
            dist.barrier(group=self.host_group)
        return self.c

    def close(self, barrier: bool = True, free_own: bool = True) -> None:
        """Unmap the peers' buffers, then (after a barrier, unless a rank is
        known to be gone) free this rank's.  free_own=False leaves this rank's
        buffer allocated: a rank that departs while others may still have it
        mapped must not free it (process exit releases it)."""
        for ptr in self._opened:
            self._gemm.shared_close(ptr)
        self._opened = []
        if self.world > 1 and barrier:
            dist.barrier(group=self.host_group)
        self.c = None
        if free_own:
            self._buf.free()

    def __del__(self):
        # a dropped instance must not leak its mappings of the peers' memory
        try:
            for ptr in getattr(self, "_opened", []):
                self._gemm.shared_close(ptr)
            self._opened = []
        except Exception:                    # noqa: BLE001 - interpreter shutdown
            pass
