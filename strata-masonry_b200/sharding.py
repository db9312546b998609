"""Column-parallel (N) sharding of the GEMM path across the GPUs of one box.

Rank r of g computes D[:, r*N/g : (r+1)*N/g] from all of A and rows [r*N/g, (r+1)*N/g) of
BT (and of the B scales).  There is no exchange inside the kernel; the optional collective is an
all-gather of the [M, N/g] slabs, which NCCL concatenates rank-major as [g, M, N/g].
The reference has no multi-GPU code; the operand index rules that make the union of the slabs
equal to the single-GPU result are those of its drivers (dense_gemm_bf16.cu:298-304: B index
k*N + n with the global n and the global N).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class ColumnShard:
    rank: int
    world: int
    n_total: int
    n0: int        # first global column of this rank
    n_local: int   # number of columns of this rank


def column_shard(n_total: int, world: int, rank: int, align: int = 8) -> ColumnShard:
    """Equal split of N; every slab must keep 16-byte-aligned bf16 rows (N/g % 8 == 0)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if n_total % world != 0:
        raise ValueError(f"N={n_total} is not divisible by {world} ranks")
    n_local = n_total // world
    if n_local % align != 0:
        raise ValueError(f"N/g={n_local} must be a multiple of {align} (16-byte rows of D)")
    return ColumnShard(rank, world, n_total, rank * n_local, n_local)


def gathered_to_row_major(gathered: np.ndarray) -> np.ndarray:
    """[g, M, N/g] (what an all-gather of the slabs yields) -> [M, N] row-major."""
    g, m, nl = gathered.shape
    return np.ascontiguousarray(np.transpose(gathered, (1, 0, 2))).reshape(m, g * nl)


def allgather_bytes_received(m: int, n_total: int, world: int, elem_bytes: int = 2) -> int:
    """Bytes every GPU receives in the all-gather of D."""
    return (world - 1) * m * (n_total // world) * elem_bytes


# ------------------------------------------------------------------ fused all-gather plumbing
def peer_copy_order(rank: int, world: int) -> list[int]:
    """Other ranks in the order a rank writes to them: r+1, r+2, ... (mod g), so that at any
    moment the g ranks target g different GPUs."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    return [(rank + i) % world for i in range(1, world)]


def peer_copy_targets(bases: list[int], shard: ColumnShard, elem_bytes: int = 2) -> list[int]:
    """Address of element (0, n0) of this rank's slab inside the full row-major D of every other
    rank (`bases[r]` = address of rank r's D as mapped into this process)."""
    if len(bases) != shard.world:
        raise ValueError("one base address per rank")
    return [bases[r] + shard.n0 * elem_bytes for r in peer_copy_order(shard.rank, shard.world)]


class _CudaPeerMemory:
    """Exportable device memory through the library's C entry points."""

    def __init__(self):
        import ctypes as C

        from . import capi
        self._C, self._capi, self._lib = C, capi, capi.lib()

    def alloc(self, nbytes: int) -> int:
        p = self._C.c_void_p()
        self._capi.check(self._lib.smb_peer_alloc(self._C.byref(p), nbytes))
        return int(p.value)

    def export(self, ptr: int) -> bytes:
        buf = self._C.create_string_buffer(self._capi.PEER_HANDLE_BYTES)
        self._capi.check(self._lib.smb_peer_export(ptr, buf))
        return buf.raw

    def open(self, handle: bytes) -> int:
        p = self._C.c_void_p()
        self._capi.check(self._lib.smb_peer_open(handle, self._C.byref(p)))
        return int(p.value)

    def close(self, ptr: int) -> None:
        self._capi.check(self._lib.smb_peer_close(ptr))

    def synchronize(self) -> None:
        """Wait for all work of this process on the current device (kernels whose epilogues may
        still be storing into peers' buffers)."""
        self._capi.check(self._lib.smb_device_synchronize())

    def free(self, ptr: int) -> None:
        self._capi.check(self._lib.smb_peer_free(ptr))


def _close_shared(dist, mem, bases, rank, local) -> None:
    """Tear-down order of peer-mapped buffers.  A kernel of this rank may still be storing into the
    other ranks' buffers (its epilogue writes them with plain stores), and the host barrier below
    says nothing about the device: so every rank first drains its own device, then all meet (now
    nobody writes into anybody's buffer), unmap, meet again (nobody still has a mapping), free."""
    mem.synchronize()
    dist.barrier()
    for r, base in enumerate(bases):
        if r != rank:
            mem.close(base)
    dist.barrier()
    mem.free(local)


class SharedOutput:
    """A full row-major D [M, N] on every GPU of the box, each one mapped into every process, so
    that the GEMM epilogue of rank r can write its column slab into all g copies.

    `dist` is `torch.distributed` (initialised; any backend: only objects are exchanged here).
    `memory` is an object with alloc/export/open/close/free (default: CUDA IPC through the
    library); tests on CPU pass a fake."""

    def __init__(self, m: int, n_total: int, dist, memory=None, elem_bytes: int = 2):
        self.m, self.n_total, self.elem_bytes = m, n_total, elem_bytes
        self._dist = dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        if self.world - 1 > 7:
            raise ValueError("at most 8 ranks (7 peer copies per stored box)")
        self._mem = memory if memory is not None else _CudaPeerMemory()
        self.nbytes = m * n_total * elem_bytes
        self.local = self._mem.alloc(self.nbytes)
        handles: list = [None] * self.world
        dist.all_gather_object(handles, self._mem.export(self.local))
        self.bases = [self.local if r == self.rank else self._mem.open(handles[r])
                      for r in range(self.world)]
        self._open = True

    def shard(self) -> ColumnShard:
        return column_shard(self.n_total, self.world, self.rank)

    def slab_address(self) -> int:
        """Where this rank's GEMM writes its own slab: element (0, n0) of the local D."""
        return self.local + self.shard().n0 * self.elem_bytes

    def peer_targets(self) -> list[int]:
        return peer_copy_targets(self.bases, self.shard(), self.elem_bytes)

    def local_tensor(self):
        """The local D as a torch uint16-sized view ([M, N] of bfloat16)."""
        import torch

        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (self.nbytes,), "typestr": "|u1",
                                        "data": (self.local, False), "version": 2}
        flat = torch.as_tensor(raw, device=torch.device("cuda", torch.cuda.current_device()))
        return flat.view(torch.bfloat16).view(self.m, self.n_total)

    def close(self) -> None:
        """Collective: device synchronize, barrier, unmap, barrier, free (see _close_shared)."""
        if not self._open:
            return
        self._open = False
        _close_shared(self._dist, self._mem, self.bases, self.rank, self.local)


# ------------------------------------------------------------------ fused reduce-scatter plumbing
def route_targets(bases: list[int], rank: int, slot_bytes: int) -> list[int]:
    """Where rank `rank` delivers row block b of its partial product: slot `rank` of rank b's
    receive buffer (`bases[b]` = that buffer as mapped into this process)."""
    return [base + rank * slot_bytes for base in bases]


class ScatterSlots:
    """Receive side of the fused reduce-scatter of a K-sharded GEMM: on every rank a buffer of g
    slots [M/g, N] bf16, slot s filled by rank s with the row block this rank owns of rank s's
    partial product; all buffers mapped into every process.  `dist` and `memory` as for
    SharedOutput."""

    def __init__(self, m: int, n: int, dist, memory=None, elem_bytes: int = 2):
        self._dist = dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        if self.world > 8:
            raise ValueError("at most 8 ranks (8 routed row blocks)")
        if m % self.world != 0 or (m // self.world) % 256 != 0:
            raise ValueError(f"M/g = {m}/{self.world} must be a multiple of 256 rows")
        self.m, self.n, self.elem_bytes = m, n, elem_bytes
        self.rows_per_block = m // self.world
        self.slot_bytes = self.rows_per_block * n * elem_bytes
        self._mem = memory if memory is not None else _CudaPeerMemory()
        self.local = self._mem.alloc(self.world * self.slot_bytes)
        handles: list = [None] * self.world
        dist.all_gather_object(handles, self._mem.export(self.local))
        self.bases = [self.local if r == self.rank else self._mem.open(handles[r]) for r in range(self.world)]
        self._open = True

    def targets(self) -> list[int]:
        return route_targets(self.bases, self.rank, self.slot_bytes)

    def first_block(self) -> int:
        """Row block at which this rank's kernel should start its tile walk: a different one on
        every rank, so that the ranks do not all deliver to the same owner at the same time."""
        return (self.rank + 1) % self.world

    def close(self) -> None:
        if not self._open:
            return
        self._open = False
        _close_shared(self._dist, self._mem, self.bases, self.rank, self.local)
