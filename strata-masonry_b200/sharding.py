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
