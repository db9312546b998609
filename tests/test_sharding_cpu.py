"""Column-parallel sharding, world size 2, gloo backend on the CPU: the slabs every rank generates
with *global* fill indices reassemble into the single-process operands bit for bit, and the
rank-major all-gather layout converts back to row-major D.  No GPU involved: the generators are
the library's host entry points."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    smb = entry.load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n, k, fill = 48, 64, 96, 5
        sh = smb.sharding.column_shard(n, world, rank)
        # BT slab with global indices: element (n, k) has index k * N + n.
        bt_local = smb.gemm.fill_bf16_host(sh.n_local, k, fill, 2, sh.n0, 1, n)
        b_local, _, sfb_local = smb.gemm.fill_fp4_host(sh.n_local, k, 5, 1, sh.n0)
        # A stand-in for the GEMM: D slab = function of (global column, row) only.
        d_local = (np.arange(m)[:, None] * 1000 + (np.arange(sh.n_local)[None, :] + sh.n0)).astype(np.int32)
        pieces = {}
        for name, arr in (("bt", bt_local.astype(np.int32)), ("b", b_local.astype(np.int32)),
                          ("sfb", sfb_local.astype(np.int32)), ("d", d_local)):
            t = torch.from_numpy(np.ascontiguousarray(arr))
            gathered = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(gathered, t)
            pieces[name] = np.stack([x.numpy() for x in gathered])
        if rank == 0:
            bt_full = smb.gemm.fill_bf16_host(n, k, fill, 2, 0, 1, n)
            b_full, _, sfb_full = smb.gemm.fill_fp4_host(n, k, 5, 1, 0)
            ok = np.array_equal(pieces["bt"].reshape(n, k), bt_full.astype(np.int32))
            ok &= np.array_equal(pieces["b"].reshape(n, k // 2), b_full.astype(np.int32))
            ok &= np.array_equal(pieces["sfb"].reshape(n, k // 32), sfb_full.astype(np.int32))
            d_full = smb.sharding.gathered_to_row_major(pieces["d"])
            want = (np.arange(m)[:, None] * 1000 + np.arange(n)[None, :]).astype(np.int32)
            ok &= np.array_equal(d_full, want)
            out.put(bool(ok))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_column_sharding_on_gloo(smb):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert out.get(timeout=5) is True


def test_column_shard_rules(smb):
    sh = smb.sharding.column_shard(57344, 8, 3)
    assert (sh.n0, sh.n_local) == (3 * 7168, 7168)
    assert smb.sharding.column_shard(8192, 8, 7).n_local == 1024
    with pytest.raises(ValueError):
        smb.sharding.column_shard(8192, 3, 0)
    with pytest.raises(ValueError):
        smb.sharding.column_shard(36, 4, 0)       # 9 columns per rank: rows of D not 16-byte aligned
    with pytest.raises(ValueError):
        smb.sharding.column_shard(64, 2, 2)
    assert smb.sharding.allgather_bytes_received(32768, 57344, 8) == 7 * 32768 * 7168 * 2
    g = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    rm = smb.sharding.gathered_to_row_major(g)
    assert rm.shape == (3, 8) and list(rm[1]) == [4, 5, 6, 7, 16, 17, 18, 19]
