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


# ------------------------------------------------------------------ fused all-gather plumbing
class _FileBackedMemory:
    """Stand-in for peer-mappable device memory: every rank's "allocation" is a region of one
    shared file, an address is an offset into it (plus a base, so that 0 is never valid)."""
    BASE = 1 << 20

    def __init__(self, path, rank, region_bytes):
        self.path, self.rank, self.region = path, rank, region_bytes
        self.opened, self.closed, self.freed = [], [], []

    def alloc(self, nbytes):
        assert nbytes <= self.region
        return self.BASE + self.rank * self.region

    def export(self, ptr):
        return int(ptr).to_bytes(8, "little") + bytes(56)

    def open(self, handle):
        assert len(handle) == 64
        addr = int.from_bytes(handle[:8], "little")
        self.opened.append(addr)
        return addr

    def close(self, ptr):
        self.closed.append(ptr)

    def free(self, ptr):
        self.freed.append(ptr)

    def synchronize(self):
        self.synced = getattr(self, "synced", 0) + 1


def _fused_worker(rank, world, port, path, out):
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    smb = entry.load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n = 12, 8 * world * 3
        region = m * n * 2
        mem = _FileBackedMemory(path, rank, region)
        shared = smb.sharding.SharedOutput(m, n, dist, memory=mem)
        sh = shared.shard()
        backing = np.memmap(path, dtype=np.uint8, mode="r+", shape=(world * region,))
        # What the epilogue does: the slab goes to the local D and, with the same row pitch, to
        # every peer target.
        slab = (np.arange(m)[:, None] * 1000 + sh.n0 + np.arange(sh.n_local)[None, :]).astype(np.uint16)
        targets = [shared.slab_address()] + shared.peer_targets()
        assert len(targets) == world and len(set(targets)) == world
        for addr in targets:
            off = addr - mem.BASE
            for row in range(m):
                start = off + row * n * 2
                backing[start:start + sh.n_local * 2] = slab[row].view(np.uint8)
        backing.flush()
        dist.barrier()
        mine = np.memmap(path, dtype=np.uint16, mode="r", offset=rank * region, shape=(m, n))
        want = (np.arange(m)[:, None] * 1000 + np.arange(n)[None, :]).astype(np.uint16)
        ok = np.array_equal(np.asarray(mine), want)
        order = smb.sharding.peer_copy_order(rank, world)
        ok &= order == [(rank + i) % world for i in range(1, world)]
        ok &= sorted(mem.opened) == sorted(mem.BASE + r * region for r in range(world) if r != rank)
        shared.close()
        ok &= sorted(mem.closed) == sorted(mem.opened) and mem.freed == [shared.local] and mem.synced == 1
        out.put(bool(ok))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_shared_output_addresses_on_gloo(smb, tmp_path, world):
    """Every rank writes its column slab into every rank's full D through the addresses that
    SharedOutput hands to the plans; each full D must come out complete and row-major."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    path = str(tmp_path / "peers.bin")
    m, n = 12, 8 * world * 3
    with open(path, "wb") as f:
        f.write(bytes(world * m * n * 2))
    procs = [ctx.Process(target=_fused_worker, args=(r, world, port, path, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(out.get(timeout=5) is True for _ in range(world))


class _Recorder:
    """Stand-ins for `dist` and the peer memory that log the order of what close() does."""

    def __init__(self):
        self.log = []

    # torch.distributed face
    def get_rank(self):
        return 0

    def get_world_size(self):
        return 2

    def barrier(self):
        self.log.append("barrier")

    def all_gather_object(self, handles, mine):
        handles[0] = mine
        handles[1] = (0x9000).to_bytes(8, "little") + bytes(56)

    # memory face
    def alloc(self, nbytes):
        return 0x5000

    def export(self, ptr):
        return int(ptr).to_bytes(8, "little") + bytes(56)

    def open(self, handle):
        return int.from_bytes(handle[:8], "little")

    def close(self, ptr):
        self.log.append("unmap")

    def free(self, ptr):
        self.log.append("free")

    def synchronize(self):
        self.log.append("sync")


@pytest.mark.parametrize("kind", ["SharedOutput", "ScatterSlots"])
def test_close_drains_the_device_before_peers_may_free(smb, kind):
    """A rank's GEMM epilogue may still be storing into the other ranks' buffers when close() is
    called; a host barrier alone does not wait for it.  Order: device synchronize, barrier, unmap,
    barrier, free."""
    rec = _Recorder()
    obj = (smb.sharding.SharedOutput(16, 32, rec, memory=rec) if kind == "SharedOutput"
           else smb.sharding.ScatterSlots(512, 32, rec, memory=rec))
    obj.close()
    assert rec.log == ["sync", "barrier", "unmap", "barrier", "free"]
    obj.close()                       # idempotent
    assert len(rec.log) == 5


def test_peer_copy_rules(smb):
    sh = smb.sharding.column_shard(64, 4, 1)
    bases = [0x1000, 0x2000, 0x3000, 0x4000]
    assert smb.sharding.peer_copy_targets(bases, sh) == [0x3000 + 32, 0x4000 + 32, 0x1000 + 32]
    with pytest.raises(ValueError):
        smb.sharding.peer_copy_targets(bases[:3], sh)
    lib = smb.capi.lib()
    # No plan: the setters validate the handle before anything else.
    assert lib.smb_bf16_plan_set_peer_copies(None, 0, None, 0) == smb.capi.SMB_ERR_INVALID
    assert lib.smb_fp4_plan_set_peer_copies(None, 0, None, 0) == smb.capi.SMB_ERR_INVALID
    assert lib.smb_unshard_columns_device(None, None, 2, 4, 8, 16, None) == smb.capi.SMB_ERR_INVALID
    assert lib.smb_peer_export(None, None) == smb.capi.SMB_ERR_INVALID


# ------------------------------------------------------------------ fused reduce-scatter plumbing
def _scatter_worker(rank, world, port, path, out):
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    smb = entry.load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, n = 256 * world, 16
        rows = m // world
        region = world * rows * n * 2
        mem = _FileBackedMemory(path, rank, region)
        slots = smb.sharding.ScatterSlots(m, n, dist, memory=mem)
        assert slots.rows_per_block == rows and slots.slot_bytes == rows * n * 2
        backing = np.memmap(path, dtype=np.uint8, mode="r+", shape=(world * region,))
        # What the routed epilogue does: row block b of this rank's partial product goes to
        # targets[b], a [rows, n] block with pitch n.
        partial = ((rank + 1) * 100 + np.arange(m)[:, None] + np.arange(n)[None, :] * 0).astype(np.uint16)
        partial = np.broadcast_to(partial, (m, n)).copy()
        for b, addr in enumerate(slots.targets()):
            off = addr - mem.BASE
            backing[off:off + rows * n * 2] = partial[b * rows:(b + 1) * rows].reshape(-1).view(np.uint8)
        backing.flush()
        dist.barrier()
        mine = np.memmap(path, dtype=np.uint16, mode="r", offset=rank * region, shape=(world, rows, n))
        ok = True
        for s in range(world):   # slot s holds rank s's partial rows of MY block
            want = ((s + 1) * 100 + np.arange(rank * rows, (rank + 1) * rows)[:, None]).astype(np.uint16)
            ok &= np.array_equal(np.asarray(mine[s]), np.broadcast_to(want, (rows, n)))
        slots.close()
        out.put(bool(ok))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_scatter_slots_addresses_on_gloo(smb, tmp_path):
    import torch.multiprocessing as mp
    world = 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    path = str(tmp_path / "slots.bin")
    with open(path, "wb") as f:
        f.write(bytes(world * world * 256 * 16 * 2))
    procs = [ctx.Process(target=_scatter_worker, args=(r, world, port, path, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    assert all(out.get(timeout=5) is True for _ in range(world))
    assert smb.sharding.route_targets([0x1000, 0x9000], 1, 0x100) == [0x1100, 0x9100]
    lib = smb.capi.lib()
    assert lib.smb_bf16_plan_set_row_route(None, 0, None, 256, 8, 0) == smb.capi.SMB_ERR_INVALID
    assert lib.smb_sum_slots_bf16_device(None, None, 2, 8, None) == smb.capi.SMB_ERR_INVALID


def test_c_abi_column_shard_agrees_with_the_python_helper(smb):
    """smb_column_shard (what the drivers' --shard uses) and sharding.column_shard state the same
    split and refuse the same inputs."""
    import ctypes as C
    lib = smb.capi.lib()
    for n_total, world in ((8192, 8), (57344, 8), (768, 3), (64, 2), (8192, 1), (100, 4), (72, 3), (64, 3), (96, 0)):
        for rank in (0, max(world - 1, 0), world):
            n0, nl = C.c_int(-1), C.c_int(-1)
            rc = lib.smb_column_shard(n_total, world, rank, C.byref(n0), C.byref(nl))
            try:
                want = smb.sharding.column_shard(n_total, world, rank)
            except ValueError:
                assert rc != 0, (n_total, world, rank)
                assert "column shard" in smb.capi.last_error()
                continue
            assert rc == 0 and (n0.value, nl.value) == (want.n0, want.n_local), (n_total, world, rank)
    assert lib.smb_column_shard(64, 2, 0, None, None) != 0
