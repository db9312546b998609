"""GPU tests of the column-sharded path: the epilogue's extra destinations (the fused all-gather),
the unshard copy of the unfused path, and exportable device memory.

The extra destinations are plain global addresses for the kernel, so most of the path is tested
on ONE GPU with destination buffers on the same device; the two-process test at the end needs two
GPUs and checks the real thing: every rank's full D, written by all ranks over peer-mapped memory,
equals the single-GPU result bit for bit."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def _torch():
    import torch
    return torch


def _bits(t):
    torch = _torch()
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


SENTINEL = 0x7FC1  # a NaN pattern no GEMM here produces


def _full(torch, m, n_total, dev):
    t = torch.empty(m, n_total, device=dev, dtype=torch.int16)
    t.fill_(SENTINEL)
    return t.view(torch.bfloat16)


@pytest.mark.parametrize("shape_flags", [((1000, 1024, 512), "FLAG_NONE"), ((256, 72, 64), "FLAG_NONE"),
                                         ((777, 512, 256), "FLAG_TILE_N_256"), ((512, 256, 128), "FLAG_TILE_N_64")])
def test_bf16_peer_copies_on_one_device(smb, cuda_device, shape_flags):
    """Slab [M, N] at columns [n0, n0 + N) of a [M, 3 N] buffer; two more such buffers get the same
    slab from the same kernel; nothing outside the slab is touched in any of them."""
    torch = _torch()
    (m, n, k), flag = shape_flags
    flags = getattr(smb.capi, flag)
    n_total, n0 = 3 * n, n
    a = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=cuda_device, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a, bt, m, n, k, 5)
    plain = torch.empty(m, n, device=cuda_device, dtype=torch.bfloat16)
    p0 = smb.gemm.Bf16Plan(a, bt, plain, m, n, k, flags=flags)
    p0.run(); p0.check(); p0.close()
    fulls = [_full(torch, m, n_total, cuda_device) for _ in range(3)]
    elem = 2
    plan = smb.gemm.Bf16Plan(a, bt, fulls[0].data_ptr() + n0 * elem, m, n, k, ldd=n_total, flags=flags)
    plan.set_peer_copies([f.data_ptr() + n0 * elem for f in fulls[1:]], n_total)
    for _ in range(2):
        plan.run()
    plan.check()
    for f in fulls:
        got = _bits(f)
        np.testing.assert_array_equal(got[:, n0:n0 + n], _bits(plain))
        assert np.all(got[:, :n0] == SENTINEL) and np.all(got[:, n0 + n:] == SENTINEL)
    # Switching the copies off again leaves the other buffers alone.
    plan.set_peer_copies([], n_total)
    fulls[1].view(torch.int16).fill_(SENTINEL)
    plan.run(); plan.check(); plan.close()
    assert np.all(_bits(fulls[1]) == SENTINEL)


def test_fp4_peer_copies_on_one_device(smb, cuda_device):
    torch = _torch()
    sys.path.insert(0, str(ROOT / "tests"))
    from test_gemm_gpu import _fp4_operand
    m, n, k = 520, 768, 512
    n_total, n0 = 2 * n, n
    a, sfa, _ = _fp4_operand(smb, m, k, 5, 0)
    b, sfb, _ = _fp4_operand(smb, n, k, 5, 1)
    plain = torch.empty(m, n, device=cuda_device, dtype=torch.bfloat16)
    p0 = smb.gemm.Fp4Plan(a, sfa, b, sfb, plain, m, n, k)
    p0.run(); p0.check(); p0.close()
    fulls = [_full(torch, m, n_total, cuda_device) for _ in range(8)]
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, fulls[0].data_ptr() + n0 * 2, m, n, k, ldd=n_total)
    plan.set_peer_copies([f.data_ptr() + n0 * 2 for f in fulls[1:]], n_total)   # 7: the maximum
    plan.run(); plan.check(); plan.close()
    for f in fulls:
        got = _bits(f)
        np.testing.assert_array_equal(got[:, n0:], _bits(plain))
        assert np.all(got[:, :n0] == SENTINEL)


def test_peer_copies_are_refused_where_they_cannot_work(smb, cuda_device):
    torch = _torch()
    lib, capi = smb.capi.lib(), smb.capi
    m, n, k = 256, 128, 64
    a = torch.zeros(m, k, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.zeros(n, k, device=cuda_device, dtype=torch.bfloat16)
    d = torch.zeros(m, n, device=cuda_device, dtype=torch.bfloat16)
    other = torch.zeros(m, n + 8, device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Bf16Plan(a, bt, d, m, n, k)
    with pytest.raises(capi.SmbError):
        plan.set_peer_copies([other] * 8, n)                      # more than 7
    with pytest.raises(capi.SmbError):
        plan.set_peer_copies([other.data_ptr() + 2], n)           # not 16-byte aligned
    with pytest.raises(capi.SmbError):
        plan.set_peer_copies([other], n - 8)                      # pitch shorter than a row
    with pytest.raises(capi.SmbError):
        plan.set_peer_copies([other], n + 4)                      # pitch not a multiple of 8
    plan.close()
    plain_store = smb.gemm.Bf16Plan(a, bt, d, m, n, k, flags=capi.FLAG_FORCE_PLAIN_STORE)
    with pytest.raises(capi.SmbError):
        plain_store.set_peer_copies([other], n + 8)
    plain_store.close()
    # FP4 decode-path plans (M <= 128) have a different epilogue.
    sys.path.insert(0, str(ROOT / "tests"))
    from test_gemm_gpu import _fp4_operand
    xa, xsfa, _ = _fp4_operand(smb, 16, 256, 6, 0)
    w, wsf, _ = _fp4_operand(smb, 256, 256, 5, 1)
    dd = torch.zeros(16, 256, device=cuda_device, dtype=torch.bfloat16)
    dplan = smb.gemm.Fp4Plan(xa, xsfa, w, wsf, dd, 16, 256, 256)
    with pytest.raises(capi.SmbError):
        dplan.set_peer_copies([other], 256)
    dplan.close()
    del lib


@pytest.mark.parametrize("dims", [(2, 100, 64), (8, 257, 1024), (4, 33, 8)])
def test_unshard_columns_matches_a_permute(smb, cuda_device, dims):
    torch = _torch()
    g, m, nl = dims
    gathered = torch.randint(-32768, 32767, (g, m, nl), device=cuda_device, dtype=torch.int16)
    ldd = g * nl + 8
    out = torch.full((m, ldd), -1, device=cuda_device, dtype=torch.int16)
    smb.gemm.unshard_columns_device(gathered, out, g, m, nl, ldd=ldd)
    torch.cuda.synchronize()
    want = gathered.permute(1, 0, 2).reshape(m, g * nl)
    assert torch.equal(out[:, :g * nl], want)
    assert bool((out[:, g * nl:] == -1).all())


def test_exportable_memory_round_trip(smb, cuda_device):
    """Allocate, export a handle, use the memory as a GEMM output, free.  (Opening the handle needs
    a second process: covered by the two-GPU test.)"""
    torch = _torch()
    mem = smb.sharding._CudaPeerMemory()
    ptr = mem.alloc(256 * 128 * 2)
    handle = mem.export(ptr)
    assert len(handle) == smb.capi.PEER_HANDLE_BYTES and any(handle)
    a = torch.empty(256, 64, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.empty(128, 64, device=cuda_device, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a, bt, 256, 128, 64, 3)
    plan = smb.gemm.Bf16Plan(a, bt, ptr, 256, 128, 64)
    plan.run(); plan.check(); plan.close()
    host = np.empty((256, 128), dtype=np.uint16)
    torch.cuda.synchronize()
    # Read back through a torch view of the raw pointer.
    class _Raw:
        pass
    raw = _Raw()
    raw.__cuda_array_interface__ = {"shape": (256 * 128 * 2,), "typestr": "|u1", "data": (ptr, False),
                                    "version": 2}
    view = torch.as_tensor(raw, device=cuda_device).view(torch.bfloat16).view(256, 128)
    host[:] = _bits(view)
    assert np.all(host == 0x4280)   # fill 3: every product is 1, K = 64 -> 64.0
    del view
    mem.free(ptr)


# ------------------------------------------------------------------ two GPUs, two processes
def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


_PG_TIMEOUT = __import__("datetime").timedelta(seconds=120)


def _run_ranks(ctx, target, world, args, out, timeout=300):
    """Start one child per rank, wait, and never leave one behind: a child that is still alive at
    the deadline is terminated (then killed) so that it does not keep its GPU, and the test fails
    with what the children reported."""
    procs = [ctx.Process(target=target, args=(r, world, *args)) for r in range(world)]
    for p in procs:
        p.start()
    deadline = __import__("time").time() + timeout
    for p in procs:
        p.join(timeout=max(1.0, deadline - __import__("time").time()))
    stuck = [p for p in procs if p.is_alive()]
    for p in stuck:
        p.terminate()
    for p in stuck:
        p.join(timeout=10)
        if p.is_alive():
            p.kill()
            p.join(timeout=10)
    results = {}
    while len(results) < world:
        try:
            rank, ok = out.get(timeout=2)
        except Exception:
            break
        results[rank] = ok
    assert not stuck, f"{len(stuck)} rank(s) did not finish within {timeout} s; reports so far: {results}"
    assert all(p.exitcode == 0 for p in procs), f"exit codes {[p.exitcode for p in procs]}; reports: {results}"
    assert results == {r: True for r in range(world)}, results


def _two_gpu_worker(rank, world, port, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    smb = entry.load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=_PG_TIMEOUT)
    try:
        m, n, k, fill = 1000, 2048, 512, 5
        shared = smb.sharding.SharedOutput(m, n, dist)
        sh = shared.shard()
        d_full = shared.local_tensor()
        d_full.view(torch.int16).fill_(SENTINEL)
        torch.cuda.synchronize()
        dist.barrier()
        a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
        bt = torch.empty(sh.n_local, k, device=dev, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt, m, sh.n_local, k, fill, n0=sh.n0, n_total=n)
        plan = smb.gemm.Bf16Plan(a, bt, shared.slab_address(), m, sh.n_local, k, ldd=n)
        plan.set_peer_copies(shared.peer_targets(), n)
        plan.run()
        plan.check()            # synchronises the stream: this rank's writes are complete
        dist.barrier()          # ... and so are everybody else's
        # Single-GPU result of the whole problem, computed locally.
        bt_all = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt_all, m, n, k, fill)
        ref = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        p1 = smb.gemm.Bf16Plan(a, bt_all, ref, m, n, k)
        p1.run(); p1.check(); p1.close()
        ok = torch.equal(d_full.view(torch.int16), ref.view(torch.int16))
        plan.close()
        del d_full
        shared.close()
        out.put((rank, bool(ok)))
    except BaseException:
        import traceback
        out.put((rank, traceback.format_exc()))
        raise
    finally:
        dist.destroy_process_group()


def test_fused_all_gather_on_two_gpus(smb, cuda_device):
    torch = _torch()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    _run_ranks(ctx, _two_gpu_worker, 2, (port, out), out)


# ------------------------------------------------------------------ K-sharded GEMM + fused scatter
@pytest.mark.parametrize("kind", ["bf16", "fp4"])
def test_row_route_and_slot_sum_on_one_device(smb, cuda_device, kind):
    """Two "ranks" on one GPU: each multiplies its half of K and routes row block b of its partial
    product into slot [rank] of "rank" b's receive buffer; summing the slots gives the full
    product (to the rounding of the bf16 partials)."""
    torch = _torch()
    sys.path.insert(0, str(ROOT / "tests"))
    from test_gemm_gpu import _fp4_operand, _dequant
    g, m, n, k = 2, 1024, 384, 1024
    rows, kl = m // g, k // g
    recv = [torch.full((g, rows, n), float("nan"), device=cuda_device, dtype=torch.bfloat16) for _ in range(g)]
    d_unused = torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    if kind == "bf16":
        a = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=cuda_device, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt, m, n, k, 5)
        ref = a.double() @ bt.double().t()
    else:
        a, sfa, sfar = _fp4_operand(smb, m, k, 5, 0)
        b, sfb, sfbr = _fp4_operand(smb, n, k, 5, 1)
        ref = _dequant(a, sfar) @ _dequant(b, sfbr).t()
    for r in range(g):
        targets = [recv[b][r].data_ptr() for b in range(g)]
        if kind == "bf16":
            a_r = a[:, r * kl:(r + 1) * kl].contiguous()
            bt_r = bt[:, r * kl:(r + 1) * kl].contiguous()
            plan = smb.gemm.Bf16Plan(a_r, bt_r, d_unused, m, n, kl)
        else:
            a_r, sfa_r, _ = _fp4_slice(smb, a, sfar, r, g)
            b_r, sfb_r, _ = _fp4_slice(smb, b, sfbr, r, g)
            plan = smb.gemm.Fp4Plan(a_r, sfa_r, b_r, sfb_r, d_unused, m, n, kl)
        plan.set_row_route(targets, rows, n, (r + 1) % g)
        plan.run(); plan.check()
        with pytest.raises(smb.capi.SmbError):
            plan.set_row_route(targets, rows + 8, n)          # not a multiple of the tile height
        plan.close()
    assert bool(torch.isnan(d_unused).all())                   # a routed plan does not write its D
    out = torch.empty(m, n, device=cuda_device, dtype=torch.bfloat16)
    for b in range(g):
        smb.gemm.sum_slots_bf16_device(recv[b], out[b * rows:(b + 1) * rows], g, rows * n)
    torch.cuda.synchronize()
    got = out.double()
    rms = float(ref.pow(2).mean().sqrt())
    bound = 2.0 ** -6 * ref.abs() + 2.0 ** -9 * (k ** 0.5) * rms     # two bf16 roundings of partials + sum
    assert int((~torch.isfinite(got) | ((got - ref).abs() > bound)).sum()) == 0
    # The sum kernel alone: exact against torch on the same slots.
    want = recv[0].float().sum(dim=0).to(torch.bfloat16)
    assert torch.equal(out[:rows].view(torch.int16), want.view(torch.int16))


def _fp4_slice(smb, codes, sf_rowmajor, r, g):
    """K slice r of g of a quantised operand: codes, packed scales, row-major scales."""
    torch = _torch()
    kb = codes.shape[1] // g
    sb = sf_rowmajor.shape[1] // g
    c = codes[:, r * kb:(r + 1) * kb].contiguous()
    s = sf_rowmajor[:, r * sb:(r + 1) * sb].contiguous()
    packed = np.zeros(smb.capi.lib().smb_sf_packed_bytes(c.shape[0], sb), dtype=np.uint8)
    s_host = s.cpu().numpy()
    smb.capi.check(smb.capi.lib().smb_sf_pack_host(s_host.ctypes.data, c.shape[0], sb, packed.ctypes.data))
    return c, torch.from_numpy(packed).to(codes.device), s


def _two_gpu_scatter_worker(rank, world, port, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    smb = entry.load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=_PG_TIMEOUT)
    try:
        m, n, k, fill = 1024, 512, 2048, 5
        kl = k // world
        slots = smb.sharding.ScatterSlots(m, n, dist)
        rows = slots.rows_per_block
        a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt, m, n, k, fill)
        a_r = a[:, rank * kl:(rank + 1) * kl].contiguous()
        bt_r = bt[:, rank * kl:(rank + 1) * kl].contiguous()
        unused = torch.zeros(m, n, device=dev, dtype=torch.bfloat16)
        plan = smb.gemm.Bf16Plan(a_r, bt_r, unused, m, n, kl)
        plan.set_row_route(slots.targets(), rows, n, slots.first_block())
        dist.barrier()
        plan.run()
        plan.check()            # own deliveries complete
        dist.barrier()          # everybody's deliveries complete
        mine = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        smb.gemm.sum_slots_bf16_device(slots.local, mine, world, rows * n)
        torch.cuda.synchronize()
        ref = (a.double() @ bt.double().t())[rank * rows:(rank + 1) * rows]
        rms = float(ref.pow(2).mean().sqrt())
        bound = 2.0 ** -6 * ref.abs() + 2.0 ** -9 * (k ** 0.5) * rms
        got = mine.double()
        ok = int((~torch.isfinite(got) | ((got - ref).abs() > bound)).sum()) == 0
        plan.close()
        slots.close()
        out.put((rank, bool(ok)))
    except BaseException:
        import traceback
        out.put((rank, traceback.format_exc()))
        raise
    finally:
        dist.destroy_process_group()


def test_fused_scatter_on_two_gpus(smb, cuda_device):
    torch = _torch()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    _run_ranks(ctx, _two_gpu_scatter_worker, 2, (port, out), out)


def test_plan_refuses_to_run_on_another_device(smb, cuda_device):
    """A plan's pointers, tensor maps and status word belong to the device that was current when it
    was created; running it with another device current is an error, not a launch."""
    torch = _torch()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    m, n, k = 256, 256, 128
    a = torch.zeros(m, k, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.zeros(n, k, device=cuda_device, dtype=torch.bfloat16)
    d = torch.zeros(m, n, device=cuda_device, dtype=torch.bfloat16)
    with torch.cuda.device(0):
        plan = smb.gemm.Bf16Plan(a, bt, d, m, n, k)
    try:
        with torch.cuda.device(1):
            with pytest.raises(smb.capi.SmbError, match="created on device 0"):
                plan.run()
        with torch.cuda.device(0):
            plan.run()
            plan.check()
    finally:
        plan.close()


# ------------------------------------------------------------------ all-gather and sharded host contexts behind the C ABI
def _capi_gather_worker(rank, world, port, out):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, str(ROOT))
    import __graft_entry__ as entry
    smb = entry.load_package()
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=_PG_TIMEOUT)
    try:
        # The library's own communicator: rank 0 makes the id, the others get it over the host channel.
        ident = [smb.gemm.Comm.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(ident, 0)
        comm = smb.gemm.Comm(ident[0], world, rank)
        m, n, k, fill = 1024, 1536, 512, 5
        sh = smb.sharding.column_shard(n, world, rank)
        a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
        bt = torch.empty(sh.n_local, k, device=dev, dtype=torch.bfloat16)
        slab = torch.empty(m, sh.n_local, device=dev, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt, m, sh.n_local, k, fill, n0=sh.n0, n_total=n)
        plan = smb.gemm.Bf16Plan(a, bt, slab, m, sh.n_local, k)
        plan.run(); plan.check(); plan.close()
        # Single-GPU result of the whole problem, computed locally.
        bt_all = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt_all, m, n, k, fill)
        ref = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
        p1 = smb.gemm.Bf16Plan(a, bt_all, ref, m, n, k)
        p1.run(); p1.check(); p1.close()
        gathered = torch.full((world, m, sh.n_local), float("nan"), device=dev, dtype=torch.bfloat16)
        full = torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16)
        comm.allgather_columns(slab, gathered, full, m, sh.n_local)
        torch.cuda.synchronize()
        ok = torch.equal(full.view(torch.int16), ref.view(torch.int16))
        ok &= torch.equal(gathered[rank].view(torch.int16), slab.view(torch.int16))
        # Sharded host context: this rank sends its M / world rows of A and its shard of BT; the
        # GPUs complete A over NVLink inside the run.
        rows = m // world
        a_host = a[rank * rows:(rank + 1) * rows].view(torch.int16).cpu().numpy().view(np.uint16)
        bt_host = bt.view(torch.int16).cpu().numpy().view(np.uint16)
        ctx = smb.gemm.Bf16HostContext(m, sh.n_local, k, comm=comm)
        for _ in range(2):
            d_host = np.zeros((m, sh.n_local), dtype=np.uint16)
            ctx.run(a_host, bt_host, d_host)
            ok &= np.array_equal(d_host, slab.view(torch.int16).cpu().numpy().view(np.uint16))
        ctx.close()
        # The same for the block-scaled GEMM (codes and row-major scales of A travel in blocks).
        def fp4_operand(rows_, fill_, which, row0):
            data = torch.empty(rows_, k // 2, device=dev, dtype=torch.uint8)
            sfp = torch.empty(smb.gemm.sf_packed_bytes(rows_, k), device=dev, dtype=torch.uint8)
            sfr = torch.empty(rows_, k // 32, device=dev, dtype=torch.uint8)
            smb.gemm.fill_fp4_device(data, sfp, sfr, rows_, k, fill_, which, row0)
            return data, sfp, sfr

        fa, fsfa, fsfar = fp4_operand(m, 6, 0, 0)
        fb, fsfb, fsfbr = fp4_operand(sh.n_local, 5, 1, sh.n0)
        fd = torch.empty(m, sh.n_local, device=dev, dtype=torch.bfloat16)
        fplan = smb.gemm.Fp4Plan(fa, fsfa, fb, fsfb, fd, m, sh.n_local, k)
        fplan.run(); fplan.check(); fplan.close()
        fctx = smb.gemm.Fp4HostContext(m, sh.n_local, k, comm=comm)
        d_host = np.zeros((m, sh.n_local), dtype=np.uint16)
        fctx.run(fa[rank * rows:(rank + 1) * rows].cpu().numpy(), fsfar[rank * rows:(rank + 1) * rows].cpu().numpy(),
                 fb.cpu().numpy(), fsfbr.cpu().numpy(), d_host)
        ok &= np.array_equal(d_host, fd.view(torch.int16).cpu().numpy().view(np.uint16))
        fctx.close()
        dist.barrier()
        comm.close()
        out.put((rank, bool(ok)))
    except BaseException:
        import traceback
        out.put((rank, traceback.format_exc()))
        raise
    finally:
        dist.destroy_process_group()


def test_capi_allgather_and_sharded_host_contexts_on_two_gpus(smb, cuda_device):
    """smb_comm_* + smb_allgather_columns (NCCL resolved at run time) give every rank the
    single-GPU result bit for bit; the sharded host contexts give each rank its slab while the host
    sends every row of A once."""
    torch = _torch()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    _run_ranks(ctx, _capi_gather_worker, 2, (_free_port(), out), out)


def test_capi_allgather_single_rank(smb, cuda_device):
    """A world of one: the all-gather is a copy and the unshard copy the identity.  Exercises the
    run-time NCCL binding on a 1-GPU box."""
    torch = _torch()
    m, nl = 512, 256
    comm = smb.gemm.Comm(smb.gemm.Comm.unique_id(), 1, 0)
    slab = torch.randn(m, nl, device=cuda_device).to(torch.bfloat16)
    gathered = torch.zeros(1, m, nl, device=cuda_device, dtype=torch.bfloat16)
    full = torch.zeros(m, nl, device=cuda_device, dtype=torch.bfloat16)
    comm.allgather_columns(slab, gathered, full, m, nl)
    torch.cuda.synchronize()
    assert torch.equal(gathered[0], slab) and torch.equal(full, slab)
    with pytest.raises(smb.capi.SmbError):
        comm.allgather_columns(slab, gathered, full, m, 100)      # slab width not a multiple of 8
    comm.close()
