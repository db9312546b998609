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
    dist.init_process_group("gloo", rank=rank, world_size=world)
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
    procs = [ctx.Process(target=_two_gpu_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    results = dict(out.get(timeout=5) for _ in range(2))
    assert results == {0: True, 1: True}
