"""The allocation-free decode entry point, for hosts that may not call cudaMalloc where the GEMM
runs (a memory pool that owns all of HBM, a plugin inside another framework's allocator, a
stream capture in progress).  It must give what the plan-based entry point gives, call after
call, although every call reuses the same built-in scratch array.

Collected last on purpose (file name): a failure here stops `pytest -x` only after every
other test has run.  Passes alone in a fresh process and after the rest of the suite."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _operand(smb, torch, rows, k, fill, which):
    dev = torch.device("cuda:0")
    data = torch.empty(rows, k // 2, device=dev, dtype=torch.uint8)
    sfp = torch.empty(smb.gemm.sf_packed_bytes(rows, k), device=dev, dtype=torch.uint8)
    smb.gemm.fill_fp4_device(data, sfp, None, rows, k, fill, which, 0)
    return data, sfp


@pytest.mark.parametrize("shape", [(16, 28672, 8192), (64, 4096, 2048), (100, 1000, 1056)])
def test_no_alloc_decode_matches_plan_entry_point_twice(smb, cuda_device, shape):
    import torch
    lib = smb.capi.lib()
    m, n, k = shape
    a, sfa = _operand(smb, torch, m, k, 6, 0)
    b, sfb = _operand(smb, torch, n, k, 5, 1)
    want = torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, want, m, n, k)
    plan.run()
    plan.check()
    plan.close()
    assert bool(torch.isfinite(want.float()).all())
    outs = [torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16) for _ in range(2)]
    torch.cuda.synchronize()
    for call in range(2):
        got = outs[call]
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.smb_dense_gemm_nvfp4_decode_noalloc(a.data_ptr(), sfa.data_ptr(), b.data_ptr(),
                                                     sfb.data_ptr(), got.data_ptr(), m, n, k, None)
        assert rc == 0, smb.capi.last_error()
        torch.cuda.synchronize()
        free_after = torch.cuda.mem_get_info()[0]
        # No device memory is taken from the driver by a call.  (Checked on the second call:
        # during the first one the driver may still be loading kernels, which costs it memory.)
        if call == 1:
            assert free_after >= free_before
        # Same kernel, same split of the work: at most the order of two fp32 additions differs.
        diff = (got.float() - want.float()).abs()
        tol = 2.0 ** -7 * want.float().abs() + 2.0 ** -10 * (k ** 0.5) * float(want.float().pow(2).mean().sqrt())
        assert bool(torch.isfinite(got.float()).all()), f"call {call}: non-finite output"
        assert int((diff > tol).sum()) == 0, f"call {call}: {int((diff > tol).sum())} elements differ"
    # The bf16 results of the two calls agree bit for bit with each other.
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


def test_no_alloc_decode_rejects_what_does_not_fit(smb, cuda_device):
    import torch
    lib = smb.capi.lib()
    t = torch.zeros(4096, device=cuda_device, dtype=torch.uint8)
    p = t.data_ptr()
    limit = lib.smb_decode_noalloc_scratch_limit()
    assert limit == (2 << 20) - 256
    # The array holds one counter per tile and partial-sum slots for at least one CTA: 2^31 - 1
    # columns are 16.8 M tiles = 67 MB of counters.
    assert lib.smb_dense_gemm_nvfp4_decode_noalloc(p, p, p, p, p, 128, 2 ** 31 - 1, 256, None) == smb.capi.SMB_ERR_UNSUPPORTED
    assert "scratch" in smb.capi.last_error()
    assert lib.smb_dense_gemm_nvfp4_decode_noalloc(p, p, p, p, p, 129, 256, 256, None) == smb.capi.SMB_ERR_UNSUPPORTED
    assert lib.smb_dense_gemm_nvfp4_decode_noalloc(p, p, p, p, p, 16, 256, 100, None) == smb.capi.SMB_ERR_UNSUPPORTED
    assert lib.smb_dense_gemm_nvfp4_decode_noalloc(None, p, p, p, p, 16, 256, 256, None) == smb.capi.SMB_ERR_INVALID
