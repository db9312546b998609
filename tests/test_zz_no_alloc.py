"""The allocation-free decode entry point.

Who needs it: a serving process whose memory pool took all of HBM at start-up, or a plugin that
lives inside another framework's allocator.  For both, a cudaMalloc on the request path either
fails outright or stalls every stream of the device, so the decode GEMM must run with nothing but
its operands and a scratch array that is part of the library image.  Every call reuses that one
array, so the test makes two calls in a row and holds each to the float64 product and to the
plan-based entry point.

Collected last on purpose (file name): a failure here stops `pytest -x` only after every
other test has run.  Passes alone in a fresh process and after the rest of the suite."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LUT = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0]


def _operand(smb, torch, rows, k, fill, which):
    dev = torch.device("cuda:0")
    data = torch.empty(rows, k // 2, device=dev, dtype=torch.uint8)
    sfp = torch.empty(smb.gemm.sf_packed_bytes(rows, k), device=dev, dtype=torch.uint8)
    sfr = torch.empty(rows, k // 32, device=dev, dtype=torch.uint8)
    smb.gemm.fill_fp4_device(data, sfp, sfr, rows, k, fill, which, 0)
    return data, sfp, sfr


def _dequant(torch, data, sfr):
    lut = torch.tensor(LUT, device=data.device, dtype=torch.float64)
    v = torch.stack([lut[(data & 15).long()], lut[(data >> 4).long()]], dim=-1).reshape(data.shape[0], -1)
    return v * torch.exp2(sfr.double() - 127).repeat_interleave(32, dim=1)


@pytest.mark.parametrize("split", [0, 96], ids=["whole_tile_pairs", "stream_k_96_ctas"])
@pytest.mark.parametrize("shape", [(16, 28672, 8192), (64, 4096, 2048), (100, 1000, 1056)])
def test_no_alloc_decode_twice_against_fp64_and_plan(smb, cuda_device, shape, split):
    """split = 0: every CTA owns whole tile pairs, only the status word of the built-in array is
    used.  split = 96: stream-K ranges over (at most) 96 CTAs, so tiles are shared between CTAs
    and the counters and partial-sum slots of the built-in array carry the hand-over."""
    import torch
    lib = smb.capi.lib()
    m, n, k = shape
    a, sfa, sfar = _operand(smb, torch, m, k, 6, 0)
    b, sfb, sfbr = _operand(smb, torch, n, k, 5, 1)
    ref = _dequant(torch, a, sfar) @ _dequant(torch, b, sfbr).t()
    bound = 2.0 ** -7 * ref.abs() + 2.0 ** -10 * (k ** 0.5) * float(ref.pow(2).mean().sqrt())
    want = torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, want, m, n, k)
    # The plan-based entry point with the same work split: the built-in array lowers the CTA
    # count to the partial-sum slots that fit beside the tile counters.
    m_pad = (m + 15) // 16 * 16
    fit = (lib.smb_decode_noalloc_scratch_limit() - (n + 127) // 128 * 4) // (2 * m_pad * 512)
    plan.tune(0, min(split, fit), -1)
    plan.run()
    plan.check()
    plan.close()
    outs = [torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16) for _ in range(2)]
    assert lib.smb_decode_noalloc_set_split(split) == 0
    try:
        for call in range(2):
            got = outs[call]
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            rc = lib.smb_dense_gemm_nvfp4_decode_noalloc(a.data_ptr(), sfa.data_ptr(), b.data_ptr(),
                                                         sfb.data_ptr(), got.data_ptr(), m, n, k, None)
            assert rc == 0, smb.capi.last_error()
            assert lib.smb_decode_noalloc_check(None) == 0, smb.capi.last_error()
            free_after = torch.cuda.mem_get_info()[0]
            # No device memory is taken from the driver by a call.  (Checked on the second call:
            # during the first one the driver may still be loading kernels, which costs it memory.)
            if call == 1:
                assert free_after >= free_before
            # Parity proper: the float64 product of the represented values, north-star bound
            # |C - C64| <= 2^-7 |C64| + 2^-10 sqrt(K) rms(C64).
            bad = ~torch.isfinite(got.double()) | ((got.double() - ref).abs() > bound)
            assert int(bad.sum()) == 0, f"call {call}: {int(bad.sum())} elements outside the bound"
            # Same kernel and same work split as the plan-based entry point: the same bits.
            assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}"
    finally:
        lib.smb_decode_noalloc_set_split(0)


def test_no_alloc_decode_rejects_what_does_not_fit(smb, cuda_device):
    import torch
    lib = smb.capi.lib()
    t = torch.zeros(4096, device=cuda_device, dtype=torch.uint8)
    p = t.data_ptr()
    limit = lib.smb_decode_noalloc_scratch_limit()
    assert limit == (2 << 20) - 256
    assert lib.smb_decode_noalloc_set_split(-1) == smb.capi.SMB_ERR_INVALID
    assert lib.smb_decode_noalloc_set_split(5000) == smb.capi.SMB_ERR_INVALID
    # With the stream-K split the array must hold one counter per tile and partial-sum slots for at
    # least one CTA: 2^31 - 1 columns are 16.8 M tiles = 67 MB of counters.
    assert lib.smb_decode_noalloc_set_split(8) == 0
    try:
        rc = lib.smb_dense_gemm_nvfp4_decode_noalloc(p, p, p, p, p, 128, 2 ** 31 - 1, 256, None)
        assert rc == smb.capi.SMB_ERR_UNSUPPORTED
        assert "scratch" in smb.capi.last_error()
    finally:
        lib.smb_decode_noalloc_set_split(0)
    assert lib.smb_dense_gemm_nvfp4_decode_noalloc(p, p, p, p, p, 129, 256, 256, None) == smb.capi.SMB_ERR_UNSUPPORTED
    assert lib.smb_dense_gemm_nvfp4_decode_noalloc(p, p, p, p, p, 16, 256, 100, None) == smb.capi.SMB_ERR_UNSUPPORTED
    assert lib.smb_dense_gemm_nvfp4_decode_noalloc(None, p, p, p, p, 16, 256, 256, None) == smb.capi.SMB_ERR_INVALID
