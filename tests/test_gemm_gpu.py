"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle and the
golden vectors produced by the reference's own verifier code.

Tolerances (stated where used):
  * north-star bound  |C - C64| <= 2^-7 |C64| + 2^-10 sqrt(K) rms(C64)  against an fp64 reference;
  * the reference verifiers' bounds: BF16 max(0.05, 0.05 |ref|), NVFP4 max(16, 0.008 |ref|)
    against the reference CPU path's fp32 result;
  * exact equality where the arithmetic is exact (constant fills, generators, quantiser).
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _torch():
    import torch
    return torch


def _bits(t):
    """bf16 CUDA tensor -> uint16 numpy."""
    torch = _torch()
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _run_bf16(smb, m, n, k, fill, flags=0, ldd=None, group_m=0, max_clusters=0):
    torch = _torch()
    dev = torch.device("cuda:0")
    a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
    ldd = n if ldd is None else ldd
    d = torch.full((m, ldd), float("nan"), device=dev, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a, bt, m, n, k, fill)
    plan = smb.gemm.Bf16Plan(a, bt, d, m, n, k, ldd=ldd, flags=flags)
    plan.tune(group_m, max_clusters)
    plan.run()
    plan.check()
    plan.close()
    return a, bt, d


def _check_bf16_full(oracle, a, bt, d, n, k):
    torch = _torch()
    ref = a.double() @ bt.double().t()
    got = d[:, :n].double()
    rms = float(ref.pow(2).mean().sqrt())
    bound = 2.0 ** -7 * ref.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    bad = ~torch.isfinite(got) | ((got - ref).abs() > bound)
    assert int(bad.sum()) == 0, f"{int(bad.sum())} elements outside the north-star bound"


# ------------------------------------------------------------------------------- generators
@pytest.mark.parametrize("fill", [1, 2, 3, 4, 5, 6, 7])
def test_device_bf16_fill_is_bit_identical_to_oracle(smb, oracle, cuda_device, fill):
    torch = _torch()
    m, k, n = 130, 264, 77
    a = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=cuda_device, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a, bt, m, n, k, fill)
    wa, wbt = oracle.bf16_operands(m, n, k, fill)
    np.testing.assert_array_equal(_bits(a), wa)
    np.testing.assert_array_equal(_bits(bt), wbt)
    # N-shard slab with global indices.
    slab = torch.empty(16, k, device=cuda_device, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a, slab, m, 16, k, fill, n0=40, n_total=n)
    np.testing.assert_array_equal(_bits(slab), wbt[40:56])


@pytest.mark.parametrize("fill", [1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("which", [0, 1])
def test_device_fp4_fill_is_bit_identical_to_oracle(smb, oracle, cuda_device, fill, which):
    torch = _torch()
    rows, k, row0 = 200, 384, 11
    data = torch.empty(rows, k // 2, device=cuda_device, dtype=torch.uint8)
    sfp = torch.empty(smb.gemm.sf_packed_bytes(rows, k), device=cuda_device, dtype=torch.uint8)
    sfr = torch.empty(rows, k // 32, device=cuda_device, dtype=torch.uint8)
    smb.gemm.fill_fp4_device(data, sfp, sfr, rows, k, fill, which, row0)
    codes, sf = oracle.fp4_operand(rows, k, fill, which, row0)
    np.testing.assert_array_equal(data.cpu().numpy(), oracle.pack_codes(codes))
    np.testing.assert_array_equal(sfr.cpu().numpy(), sf)
    np.testing.assert_array_equal(sfp.cpu().numpy(), oracle.sf_pack(sf))


def test_device_quantizer_is_bit_identical_to_oracle(smb, oracle, cuda_device):
    torch = _torch()
    rng = np.random.default_rng(21)
    x = (rng.standard_normal((96, 512)) * np.exp2(rng.integers(-8, 8, (96, 1)))).astype(np.float32)
    x[0, :32] = 0
    x[1, :8] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0]
    x[1, 8:32] = 0
    xs = torch.from_numpy(x).to(cuda_device)
    data = torch.empty(96, 256, device=cuda_device, dtype=torch.uint8)
    sfp = torch.empty(smb.gemm.sf_packed_bytes(96, 512), device=cuda_device, dtype=torch.uint8)
    sfr = torch.empty(96, 16, device=cuda_device, dtype=torch.uint8)
    smb.capi.check(smb.capi.lib().smb_quantize_mx_device(
        xs.data_ptr(), 512, data.data_ptr(), 256, sfp.data_ptr(), sfr.data_ptr(), 96, 512, None))
    torch.cuda.synchronize()
    codes, sf = oracle.quantize_mx(x)
    np.testing.assert_array_equal(sfr.cpu().numpy(), sf)
    np.testing.assert_array_equal(data.cpu().numpy(), oracle.pack_codes(codes))
    # "Dequantised operands match bit-exactly": decode both and compare.
    np.testing.assert_array_equal(
        oracle.dequantize(oracle.unpack_codes(data.cpu().numpy()), sfr.cpu().numpy()).view(np.uint32),
        oracle.dequantize(codes, sf).view(np.uint32))


# ------------------------------------------------------------------------------- BF16 GEMM
@pytest.mark.parametrize("fill", [1, 2, 3, 4])
def test_bf16_smoke_against_reference_golden(smb, oracle, golden, cuda_device, fill):
    """The reference's smoke case (--shape=256,64,128): output vs the reference CPU path."""
    m, k, n = 256, 64, 128
    a, bt, d = _run_bf16(smb, m, n, k, fill)
    got = _bits(d)
    want = golden[f"bf16_smoke_out_m{fill}"]
    # Verifier tolerance on every element (it samples 64; here all 32768).
    ok, bad = oracle.check_verifier_bf16(got, oracle.bf16_to_f32(want))
    assert ok, bad
    # And bit-level: fp32 accumulation order may move a result by one bf16 ulp at most.
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1 and (diff == 0).mean() > 0.99
    if fill == 3:
        assert np.all(oracle.bf16_to_f32(got) == 64.0)


def test_bf16_smoke_through_host_entry_point(smb, oracle, cuda_device):
    a_bits, bt_bits = oracle.bf16_operands(256, 128, 64, 1)
    d = smb.gemm.dense_gemm_bf16_host(a_bits, bt_bits)
    ref = oracle.gemm_f64(oracle.bf16_to_f32(a_bits), oracle.bf16_to_f32(bt_bits))
    ok, ratio, bad = oracle.check_north_star(d, ref, 64)
    assert ok, (ratio, bad)


@pytest.mark.parametrize("shape", [
    (256, 64, 128),      # BASELINE config 1 read as M=256, N=64, K=128
    (256, 256, 64),
    (512, 512, 512),
    (300, 200, 72),      # ragged everywhere
    (1, 8, 8),           # minimum
    (257, 513, 136),
    (1024, 2048, 4096),
    (2048, 2624, 2048),  # N tail inside a 512-wide tile
])
@pytest.mark.parametrize("fill", [2, 5])
def test_bf16_shapes_against_fp64(smb, oracle, cuda_device, shape, fill):
    m, n, k = shape
    a, bt, d = _run_bf16(smb, m, n, k, fill)
    _check_bf16_full(oracle, a, bt, d, n, k)


@pytest.mark.parametrize("flags_name", ["FLAG_TILE_N_64", "FLAG_TILE_N_128", "FLAG_TILE_N_256",
                                        "FLAG_TILE_N_512", "FLAG_FORCE_PLAIN_STORE"])
def test_bf16_every_tile_configuration(smb, oracle, cuda_device, flags_name):
    flags = getattr(smb.capi, flags_name)
    m, n, k = 768, 1088, 2112
    a, bt, d = _run_bf16(smb, m, n, k, 5, flags=flags)
    _check_bf16_full(oracle, a, bt, d, n, k)


@pytest.mark.parametrize("tile", ["FLAG_TILE_N_64", "FLAG_TILE_N_128"])
@pytest.mark.parametrize("overlap", ["FLAG_OPERANDS_STATIC", "FLAG_LAUNCH_INDEPENDENT"])
@pytest.mark.parametrize("store", ["FLAG_NONE", "FLAG_FORCE_PLAIN_STORE"])
def test_bf16_narrow_tiles_two_ctas_per_sm(smb, oracle, cuda_device, tile, overlap, store):
    """Narrow tiles launched with overlapping launches allowed run as the variant whose CTAs share
    an SM in pairs (short ring, half of tensor memory).  More tiles than cluster slots, a ragged
    edge in M and N, several launches back to back; results as for every other configuration, and
    bit-identical to the one-CTA-per-SM variant of the same tile."""
    torch = _torch()
    flags = getattr(smb.capi, tile) | getattr(smb.capi, store)
    m, n, k = 2500, 1088, 2112          # 10 x 9 (or 17) tiles of 256 x 128 (64)
    a, bt, d1 = _run_bf16(smb, m, n, k, 5, flags=flags)
    _check_bf16_full(oracle, a, bt, d1, n, k)
    d2 = torch.full_like(d1, float("nan"))
    plan = smb.gemm.Bf16Plan(a, bt, d2, m, n, k, flags=flags | getattr(smb.capi, overlap))
    for _ in range(4):
        plan.run()
    plan.check()
    plan.close()
    torch.cuda.synchronize()
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))
    # The shape class the variant is for: N = 128, one tile per cluster, launches overlapping.
    m, n, k = 14080, 128, 2048
    a, bt, d1 = _run_bf16(smb, m, n, k, 2)
    d2 = torch.full_like(d1, float("nan"))
    plan = smb.gemm.Bf16Plan(a, bt, d2, m, n, k, flags=getattr(smb.capi, overlap) | getattr(smb.capi, store))
    for _ in range(8):
        plan.run()
    plan.check()
    plan.close()
    torch.cuda.synchronize()
    assert torch.equal(d1.view(torch.int16), d2.view(torch.int16))


def test_bf16_ragged_edge_case(smb, oracle, cuda_device):
    """BASELINE config 5's ragged case: M=4095, N=12289, K=4160.  D's row pitch (24578 B) is not a
    multiple of 16, so this runs the plain-store epilogue; rows of A/B are 16-byte aligned."""
    torch = _torch()
    m, n, k = 4095, 12289, 4160
    a, bt, d = _run_bf16(smb, m, n, k, 6)
    rows, cols = oracle.sample_coordinates(m, n, 4096)
    # Sampled fp64 check on the GPU operands plus full tiles on every edge.
    ra = torch.from_numpy(rows).to(cuda_device)
    ca = torch.from_numpy(cols).to(cuda_device)
    ref = (a[ra].double() * bt[ca].double()).sum(1)
    full = a[-300:].double() @ bt.double().t()
    rms = float(full.pow(2).mean().sqrt())
    got = d[ra, ca].double()
    bound = 2.0 ** -7 * ref.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    assert int(((got - ref).abs() > bound).sum()) == 0
    got_full = d[-300:].double()
    bound = 2.0 ** -7 * full.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    assert int(((got_full - full).abs() > bound).sum()) == 0
    right = a.double() @ bt[-130:].double().t()
    bound = 2.0 ** -7 * right.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    assert int(((d[:, -130:].double() - right).abs() > bound).sum()) == 0


def test_bf16_padded_output_rows_are_not_touched(smb, oracle, cuda_device):
    """Canary columns beyond N (ldd > N) must keep their contents: no out-of-range store."""
    torch = _torch()
    m, n, k, ldd = 300, 200, 128, 264
    a, bt, d = _run_bf16(smb, m, n, k, 2, ldd=ldd)
    assert bool(torch.isnan(d[:, n:]).all())
    _check_bf16_full(oracle, a, bt, d, n, k)


def test_bf16_8192_cubed_properties(smb, oracle, cuda_device):
    """BASELINE config 2 at full size: sampled fp64 check, constant-fill exactness (every element
    written once and only once), independence from the tile walk order."""
    torch = _torch()
    m = n = k = 8192
    a, bt, d = _run_bf16(smb, m, n, k, 5)
    rows, cols = oracle.sample_coordinates(m, n, 8192)
    ra = torch.from_numpy(rows).to(cuda_device)
    ca = torch.from_numpy(cols).to(cuda_device)
    ref = (a[ra].double() * bt[ca].double()).sum(1)
    # rms of the full product estimated from a 512 x 8192 slab in fp64.
    rms = float((a[:512].double() @ bt.double().t()).pow(2).mean().sqrt())
    bound = 2.0 ** -7 * ref.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    assert int(((d[ra, ca].double() - ref).abs() > bound).sum()) == 0
    # Same product under another raster and another cluster count: bit-identical.
    _, _, d2 = _run_bf16(smb, m, n, k, 5, group_m=5, max_clusters=37)
    assert torch.equal(d.view(torch.int16), d2.view(torch.int16))
    _, _, d3 = _run_bf16(smb, m, n, k, 3)
    assert bool((d3 == 8192.0).all())


def test_bf16_large_config_slab_of_one_rank(smb, oracle, cuda_device):
    """BASELINE config 5 as one GPU of eight sees it: M = 32768, K = 8192 and the 7168 columns of
    rank 3 (rows 21504.. of BT, generated with their global indices, fill 6 = N(0,1) x 0.05
    stand-in).  Sampled fp64 check against operands generated independently on the host for the
    sampled rows, every edge tile in full, and the constant fill (every element written once)."""
    torch = _torch()
    m, n_total, k, world, rank = 32768, 57344, 8192, 8, 3
    sh = smb.sharding.column_shard(n_total, world, rank)
    n = sh.n_local
    dev = cuda_device
    a = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
    d = torch.full((m, n), float("nan"), device=dev, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a, bt, m, n, k, 6, n0=sh.n0, n_total=n_total)
    plan = smb.gemm.Bf16Plan(a, bt, d, m, n, k)
    plan.run(); plan.check(); plan.close()
    # The slab's rows of BT are the global rows n0.. of the logical operand: compare a few with the
    # host generator (index k * N_total + n_global, seed 2).
    for local in (0, 1, 4097, n - 1):
        want = smb.gemm.fill_bf16_host(1, k, 6, 2, sh.n0 + local, 1, n_total)
        assert np.array_equal(want.reshape(-1), bt[local].view(torch.int16).cpu().numpy().view(np.uint16))
    rows, cols = oracle.sample_coordinates(m, n, 8192)
    ra = torch.from_numpy(rows).to(dev)
    ca = torch.from_numpy(cols).to(dev)
    ref = (a[ra].double() * bt[ca].double()).sum(1)
    rms = float((a[:256].double() @ bt.double().t()).pow(2).mean().sqrt())
    bound = 2.0 ** -7 * ref.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    assert int(((d[ra, ca].double() - ref).abs() > bound).sum()) == 0
    last = a[-256:].double() @ bt.double().t()
    bound = 2.0 ** -7 * last.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    assert int(((d[-256:].double() - last).abs() > bound).sum()) == 0
    right = a[:2048].double() @ bt[-256:].double().t()
    bound = 2.0 ** -7 * right.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    assert int(((d[:2048, -256:].double() - right).abs() > bound).sum()) == 0
    del a, bt, d
    _, _, d3 = _run_bf16(smb, m, n, k, 3)
    assert bool((d3 == 8192.0).all())


def test_bf16_argument_errors_on_device(smb, cuda_device):
    torch = _torch()
    t = torch.zeros(1024, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(smb.capi.SmbError) as e:
        smb.gemm.Bf16Plan(t, t, t, 16, 16, 20)        # K % 8
    assert e.value.code == smb.capi.SMB_ERR_UNSUPPORTED
    with pytest.raises(smb.capi.SmbError) as e:
        smb.gemm.Bf16Plan(t[1:], t, t, 16, 16, 16)    # misaligned A
    assert e.value.code == smb.capi.SMB_ERR_INVALID


# ------------------------------------------------------------------------------- NVFP4 GEMM
LUT = [0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6]


def _fp4_operand(smb, rows, k, fill, which, row0=0):
    torch = _torch()
    dev = torch.device("cuda:0")
    data = torch.empty(rows, k // 2, device=dev, dtype=torch.uint8)
    sfp = torch.empty(smb.gemm.sf_packed_bytes(rows, k), device=dev, dtype=torch.uint8)
    sfr = torch.empty(rows, k // 32, device=dev, dtype=torch.uint8)
    smb.gemm.fill_fp4_device(data, sfp, sfr, rows, k, fill, which, row0)
    return data, sfp, sfr


def _dequant(data, sfr):
    torch = _torch()
    lut = torch.tensor(LUT, device=data.device, dtype=torch.float64)
    lo = lut[(data & 15).long()]
    hi = lut[(data >> 4).long()]
    v = torch.stack([lo, hi], dim=-1).reshape(data.shape[0], -1)
    return v * torch.exp2(sfr.double() - 127).repeat_interleave(32, dim=1)


def _run_fp4(smb, m, n, k, fill, flags=0, fill_a=None):
    torch = _torch()
    a, sfa, sfar = _fp4_operand(smb, m, k, fill if fill_a is None else fill_a, 0)
    b, sfb, sfbr = _fp4_operand(smb, n, k, fill, 1)
    d = torch.full((m, n), float("nan"), device=a.device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, flags=flags)
    plan.run()
    plan.check()
    plan.close()
    return (a, sfar), (b, sfbr), d


def _check_fp4_full(A, B, d, k):
    torch = _torch()
    ref = _dequant(*A) @ _dequant(*B).t()
    rms = float(ref.pow(2).mean().sqrt())
    bound = 2.0 ** -7 * ref.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    got = d.double()
    bad = ~torch.isfinite(got) | ((got - ref).abs() > bound)
    assert int(bad.sum()) == 0, f"{int(bad.sum())} elements outside the north-star bound"


@pytest.mark.parametrize("overlap", ["FLAG_OPERANDS_STATIC", "FLAG_LAUNCH_INDEPENDENT"])
@pytest.mark.parametrize("store", ["FLAG_NONE", "FLAG_FORCE_PLAIN_STORE"])
def test_fp4_narrow_tile_two_ctas_per_sm(smb, cuda_device, overlap, store):
    """The 128-wide FP4 tile launched with overlapping launches allowed runs as the variant whose
    CTAs share an SM in pairs (3-stage ring, one accumulator bank, 256 tensor-memory columns):
    more tiles than cluster slots with ragged edges, then the N = 128 one-wave shape it is for,
    several launches back to back; bit-identical to the one-CTA-per-SM variant."""
    torch = _torch()
    capi = smb.capi
    for (m, n, k), tile in (((2500, 1100, 2304), capi.FLAG_TILE_N_128 | capi.FLAG_NO_DECODE),
                            ((14080, 128, 2048), 0), ((300, 100, 512), 0)):
        flags = tile | getattr(capi, store)
        A, B, d1 = _run_fp4(smb, m, n, k, 5, flags=flags)
        _check_fp4_full(A, B, d1, k)
        (a, _), (b, _) = A, B
        sfa = _fp4_operand(smb, m, k, 5, 0)[1]
        sfb = _fp4_operand(smb, n, k, 5, 1)[1]
        d2 = torch.full_like(d1, float("nan"))
        plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d2, m, n, k, flags=flags | getattr(capi, overlap))
        for _ in range(6):
            plan.run()
        plan.check()
        plan.close()
        torch.cuda.synchronize()
        assert torch.equal(d1.view(torch.int16), d2.view(torch.int16)), (m, n, k)


@pytest.mark.parametrize("fill", [1, 2, 3, 4])
def test_fp4_smoke_against_reference_golden(smb, oracle, golden, cuda_device, fill):
    """The reference's smoke case (--shape=256,256,128): output vs the reference CPU path."""
    A, B, d = _run_fp4(smb, 256, 128, 256, fill)
    got = _bits(d)
    want = golden[f"fp4_smoke_out_m{fill}"]
    ok, bad = oracle.check_verifier_nvfp4(got, oracle.bf16_to_f32(want))
    assert ok, bad
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1
    if fill in (1, 3):
        # Powers of two throughout: exact, any layout slip in the scale path shows here.
        np.testing.assert_array_equal(got, want)


def test_fp4_smoke_through_host_entry_point(smb, oracle, cuda_device):
    a_codes, a_sf = oracle.fp4_operand(256, 256, 2, 0)
    b_codes, b_sf = oracle.fp4_operand(128, 256, 2, 1)
    d = smb.gemm.dense_gemm_nvfp4_host(oracle.pack_codes(a_codes), a_sf, oracle.pack_codes(b_codes), b_sf)
    ref = oracle.gemm_f64(oracle.dequantize(a_codes, a_sf), oracle.dequantize(b_codes, b_sf))
    ok, ratio, bad = oracle.check_north_star(d, ref, 256)
    assert ok, (ratio, bad)
    ref32 = oracle.bf16_to_f32(oracle.gemm_nvfp4_reference(a_codes, a_sf, b_codes, b_sf))
    ok, bad = oracle.check_verifier_nvfp4(d, ref32)
    assert ok, bad


@pytest.mark.parametrize("shape", [
    (256, 128, 256), (512, 256, 1024), (512, 768, 1024), (512, 640, 1024), (300, 200, 96),
    (1, 1, 32), (1000, 1000, 1056), (1024, 1024, 2048), (2048, 2048, 8192),
])
@pytest.mark.parametrize("fill", [2, 5])
def test_fp4_shapes_against_fp64(smb, cuda_device, shape, fill):
    m, n, k = shape
    A, B, d = _run_fp4(smb, m, n, k, fill)
    _check_fp4_full(A, B, d, k)


@pytest.mark.parametrize("flags_name", ["FLAG_TILE_N_128", "FLAG_TILE_N_256", "FLAG_TILE_N_384",
                                        "FLAG_FORCE_PLAIN_STORE"])
@pytest.mark.parametrize("fill", [3, 4, 5])
def test_fp4_every_tile_configuration(smb, cuda_device, flags_name, fill):
    flags = getattr(smb.capi, flags_name)
    m, n, k = 768, 1088, 2112 - 2112 % 32
    A, B, d = _run_fp4(smb, m, n, k, fill, flags=flags)
    _check_fp4_full(A, B, d, k)


def test_fp4_flagship_samples_against_reference_golden(smb, oracle, golden, cuda_device):
    """The reference verifier's `flagship` case (30720 x 4096 x 8192, fill 2): its own sampled
    reference values, its own tolerance."""
    torch = _torch()
    m, k, n = (int(x) for x in golden["fp4_flagship_shape"])
    A, B, d = _run_fp4(smb, m, n, k, 2)
    rows, cols = golden["fp4_flagship_rows"], golden["fp4_flagship_cols"]
    got = d[torch.from_numpy(rows).to(d.device), torch.from_numpy(cols).to(d.device)]
    ok, bad = oracle.check_verifier_nvfp4(_bits(got), golden["fp4_flagship_ref_m2"])
    assert ok, bad


def test_fp4_8192_cubed_properties(smb, oracle, cuda_device):
    """BASELINE config 3 at full size (quantised Gaussian operands): sampled fp64 check and the
    closed form of the constant fill."""
    torch = _torch()
    m = n = k = 8192
    A, B, d = _run_fp4(smb, m, n, k, 5)
    rows, cols = oracle.sample_coordinates(m, n, 4096)
    ra = torch.from_numpy(rows).to(d.device)
    ca = torch.from_numpy(cols).to(d.device)
    da = _dequant(A[0][ra], A[1][ra])
    db = _dequant(B[0][ca], B[1][ca])
    ref = (da * db).sum(1)
    rms = float((_dequant(A[0][:256], A[1][:256]) @ _dequant(*B).t()).pow(2).mean().sqrt())
    bound = 2.0 ** -7 * ref.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    assert int(((d[ra, ca].double() - ref).abs() > bound).sum()) == 0
    _, _, d3 = _run_fp4(smb, m, n, k, 3)
    mm = torch.arange(m, device=d.device).view(-1, 1)
    nn = torch.arange(n, device=d.device).view(1, -1)
    exact = (k * torch.exp2((mm % 5) - 2.0) * torch.exp2((nn % 3) - 1.0)).to(torch.bfloat16)
    assert torch.equal(d3, exact)


# ------------------------------------------------------------------------------- NVFP4 decode shapes
def _run_fp4_decode(smb, m, n, k, fill=5, flags=0, stages=0, ctas=0, runs=1):
    """Activations: fill 6 when the weights use fill 5 (bf16-rounded Gaussian, then quantised)."""
    torch = _torch()
    a, sfa, sfar = _fp4_operand(smb, m, k, 6 if fill == 5 else fill, 0)
    b, sfb, sfbr = _fp4_operand(smb, n, k, fill, 1)
    d = torch.full((m, n), float("nan"), device=a.device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, flags=flags)
    plan.tune(stages, ctas, -1)
    outs = []
    for _ in range(runs):
        d.fill_(float("nan"))
        plan.run()
        plan.check()
        outs.append(d.clone())
    plan.close()
    return (a, sfar), (b, sfbr), outs


@pytest.mark.parametrize("m", [16, 64, 128])
def test_fp4_decode_shapes_of_the_baseline(smb, cuda_device, m):
    """BASELINE config 4: M in {16, 64, 128}, N = 28672, K = 8192, full fp64 comparison.  Run
    twice on one plan: the scratch slabs must come back to zero after every call."""
    torch = _torch()
    A, B, outs = _run_fp4_decode(smb, m, 28672, 8192, runs=2)
    _check_fp4_full(A, B, outs[0], 8192)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


@pytest.mark.parametrize("shape", [(1, 384, 256), (16, 256, 512), (100, 1000, 1056), (17, 130, 32),
                                   (128, 4096, 4096), (48, 3000, 2048)])
@pytest.mark.parametrize("fill", [2, 3, 5])
def test_fp4_decode_ragged_and_small(smb, cuda_device, shape, fill):
    m, n, k = shape
    A, B, outs = _run_fp4_decode(smb, m, n, k, fill=fill)
    _check_fp4_full(A, B, outs[0], k)


def test_fp4_decode_matches_tiled_kernel_and_any_split(smb, cuda_device):
    """The stream-K split (how many CTAs share a tile, ring depth) must not change the result
    beyond fp32 summation order: compare against the tiled kernel and against other splits."""
    torch = _torch()
    m, n, k = 16, 28672, 8192
    A, B, base = _run_fp4_decode(smb, m, n, k)
    _, _, tiled = _run_fp4_decode(smb, m, n, k, flags=smb.capi.FLAG_NO_DECODE)
    _check_fp4_full(A, B, tiled[0], k)
    for ctas, stages in ((37, 0), (100, 3), (148, 6), (1, 4)):
        _, _, other = _run_fp4_decode(smb, m, n, k, ctas=ctas, stages=stages)
        _check_fp4_full(A, B, other[0], k)
        diff = (other[0].float() - base[0].float()).abs()
        scale = base[0].float().abs().clamp_min(1.0)
        assert float((diff / scale).max()) <= 2 ** -6    # at most a couple of bf16 ulps apart


def test_fp4_decode_constant_fill_is_exact(smb, cuda_device):
    torch = _torch()
    m, n, k = 64, 28672, 8192
    _, _, outs = _run_fp4_decode(smb, m, n, k, fill=3)
    mm = torch.arange(m, device=outs[0].device).view(-1, 1)
    nn = torch.arange(n, device=outs[0].device).view(1, -1)
    exact = (k * torch.exp2((mm % 5) - 2.0) * torch.exp2((nn % 3) - 1.0)).to(torch.bfloat16)
    assert torch.equal(outs[0], exact)


# ------------------------------------------------------------------------------- hardware work queue
@pytest.mark.parametrize("shape", [(256, 128, 64), (1024, 2048, 4096), (2048, 2624, 2048), (300, 200, 72),
                                   (8192, 8192, 1024)])
def test_bf16_dynamic_tile_queue(smb, oracle, cuda_device, shape):
    """Tiles handed out by clusterlaunchcontrol.try_cancel instead of the static walk: same bits."""
    torch = _torch()
    m, n, k = shape
    a, bt, d_static = _run_bf16(smb, m, n, k, 5)
    _, _, d_dyn = _run_bf16(smb, m, n, k, 5, flags=smb.capi.FLAG_DYNAMIC_TILES)
    assert torch.equal(d_static.view(torch.int16), d_dyn.view(torch.int16))
    _check_bf16_full(oracle, a, bt, d_dyn, n, k)


@pytest.mark.parametrize("shape_flags", [((512, 768, 1024), "FLAG_TILE_N_384"), ((1024, 1024, 2048), "FLAG_TILE_N_256"),
                                         ((1024, 1024, 2048), "FLAG_TILE_N_128"), ((4096, 8192, 1024), "FLAG_NONE")])
def test_fp4_dynamic_tile_queue(smb, cuda_device, shape_flags):
    torch = _torch()
    (m, n, k), name = shape_flags
    flags = getattr(smb.capi, name)
    A, B, d_static = _run_fp4(smb, m, n, k, 5, flags=flags)
    _, _, d_dyn = _run_fp4(smb, m, n, k, 5, flags=flags | smb.capi.FLAG_DYNAMIC_TILES)
    assert torch.equal(d_static.view(torch.int16), d_dyn.view(torch.int16))
    _check_fp4_full(A, B, d_dyn, k)


@pytest.mark.parametrize("shape", [(2500, 1000, 512), (5000, 1001, 256), (100, 72, 64)])
def test_bf16_host_context_chunked_pipeline(smb, oracle, cuda_device, shape):
    """Host-buffer context (what `e2e` in bench.py times): row chunks that shrink towards the end,
    a ragged last chunk, a D whose rows need padding on the device (N = 1001), two runs on one
    context; result identical to the device-resident path."""
    torch = _torch()
    m, n, k = shape
    a, bt, d = _run_bf16(smb, m, n, k, 5)
    a_host = a.view(torch.int16).cpu().numpy().view(np.uint16)
    bt_host = bt.view(torch.int16).cpu().numpy().view(np.uint16)
    ctx = smb.gemm.Bf16HostContext(m, n, k)
    for _ in range(2):
        out = np.zeros((m, n), dtype=np.uint16)
        ctx.run(a_host, bt_host, out)
        np.testing.assert_array_equal(out, _bits(d))
    ctx.close()


def test_back_to_back_launches_with_overlap_flag(smb, oracle, cuda_device):
    """FLAG_OPERANDS_STATIC lets a launch load and multiply while the previous kernel on the stream
    is still finishing; its stores to D still wait.  Two plans sharing D, launched back to back
    many times: the last writer must win completely, every time."""
    torch = _torch()
    m, n, k = 1024, 1024, 512
    dev = torch.device("cuda:0")
    a1 = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
    a2 = torch.empty(m, k, device=dev, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=dev, dtype=torch.bfloat16)
    d = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a1, bt, m, n, k, 5)
    smb.gemm.fill_bf16_device(a2, m, k, 2, 7, 0, k, 1)
    f = smb.capi.FLAG_OPERANDS_STATIC
    p1 = smb.gemm.Bf16Plan(a1, bt, d, m, n, k, flags=f)
    p2 = smb.gemm.Bf16Plan(a2, bt, d, m, n, k, flags=f)
    for _ in range(20):
        p1.run()
        p2.run()
    p2.check()
    want2 = d.clone()
    for _ in range(20):
        p2.run()
        p1.run()
    p1.check()
    want1 = d.clone()
    ref1 = a1.double() @ bt.double().t()
    ref2 = a2.double() @ bt.double().t()
    for got, ref in ((want1, ref1), (want2, ref2)):
        bound = 2.0 ** -7 * ref.abs() + 2.0 ** -10 * (k ** 0.5) * float(ref.pow(2).mean().sqrt())
        assert int(((got.double() - ref).abs() > bound).sum()) == 0
    p1.close()
    p2.close()


# ------------------------------------------------------------------------------- BF16 activations
def test_bf16_quantizer_is_bit_identical_to_oracle(smb, oracle, cuda_device):
    torch = _torch()
    g = torch.Generator(device="cpu").manual_seed(5)
    x = (torch.randn(40, 512, generator=g) * torch.exp2(torch.randint(-6, 6, (40, 1), generator=g).float()))
    x[0, :32] = 0
    xb = x.to(torch.bfloat16).to(cuda_device)
    data = torch.empty(40, 256, device=cuda_device, dtype=torch.uint8)
    sfp = torch.empty(smb.gemm.sf_packed_bytes(40, 512), device=cuda_device, dtype=torch.uint8)
    sfr = torch.empty(40, 16, device=cuda_device, dtype=torch.uint8)
    smb.capi.check(smb.capi.lib().smb_quantize_mx_bf16_device(
        xb.data_ptr(), 512, data.data_ptr(), 256, sfp.data_ptr(), sfr.data_ptr(), 40, 512, None))
    torch.cuda.synchronize()
    codes, sf = oracle.quantize_mx(xb.float().cpu().numpy())
    np.testing.assert_array_equal(sfr.cpu().numpy(), sf)
    np.testing.assert_array_equal(data.cpu().numpy(), oracle.pack_codes(codes))
    np.testing.assert_array_equal(sfp.cpu().numpy(), oracle.sf_pack(sf))


@pytest.mark.parametrize("shape", [(16, 1024, 2048), (64, 2560, 1024), (128, 1152, 512), (7, 300, 96),
                                   (300, 512, 256), (1, 256, 8192), (16, 28672, 8192), (48, 3000, 2048),
                                   (33, 1000, 1056), (64, 38400, 512), (16, 38400, 512), (9, 1001, 352)])
@pytest.mark.parametrize("mode", ["FLAG_NONE", "FLAG_ACT_QUANT_SHARED", "FLAG_ACT_QUANT_PER_CTA", "FLAG_ACT_QUANT_CHAINED"])
def test_fp4_plan_fed_with_bf16_activations(smb, cuda_device, shape, mode):
    """The plan that takes BF16 activations equals quantise-then-multiply done as two separate
    calls, and follows the activations when they change between runs, in each of its forms: the
    default (up to 128 rows the CTAs of the decode kernel share the quantisation and meet on a
    counter; above, a quantiser kernel in front of the tiled kernel), every CTA quantising all
    activations into its own ring (up to 16 rows), and the quantiser kernel chained in front."""
    torch = _torch()
    m, n, k = shape
    g = torch.Generator(device="cpu").manual_seed(m * 7 + n)
    w, sfw, _ = _fp4_operand(smb, n, k, 5, 1)
    d = torch.empty(m, n, device=cuda_device, dtype=torch.bfloat16)
    x = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan.from_bf16_activations(x, w, sfw, d, m, n, k, flags=getattr(smb.capi, mode))
    if m <= 128:
        assert "bf16-activations" in plan.describe()
    codes = torch.empty(m, k // 2, device=cuda_device, dtype=torch.uint8)
    sfp = torch.empty(smb.gemm.sf_packed_bytes(m, k), device=cuda_device, dtype=torch.uint8)
    d_ref = torch.empty(m, n, device=cuda_device, dtype=torch.bfloat16)
    ref_plan = smb.gemm.Fp4Plan(codes, sfp, w, sfw, d_ref, m, n, k)
    for step in range(3):
        x.copy_((torch.randn(m, k, generator=g) * (0.5 + step)).to(torch.bfloat16))
        x[0, :32] = 0                      # an all-zero block: neutral scale, zero codes
        x[0, 32:36] = -0.0                 # negative zeros and values that round to zero
        x[0, 36:40] = -1e-3
        x[m - 1, k - 32:] *= 2.0 ** 20     # and a large one in the last block of the last row
        d.fill_(float("nan"))
        plan.run()
        plan.run()     # back to back: the second launch's quantiser must not disturb the first GEMM
        plan.run()
        plan.check()
        smb.capi.check(smb.capi.lib().smb_quantize_mx_bf16_device(
            x.data_ptr(), k, codes.data_ptr(), k // 2, sfp.data_ptr(), None, m, k, None))
        ref_plan.run()
        ref_plan.check()
        assert torch.equal(d.view(torch.int16), d_ref.view(torch.int16)), f"step {step}"
    if m <= 16:
        # A ring shallower than the number of quantising warps: only as many warps as ring slots
        # may take part (a warp further ahead would pass a parity wait two phases early).
        for depth in (2, 3):
            plan.tune(depth, 0, -1)
            d.fill_(float("nan"))
            plan.run(); plan.run(); plan.check()
            assert torch.equal(d.view(torch.int16), d_ref.view(torch.int16)), f"ring depth {depth}"
    plan.close()
    ref_plan.close()


@pytest.mark.parametrize("kind", ["bf16", "fp4"])
def test_independent_launches_run_side_by_side(smb, oracle, cuda_device, kind):
    """FLAG_LAUNCH_INDEPENDENT: no launch waits for the previous one (the reference kernels'
    behaviour).  Small one-wave GEMMs into two different outputs, launched alternately many times
    without a pause: both outputs must be complete and right at the end."""
    torch = _torch()
    f = smb.capi.FLAG_LAUNCH_INDEPENDENT
    m, n, k = 2048, 256, 1024
    outs = [torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16) for _ in range(2)]
    if kind == "bf16":
        a = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=cuda_device, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt, m, n, k, 5)
        plans = [smb.gemm.Bf16Plan(a, bt, d, m, n, k, flags=f) for d in outs]
    else:
        a, sfa, sfar = _fp4_operand(smb, m, k, 5, 0)
        b, sfb, sfbr = _fp4_operand(smb, n, k, 5, 1)
        plans = [smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, flags=f) for d in outs]
    for _ in range(25):
        for p in plans:
            p.run()
    for p in plans:
        p.check()
    for d in outs:
        if kind == "bf16":
            _check_bf16_full(oracle, a, bt, d, n, k)
        else:
            _check_fp4_full((a, sfar), (b, sfbr), d, k)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    for p in plans:
        p.close()


# ------------------------------------------------------------------------------- gated epilogue
def _check_swiglu(oracle, acc64, d, k):
    ref = oracle.swiglu(acc64)
    bound = oracle.swiglu_bound(acc64, k)
    got = d.double().cpu().numpy()
    assert got.shape == ref.shape
    bad = ~np.isfinite(got) | (np.abs(got - ref) > bound)
    assert int(bad.sum()) == 0, f"{int(bad.sum())} of {bad.size} outside the bound; worst {np.max(np.abs(got - ref) / bound):.2f}"


@pytest.mark.parametrize("shape_flags", [((512, 512, 256), "FLAG_NONE"), ((1024, 1024, 512), "FLAG_TILE_N_512"),
                                         ((300, 200, 72), "FLAG_NONE"), ((2048, 4096, 1024), "FLAG_NONE"),
                                         ((256, 66, 64), "FLAG_TILE_N_256")])
def test_bf16_gated_epilogue(smb, oracle, cuda_device, shape_flags):
    """FLAG_EPILOGUE_SWIGLU: D[m, n] = bf16(silu(acc[m, 2n+1]) * acc[m, 2n]) against the float64
    definition; D is [M, N/2] with a padded pitch, nothing outside it is written."""
    torch = _torch()
    (m, n, k), name = shape_flags
    a = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=cuda_device, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a, bt, m, n, k, 7)          # N(0,1): gates of both signs, |z| up to ~30
    n_out = n // 2
    ldd = (n_out + 7) // 8 * 8 + 8
    d = torch.full((m, ldd), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    flags = smb.capi.FLAG_EPILOGUE_SWIGLU | getattr(smb.capi, name)
    plan = smb.gemm.Bf16Plan(a, bt, d, m, n, k, ldd=ldd, flags=flags)
    plan.run(); plan.run(); plan.check(); plan.close()
    acc = (a.double() @ bt.double().t()).cpu().numpy()
    _check_swiglu(oracle, acc, d[:, :n_out], k)
    # The aligned store path writes whole 16-byte chunks: the padding of a row may be overwritten
    # up to the next multiple of 8 columns, nothing beyond that.
    assert bool(torch.isnan(d[:, (n_out + 7) // 8 * 8:]).all())


def test_fp4_gated_epilogue(smb, oracle, cuda_device):
    torch = _torch()
    m, n, k = 768, 1024, 512
    a, sfa, sfar = _fp4_operand(smb, m, k, 5, 0)
    b, sfb, sfbr = _fp4_operand(smb, n, k, 5, 1)
    d = torch.full((m, n // 2), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, ldd=n // 2, flags=smb.capi.FLAG_EPILOGUE_SWIGLU)
    plan.run(); plan.check(); plan.close()
    acc = (_dequant(a, sfar) @ _dequant(b, sfbr).t()).cpu().numpy()
    _check_swiglu(oracle, acc, d, k)


def test_gated_epilogue_is_refused_where_it_cannot_work(smb, cuda_device):
    torch = _torch()
    capi = smb.capi
    a = torch.zeros(256, 64, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.zeros(130, 64, device=cuda_device, dtype=torch.bfloat16)
    d = torch.zeros(256, 72, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(capi.SmbError):       # odd N
        smb.gemm.Bf16Plan(a, bt, d, 256, 129, 64, ldd=72, flags=capi.FLAG_EPILOGUE_SWIGLU)
    with pytest.raises(capi.SmbError):       # pitch not a multiple of 8 elements
        smb.gemm.Bf16Plan(a, bt, d, 256, 130, 64, ldd=70, flags=capi.FLAG_EPILOGUE_SWIGLU)
    with pytest.raises(capi.SmbError):       # pitch shorter than N/2
        smb.gemm.Bf16Plan(a, bt, d, 256, 130, 64, ldd=64, flags=capi.FLAG_EPILOGUE_SWIGLU)
    xa, xsfa, _ = _fp4_operand(smb, 16, 256, 6, 0)
    w, wsf, _ = _fp4_operand(smb, 256, 256, 5, 1)
    dd = torch.zeros(16, 128, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(capi.SmbError):       # the decode kernel's single-tile form has no gated epilogue
        smb.gemm.Fp4Plan(xa, xsfa, w, wsf, dd, 16, 256, 256, ldd=128,
                         flags=capi.FLAG_EPILOGUE_SWIGLU | capi.FLAG_DECODE_SINGLE)
    plan = smb.gemm.Fp4Plan(xa, xsfa, w, wsf, dd, 16, 256, 256, ldd=128, flags=capi.FLAG_EPILOGUE_SWIGLU)
    plan.tune(0, 4, -1)                      # ... nor do its stream-K ranges (a forced CTA count)
    with pytest.raises(capi.SmbError):
        plan.run()
    plan.close()


@pytest.mark.parametrize("form", ["FLAG_DECODE_DUAL", "FLAG_DECODE_SINGLE"])
@pytest.mark.parametrize("shape", [(16, 256, 512), (1, 384, 256), (100, 1100, 1056), (128, 4096, 4096),
                                   (64, 28672, 8192), (33, 130, 96), (128, 28672 + 128, 2048), (128, 300 * 128, 512)])
def test_fp4_decode_both_forms(smb, cuda_device, shape, form):
    """The two forms of the decode kernel (one weight tile per activation box; two adjacent weight
    tiles sharing it) on the same shapes: even and odd tile counts, more tile pairs than SMs,
    ragged M and N, several K; two runs per plan, bit-identical."""
    torch = _torch()
    m, n, k = shape
    A, B, outs = _run_fp4_decode(smb, m, n, k, flags=getattr(smb.capi, form), runs=2)
    _check_fp4_full(A, B, outs[0], k)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


def test_fp4_decode_forms_agree_bit_for_bit(smb, cuda_device):
    """Whole tiles in both forms: the same fp32 accumulation order, so the same bits."""
    torch = _torch()
    for m in (16, 128):
        _, _, single = _run_fp4_decode(smb, m, 28672, 8192, flags=smb.capi.FLAG_DECODE_SINGLE)
        _, _, dual = _run_fp4_decode(smb, m, 28672, 8192, flags=smb.capi.FLAG_DECODE_DUAL)
        assert torch.equal(single[0].view(torch.int16), dual[0].view(torch.int16))
        # The default choice: above 64 rows the dual kernel's wide form (activations as the rows of
        # the instruction, both weight tiles as its 256 columns), same sums in the same order.
        _, _, chosen = _run_fp4_decode(smb, m, 28672, 8192)
        assert torch.equal(single[0].view(torch.int16), chosen[0].view(torch.int16))


@pytest.mark.parametrize("shape", [(65, 640, 512), (100, 28672 + 128, 1024), (128, 37888, 512),
                                   (128, 37888 + 256, 512), (77, 1001, 768), (128, 128, 256), (113, 2000, 8192)])
def test_fp4_decode_wide_form_edges(smb, cuda_device, shape):
    """The wide decode form at its edges: ragged M above 64, an odd number of weight tiles, N not a
    multiple of 128, a D pitch that rules out TMA stores (N = 1001), the largest N it takes (one
    tile pair per SM) and the first N beyond it (which falls back to the swapped form): inside the
    north-star bound of the float64 product, bit-identical to the single-tile form, two runs."""
    torch = _torch()
    m, n, k = shape
    A, B, outs = _run_fp4_decode(smb, m, n, k, runs=2)
    _check_fp4_full(A, B, outs[0], k)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    _, _, single = _run_fp4_decode(smb, m, n, k, flags=smb.capi.FLAG_DECODE_SINGLE)
    assert torch.equal(single[0].view(torch.int16), outs[0].view(torch.int16))


# ------------------------------------------------------------------------------- NVFP4 proper
def _nvf4_operand(smb, oracle, rows, k, seed, sigma=1.0):
    """Gaussian data quantised on the device to E2M1 + E4M3 scale per 16 K; returns device buffers
    (codes, packed scales), the global scale and the represented values in float64."""
    torch = _torch()
    import ctypes as C
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = (torch.randn(rows, k, generator=g) * sigma).to(dev)
    gs = 448.0 * 6.0 / float(x.abs().max())
    codes = torch.empty(rows, k // 2, device=dev, dtype=torch.uint8)
    sfp = torch.empty(smb.gemm.sf_packed_bytes(rows, k * 2), device=dev, dtype=torch.uint8)   # K/16 blocks
    sfr = torch.empty(rows, k // 16, device=dev, dtype=torch.uint8)
    smb.capi.check(smb.capi.lib().smb_quantize_nvf4_device(
        x.data_ptr(), k, C.c_float(gs), codes.data_ptr(), k // 2, sfp.data_ptr(), sfr.data_ptr(), rows, k, None))
    torch.cuda.synchronize()
    want_codes, want_sb = oracle.quantize_nvf4(x.cpu().numpy(), gs)
    np.testing.assert_array_equal(sfr.cpu().numpy(), want_sb)
    np.testing.assert_array_equal(codes.cpu().numpy(), oracle.pack_codes(want_codes))
    np.testing.assert_array_equal(sfp.cpu().numpy(), oracle.sf_pack(want_sb, pad=0))
    values = oracle.dequantize_nvf4(want_codes, want_sb, gs)
    return codes, sfp, gs, values


@pytest.mark.parametrize("shape", [(256, 256, 256), (512, 768, 1024), (300, 200, 192), (64, 1024, 512),
                                   (2048, 2048, 4096), (16, 4096, 2048), (128, 2304, 1024), (100, 1100, 192),
                                   (1, 128, 64)])
def test_nvf4_block16_gemm(smb, oracle, cuda_device, shape):
    """NVFP4 proper (E4M3 scale per 16 K, scale_vec::4X, per-tensor factors folded into alpha):
    device quantiser bit-identical to the oracle, GEMM within the north-star bound of the float64
    product of the represented values."""
    torch = _torch()
    m, n, k = shape
    a, sfa, gsa, va = _nvf4_operand(smb, oracle, m, k, 3)
    b, sfb, gsb, vb = _nvf4_operand(smb, oracle, n, k, 4, sigma=0.05)
    d = torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, flags=smb.capi.FLAG_SCALE_BLOCK16)
    plan.set_alpha(1.0 / (gsa * gsb))
    plan.run(); plan.run(); plan.check(); plan.close()
    ref = va @ vb.T
    ok, worst, bad = oracle.check_north_star(_bits(d), ref, k)
    assert ok, f"{bad} elements outside the bound, worst ratio {worst:.2f}"


def test_nvf4_block16_is_refused_where_it_cannot_work(smb, cuda_device):
    torch = _torch()
    t = torch.zeros(1 << 16, device=cuda_device, dtype=torch.uint8)
    d = torch.zeros(256, 256, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(smb.capi.SmbError):     # K % 64 != 0
        smb.gemm.Fp4Plan(t, t, t, t, d, 256, 256, 96, flags=smb.capi.FLAG_SCALE_BLOCK16)
    with pytest.raises(smb.capi.SmbError):     # no gated epilogue for this variant
        smb.gemm.Fp4Plan(t, t, t, t, d, 256, 256, 128, ldd=128,
                         flags=smb.capi.FLAG_SCALE_BLOCK16 | smb.capi.FLAG_EPILOGUE_SWIGLU)
    plain = smb.gemm.Fp4Plan(t, t, t, t, d, 256, 256, 128)
    with pytest.raises(smb.capi.SmbError):     # alpha belongs to block-16 plans
        plain.set_alpha(0.5)
    plain.close()


# ------------------------------------------------------------------------------- grouped GEMM
@pytest.mark.parametrize("case", [((512, 256, 0, 768), 384, 256, "FLAG_NONE"),
                                  ((256, 256, 256, 256, 512, 1024, 256, 256), 1000, 512, "FLAG_NONE"),
                                  ((2048, 4096), 2048, 1024, "FLAG_TILE_N_512"),
                                  ((256, 512), 130, 64, "FLAG_TILE_N_128")])
def test_bf16_grouped_gemm(smb, oracle, cuda_device, case):
    """Mixture-of-experts form: rows of A sorted by group (each padded to 256 rows), one BT per
    group; every row block must meet its own group's weights."""
    torch = _torch()
    rows, n, k, name = case
    groups = len(rows)
    m_total = sum(rows)
    a = torch.empty(m_total, k, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.empty(groups * n, k, device=cuda_device, dtype=torch.bfloat16)
    smb.gemm.fill_bf16_device(a, m_total, k, 5, 1, 0, k, 1)
    smb.gemm.fill_bf16_device(bt, groups * n, k, 5, 2, 0, k, 1)
    tile_group = torch.tensor([g for g, r in enumerate(rows) for _ in range(r // 256)], device=cuda_device,
                              dtype=torch.int32)
    d = torch.full((m_total, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Bf16Plan.grouped(a, bt, d, m_total, n, k, groups, tile_group, flags=getattr(smb.capi, name))
    plan.run(); plan.run(); plan.check(); plan.close()
    row0 = 0
    for g, r in enumerate(rows):
        if r:
            _check_bf16_full(oracle, a[row0:row0 + r], bt[g * n:(g + 1) * n], d[row0:row0 + r], n, k)
        row0 += r
    lib = smb.capi.lib()
    assert lib.smb_bf16_grouped_plan_create(None, None, None, None, 300, 128, 64, 1, None, 0) == smb.capi.SMB_ERR_INVALID


@pytest.mark.parametrize("case", [((512, 0, 256, 768), 384, 512, "FLAG_NONE"), ((256, 1024), 1024, 1024, "FLAG_TILE_N_256"),
                                  ((256, 256, 512), 128, 256, "FLAG_NONE")])
def test_fp4_grouped_gemm(smb, cuda_device, case):
    """FP4 twin of the grouped BF16 test: B and its scales stacked over the groups."""
    torch = _torch()
    rows, n, k, name = case
    groups, m_total = len(rows), sum(rows)
    a, sfa, sfar = _fp4_operand(smb, m_total, k, 5, 0)
    b, sfb, sfbr = _fp4_operand(smb, groups * n, k, 5, 1)
    tile_group = torch.tensor([g for g, r in enumerate(rows) for _ in range(r // 256)], device=cuda_device,
                              dtype=torch.int32)
    d = torch.full((m_total, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan.grouped(a, sfa, b, sfb, d, m_total, n, k, groups, tile_group,
                                    flags=getattr(smb.capi, name))
    plan.run(); plan.check(); plan.close()
    row0 = 0
    for g, r in enumerate(rows):
        if r:
            _check_fp4_full((a[row0:row0 + r], sfar[row0:row0 + r]), (b[g * n:(g + 1) * n], sfbr[g * n:(g + 1) * n]),
                            d[row0:row0 + r], k)
        row0 += r
    with pytest.raises(smb.capi.SmbError):     # N must keep the scale bands of the groups apart
        smb.gemm.Fp4Plan.grouped(a, sfa, b, sfb, d, m_total, 200, k, groups, tile_group)


@pytest.mark.parametrize("case", [((300, 0, 77, 512, 1), 384, 256, "FLAG_NONE"),
                                  ((1000, 1), 1000, 512, "FLAG_NONE"),
                                  ((33, 2047, 700), 2048, 1024, "FLAG_TILE_N_512"),
                                  ((5, 250), 130, 64, "FLAG_TILE_N_128"),
                                  ((100, 260, 31), 264, 128, "FLAG_FORCE_PLAIN_STORE")])
def test_bf16_grouped_gemm_with_ragged_groups(smb, oracle, cuda_device, case):
    """Groups of any row count (no padding): the plan cuts every group into row tiles of its own;
    the last tile of a group reads on into the next group's rows and must store only its own.
    Every row of D is checked against its own group's weights, and rows are written exactly once
    (a constant fill comes back exact, canary rows after the last group stay untouched)."""
    torch = _torch()
    rows, n, k, name = case
    groups, m_total = len(rows), sum(rows)
    offsets = [0]
    for r in rows:
        offsets.append(offsets[-1] + r)
    a = torch.empty(m_total, k, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.empty(groups * n, k, device=cuda_device, dtype=torch.bfloat16)
    smb.gemm.fill_bf16_device(a, m_total, k, 5, 1, 0, k, 1)
    smb.gemm.fill_bf16_device(bt, groups * n, k, 5, 2, 0, k, 1)
    d_all = torch.full((m_total + 40, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    d = d_all[:m_total]
    plan = smb.gemm.Bf16Plan.grouped_offsets(a, bt, d, n, k, offsets, flags=getattr(smb.capi, name))
    plan.run(); plan.run(); plan.check(); plan.close()
    for g, r in enumerate(rows):
        if r:
            lo = offsets[g]
            _check_bf16_full(oracle, a[lo:lo + r], bt[g * n:(g + 1) * n], d[lo:lo + r], n, k)
    assert bool(torch.isnan(d_all[m_total:].float()).all()), "rows beyond the last group were written"
    lib = smb.capi.lib()
    import ctypes as C
    bad = (C.c_int * 3)(0, 10, 5)
    h = C.c_void_p()
    assert lib.smb_bf16_grouped_plan_create_offsets(C.byref(h), a.data_ptr(), bt.data_ptr(), d.data_ptr(), n, k, 2,
                                                    bad, 0) == smb.capi.SMB_ERR_INVALID


@pytest.mark.parametrize("case", [((384, 0, 128, 640), 384, 512, "FLAG_NONE"), ((128, 1152), 1024, 1024, "FLAG_TILE_N_256"),
                                  ((128, 128, 384), 1280, 256, "FLAG_TILE_N_384")])
def test_fp4_grouped_gemm_with_groups_of_128_rows(smb, cuda_device, case):
    """FP4 twin: groups start on multiples of 128 rows (the scale bands of A), need not fill
    256-row tiles."""
    torch = _torch()
    rows, n, k, name = case
    groups, m_total = len(rows), sum(rows)
    offsets = [0]
    for r in rows:
        offsets.append(offsets[-1] + r)
    a, sfa, sfar = _fp4_operand(smb, m_total, k, 5, 0)
    b, sfb, sfbr = _fp4_operand(smb, groups * n, k, 5, 1)
    d_all = torch.full((m_total + 40, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    d = d_all[:m_total]
    plan = smb.gemm.Fp4Plan.grouped_offsets(a, sfa, b, sfb, d, n, k, offsets, flags=getattr(smb.capi, name))
    plan.run(); plan.check(); plan.close()
    for g, r in enumerate(rows):
        if r:
            lo = offsets[g]
            _check_fp4_full((a[lo:lo + r], sfar[lo:lo + r]), (b[g * n:(g + 1) * n], sfbr[g * n:(g + 1) * n]),
                            d[lo:lo + r], k)
    assert bool(torch.isnan(d_all[m_total:].float()).all()), "rows beyond the last group were written"
    with pytest.raises(smb.capi.SmbError):     # a group that starts inside a scale band
        smb.gemm.Fp4Plan.grouped_offsets(a, sfa, b, sfb, d, n, k, [0, 100, m_total])


# ------------------------------------------------------------------------------- bounded waits
@pytest.mark.parametrize("kind", ["bf16", "fp4"])
def test_bounded_wait_probe_reports_and_recovers(smb, oracle, cuda_device, kind):
    """A wait that runs out of budget comes back as SMB_ERR_DEVICE through the plan's status word,
    the word is cleared by the check, and the same plan on the same stream then works.  The probe
    kernel waits about 100 us on an mbarrier nobody arrives at and returns normally: nothing
    faults, traps or hangs."""
    torch = _torch()
    m, n, k = 512, 512, 512
    if kind == "bf16":
        a = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=cuda_device, dtype=torch.bfloat16)
        d = torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt, m, n, k, 5)
        plan = smb.gemm.Bf16Plan(a, bt, d, m, n, k)
    else:
        a, sfa, sfar = _fp4_operand(smb, m, k, 5, 0)
        b, sfb, sfbr = _fp4_operand(smb, n, k, 5, 1)
        d = torch.full((m, n), float("nan"), device=cuda_device, dtype=torch.bfloat16)
        plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k)
    plan.run()
    plan.check()
    plan.wait_probe(200_000)
    with pytest.raises(smb.capi.SmbError) as err:
        plan.check()
    assert err.value.code == smb.capi.SMB_ERR_DEVICE
    assert "status 107" in err.value.message and "bounded-wait probe" in err.value.message
    plan.check()                      # the word was cleared: no stale error
    d.fill_(float("nan"))
    plan.run()                        # and the context, stream and plan still work
    plan.check()
    if kind == "bf16":
        _check_bf16_full(oracle, a, bt, d, n, k)
    else:
        _check_fp4_full((a, sfar), (b, sfbr), d, k)
    # Budgets outside 1 .. 2 000 000 cycles are refused on the host.
    lib = smb.capi.lib()
    fn = lib.smb_bf16_plan_wait_probe if kind == "bf16" else lib.smb_fp4_plan_wait_probe
    assert fn(plan._h, 0, None) == smb.capi.SMB_ERR_INVALID
    assert fn(plan._h, 10 ** 9, None) == smb.capi.SMB_ERR_INVALID
    plan.close()


# ------------------------------------------------------------------------------- FP4 host context
@pytest.mark.parametrize("shape", [(2500, 1000, 512), (300, 520, 256), (100, 1024, 1024), (16, 4096, 2048)])
def test_fp4_host_context(smb, cuda_device, shape):
    """Host-buffer FP4 context (what the FP4 `e2e` figures of bench.py time): codes and row-major
    scales go up, scales are packed on the device, row chunks pipeline, D comes back.  Identical
    to the device-resident plan; a second run that keeps the weights on the device agrees too."""
    torch = _torch()
    m, n, k = shape
    A, B, d = _run_fp4(smb, m, n, k, 5, fill_a=6)
    a_host, sfa_host = A[0].cpu().numpy(), A[1].cpu().numpy()
    b_host, sfb_host = B[0].cpu().numpy(), B[1].cpu().numpy()
    ctx = smb.gemm.Fp4HostContext(m, n, k)
    with pytest.raises(smb.capi.SmbError):
        ctx.run(a_host, sfa_host, None, None, np.zeros((m, n), dtype=np.uint16))   # no weights yet
    out = np.zeros((m, n), dtype=np.uint16)
    ctx.run(a_host, sfa_host, b_host, sfb_host, out)
    np.testing.assert_array_equal(out, _bits(d))
    out2 = np.zeros((m, n), dtype=np.uint16)
    ctx.run(a_host, sfa_host, None, None, out2)
    np.testing.assert_array_equal(out2, _bits(d))
    ctx.close()
    _check_fp4_full(A, B, d, k)


# ------------------------------------------------------------------------------- stream-K walk (BF16)
@pytest.mark.parametrize("case", [((512, 1024, 4096), 3), ((256, 512, 8192), 5), ((1000, 1104, 2080), 7),
                                   ((2048, 2048, 1024), 0), ((8192, 1024, 8192), 0), ((300, 600, 1024), 74)])
def test_bf16_stream_k_walk(smb, oracle, cuda_device, case):
    """K loops of the 256 x 512 tiles cut where the clusters' shares end: tiles split over two
    clusters, a tile split over five, whole tiles in between, ragged edges, more clusters than
    tiles; three launches in a row on one plan (the flags carry the launch number); full fp64
    check, within bf16 rounding of the whole-tile kernel, padding columns untouched."""
    torch = _torch()
    (m, n, k), clusters = case
    ldd = n + 24
    a = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.empty(n, k, device=cuda_device, dtype=torch.bfloat16)
    smb.gemm.bf16_operands_device(a, bt, m, n, k, 5)
    d = torch.full((m, ldd), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Bf16Plan(a, bt, d, m, n, k, ldd=ldd, flags=smb.capi.FLAG_STREAM_K)
    plan.tune(0, clusters)
    assert plan.describe().endswith("stream-k")
    for _ in range(3):
        d[:, :n] = float("nan")
        plan.run()
        plan.check()
        assert bool(torch.isnan(d[:, n:].float()).all()), "padding columns were written"
        _check_bf16_full(oracle, a, bt, d, n, k)
    plan.close()
    d2 = torch.empty((m, n), device=cuda_device, dtype=torch.bfloat16)
    whole = smb.gemm.Bf16Plan(a, bt, d2, m, n, k, flags=smb.capi.FLAG_TILE_N_512)
    whole.run()
    whole.check()
    assert not whole.describe().endswith("stream-k")
    whole.close()
    diff = (d[:, :n].float() - d2.float()).abs()
    assert float((diff / d2.float().abs().clamp_min(1e-3)).max()) <= 2.0 ** -6   # a bf16 rounding step or two


def test_bf16_stream_k_is_refused_where_it_has_no_form(smb, cuda_device):
    torch = _torch()
    a = torch.empty(1024, 4096, device=cuda_device, dtype=torch.bfloat16)
    bt = torch.empty(256, 4096, device=cuda_device, dtype=torch.bfloat16)
    d = torch.empty(1024, 256, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(smb.capi.SmbError):
        smb.gemm.Bf16Plan(a, bt, d, 1024, 256, 4096, flags=smb.capi.FLAG_STREAM_K)
    bt = torch.empty(1024, 4096, device=cuda_device, dtype=torch.bfloat16)
    d = torch.empty(1024, 1024 + 3, device=cuda_device, dtype=torch.bfloat16)
    with pytest.raises(smb.capi.SmbError):
        smb.gemm.Bf16Plan(a, bt, d, 1024, 1024, 4096, ldd=1027, flags=smb.capi.FLAG_STREAM_K)
    # Left to itself the plan keeps whole tiles for the column shards of 8192^3.
    d = torch.empty(1024, 1024, device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Bf16Plan(a, bt, d, 1024, 1024, 4096)
    assert not plan.describe().endswith("stream-k")
    plan.close()


# ------------------------------------------------------------------------------- A-resident schedule
@pytest.mark.parametrize("shape", [(512, 768, 512), (300, 400, 96), (1000, 1000, 1056), (2048, 2304, 2048),
                                   (4096, 5120, 2048), (256, 1920, 256)])
@pytest.mark.parametrize("clusters", [0, 3])
@pytest.mark.parametrize("store", ["FLAG_NONE", "FLAG_FORCE_PLAIN_STORE"])
def test_fp4_a_resident_schedule(smb, cuda_device, shape, clusters, store):
    """The short-K kernel (A panel loaded once per run of 192-column tiles, two accumulator sets):
    ragged M, N and K, odd tiles (whose B scales start half a band in), several runs per cluster
    (the A slots are handed over between runs), more and fewer runs than clusters, both store
    paths; full fp64 check, exact constant fill, padding columns of D untouched, and the same
    bits as the general kernel."""
    torch = _torch()
    m, n, k = shape
    ldd = n + (24 if store == "FLAG_NONE" else 3)
    flags = smb.capi.FLAG_TILE_N_192 | smb.capi.FLAG_NO_DECODE | getattr(smb.capi, store)
    for fill in (5, 3):
        a, sfa, sfar = _fp4_operand(smb, m, k, fill, 0)
        b, sfb, sfbr = _fp4_operand(smb, n, k, fill, 1)
        d = torch.full((m, ldd), float("nan"), device=cuda_device, dtype=torch.bfloat16)
        plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, ldd=ldd, flags=flags)
        if clusters:
            plan.tune(0, clusters, -1)
        assert plan.describe().endswith("a-resident")
        plan.run()
        plan.run()
        plan.check()
        plan.close()
        assert bool(torch.isnan(d[:, n:].float()).all()), "padding columns were written"
        if fill == 5:
            _check_fp4_full((a, sfar), (b, sfbr), d[:, :n].contiguous(), k)
            d2 = torch.empty((m, n), device=cuda_device, dtype=torch.bfloat16)
            other = smb.gemm.Fp4Plan(a, sfa, b, sfb, d2, m, n, k, flags=smb.capi.FLAG_TILE_N_256 | smb.capi.FLAG_NO_DECODE)
            other.run()
            other.check()
            other.close()
            assert torch.equal(d[:, :n], d2)
        else:
            mm = torch.arange(m, device=d.device).view(-1, 1)
            nn = torch.arange(n, device=d.device).view(1, -1)
            exact = (k * torch.exp2((mm % 5) - 2.0) * torch.exp2((nn % 3) - 1.0)).to(torch.bfloat16)
            assert torch.equal(d[:, :n], exact)


def test_fp4_a_resident_schedule_refuses_what_it_has_no_form_for(smb, cuda_device):
    torch = _torch()
    for (m, n, k), extra in (((512, 768, 4096), 0), ((512, 256, 512), 0), ((512, 768, 512), smb.capi.FLAG_SCALE_BLOCK16)):
        a, sfa, _ = _fp4_operand(smb, m, k, 5, 0)
        b, sfb, _ = _fp4_operand(smb, n, k, 5, 1)
        d = torch.empty((m, n), device=cuda_device, dtype=torch.bfloat16)
        with pytest.raises(smb.capi.SmbError):
            smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, flags=smb.capi.FLAG_TILE_N_192 | smb.capi.FLAG_NO_DECODE | extra)


# ------------------------------------------------------------------------------- mixed tile widths
@pytest.mark.parametrize("shape", [(1024, 1280, 1024), (2048, 2432, 1024), (1024, 2304, 1024), (512, 1000, 288),
                                   (8192, 8192, 256)])
@pytest.mark.parametrize("clusters", [0, 7, 3])
def test_fp4_full_and_narrow_tiles_in_one_launch(smb, cuda_device, shape, clusters):
    """The 256 x 384 kernel ends its tile list with 256-wide tiles where that evens the clusters
    out; which tiles are narrow depends on the shape and on the number of clusters.  Whatever the
    split: full fp64 check, exact constant fill (every element written exactly once, no narrow
    tile spills into its neighbour's columns), padding columns of D untouched."""
    torch = _torch()
    lib = smb.capi.lib()
    m, n, k = shape
    import ctypes as C
    wide, narrow = C.c_int(), C.c_int()
    lib.smb_debug_fp4_phases(m, n, k, clusters or 74, C.byref(wide), C.byref(narrow))
    ldd = n + 24
    for fill in (5, 3):
        a, sfa, sfar = _fp4_operand(smb, m, k, fill, 0)
        b, sfb, sfbr = _fp4_operand(smb, n, k, fill, 1)
        d = torch.full((m, ldd), float("nan"), device=cuda_device, dtype=torch.bfloat16)
        plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, ldd=ldd,
                                flags=smb.capi.FLAG_TILE_N_384 | smb.capi.FLAG_NO_DECODE)
        plan.tune(0, clusters, -1)
        assert plan.describe().startswith("fp4 tile 256x384")
        plan.run()
        plan.check()
        plan.close()
        assert bool(torch.isnan(d[:, n:].float()).all()), "padding columns were written"
        if fill == 5:
            _check_fp4_full((a, sfar), (b, sfbr), d[:, :n].contiguous(), k)
        else:
            mm = torch.arange(m, device=d.device).view(-1, 1)
            nn = torch.arange(n, device=d.device).view(1, -1)
            exact = (k * torch.exp2((mm % 5) - 2.0) * torch.exp2((nn % 3) - 1.0)).to(torch.bfloat16)
            assert torch.equal(d[:, :n], exact)
    if shape in ((1024, 1280, 1024), (2048, 2432, 1024)):
        assert narrow.value == 2      # these shapes do get narrow tiles (2 or 5 full ones before them)
    if shape == (1024, 2304, 1024):
        assert (wide.value, narrow.value) == ((4, 3) if clusters == 0 else (6, 0))


# ------------------------------------------------------------------------------- every configuration under the verifiers' rule
def _verifier_mismatches(observed_bits, reference, atol, rtol):
    """The mismatch rule of the reference verifiers' verify() (dense_gemm_bf16_cpu_verifier.py:82-83,
    nvfp4/dense_gemm_nvfp4_cpu_verifier.py:119-122): not finite, or off by more than atol AND by more
    than rtol |reference|."""
    observed = (observed_bits.astype(np.uint32) << 16).view(np.float32)
    error = np.abs(observed - reference)
    return int(np.count_nonzero(~np.isfinite(observed) | ((error > atol) & (error > rtol * np.abs(reference)))))


@pytest.mark.parametrize("name", ["bf16_8192", "bf16_ragged", "bf16_large"])
def test_bf16_configurations_under_the_reference_verifier_rule(smb, golden, cuda_device, name):
    """Each BF16 benchmark configuration once with the reference's fill 2: the CUDA output at the
    verifier's own sample coordinates against the verifier's own reference values (made by its
    code with CASES extended at run time), under its own tolerance."""
    torch = _torch()
    m, k, n = (int(x) for x in golden[f"cfg_{name}_shape"])
    a, bt, d = _run_bf16(smb, m, n, k, 2)
    rows = torch.from_numpy(golden[f"cfg_{name}_rows"]).to(d.device)
    cols = torch.from_numpy(golden[f"cfg_{name}_cols"]).to(d.device)
    atol, rtol = golden["cfg_tolerances"][:2]
    assert _verifier_mismatches(_bits(d[rows, cols]), golden[f"cfg_{name}_ref_m2"], atol, rtol) == 0
    del a, bt, d
    torch.cuda.empty_cache()


@pytest.mark.parametrize("name", ["nvfp4_8192", "decode_m16", "decode_m64", "decode_m128"])
def test_fp4_configurations_under_the_reference_verifier_rule(smb, golden, cuda_device, name):
    torch = _torch()
    m, k, n = (int(x) for x in golden[f"cfg_{name}_shape"])
    A, B, d = _run_fp4(smb, m, n, k, 2)
    rows = torch.from_numpy(golden[f"cfg_{name}_rows"]).to(d.device)
    cols = torch.from_numpy(golden[f"cfg_{name}_cols"]).to(d.device)
    atol, rtol = golden["cfg_tolerances"][2:]
    assert _verifier_mismatches(_bits(d[rows, cols]), golden[f"cfg_{name}_ref_m2"], atol, rtol) == 0


# ------------------------------------------------------------------------------- gated epilogue, wider coverage
def _check_swiglu_torch(acc64, d, k):
    """silu(gate) * up in float64 on the exact accumulators, with the bound of the tiled kernels'
    gated-epilogue test: the north-star bound on each accumulator carried through the activation."""
    torch = _torch()
    up, gate = acc64[:, 0::2], acc64[:, 1::2]
    want = gate / (1.0 + torch.exp(-gate)) * up
    rms = float(acc64.pow(2).mean().sqrt())
    eps_acc = 2.0 ** -7 * acc64.abs() + 2.0 ** -10 * (k ** 0.5) * rms
    eps_up, eps_gate = eps_acc[:, 0::2], eps_acc[:, 1::2] + 2.0 ** -10 * gate.abs() + 2.0 ** -9
    silu = gate / (1.0 + torch.exp(-gate))
    bound = 2.0 ** -7 * want.abs() + 1.1 * up.abs() * eps_gate + silu.abs() * eps_up + 1e-6
    got = d.double()
    bad = ~torch.isfinite(got) | ((got - want).abs() > bound)
    assert int(bad.sum()) == 0, f"{int(bad.sum())} gated outputs outside the bound"


@pytest.mark.parametrize("shape", [(16, 1024, 1024), (64, 4096, 512), (100, 1000, 1056), (128, 28672, 1024),
                                   (1, 256, 256), (33, 130 * 2, 96)])
def test_fp4_decode_gated_epilogue(smb, cuda_device, shape):
    """SMB_FLAG_EPILOGUE_SWIGLU on the decode kernel (an MLP up/gate projection at decode): weight
    rows interleaved (2n = up, 2n + 1 = gate), D = [M, N / 2], in the swapped forms (neighbouring
    lanes exchange their accumulators) and the wide form (M > 64)."""
    torch = _torch()
    m, n, k = shape
    a, sfa, sfar = _fp4_operand(smb, m, k, 6, 0)
    b, sfb, sfbr = _fp4_operand(smb, n, k, 5, 1)
    ldd = (n // 2 + 7) // 8 * 8 + 8
    d = torch.full((m, ldd), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, ldd=ldd, flags=smb.capi.FLAG_EPILOGUE_SWIGLU)
    assert plan.describe().startswith("fp4 decode")
    plan.run()
    plan.check()
    plan.close()
    # An aligned D is written in whole 16-byte chunks: a row's padding up to the next multiple of 8
    # elements may be overwritten, nothing beyond it.
    assert bool(torch.isnan(d[:, (n // 2 + 7) // 8 * 8:].float()).all()), "padding columns were written"
    acc = _dequant(a, sfar) @ _dequant(b, sfbr).t()
    _check_swiglu_torch(acc, d[:, :n // 2], k)


def test_fp4_gated_epilogue_on_the_384_tile(smb, cuda_device):
    torch = _torch()
    m, n, k = 768, 2432, 512
    a, sfa, sfar = _fp4_operand(smb, m, k, 5, 0)
    b, sfb, sfbr = _fp4_operand(smb, n, k, 5, 1)
    d = torch.full((m, n // 2), float("nan"), device=cuda_device, dtype=torch.bfloat16)
    plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, ldd=n // 2,
                            flags=smb.capi.FLAG_EPILOGUE_SWIGLU | smb.capi.FLAG_TILE_N_384)
    assert "256x384" in plan.describe() and "swiglu" in plan.describe()
    for clusters in (0, 5):
        d.fill_(float("nan"))
        plan.tune(0, clusters, -1)
        plan.run()
        plan.check()
        acc = _dequant(a, sfar) @ _dequant(b, sfbr).t()
        _check_swiglu_torch(acc, d, k)
    plan.close()


# ------------------------------------------------------------------------------- seeded random shapes
@pytest.mark.parametrize("seed", [1, 2, 3])
def test_fp4_schedules_agree_bit_for_bit_on_random_shapes(smb, cuda_device, seed):
    """The three FP4 schedules (256-wide tiles, the 384-wide tile list, the A-resident runs where K
    allows) accumulate every output element over K in the same order: on seeded random shapes,
    cluster counts and store paths their outputs are the same bits, and padding columns stay
    untouched."""
    import random
    torch = _torch()
    capi = smb.capi
    rng = random.Random(seed)
    for _ in range(25):
        m = rng.choice([1, 17, 129, 256, 257, 300, 512, 1000, 2048, 3000])
        n = rng.choice([384, 385, 400, 577, 768, 1000, 1152, 2048, 2432])
        k = 32 * rng.randint(1, 96)
        clusters = rng.choice([0, 0, 1, 3, 7, 20, 74])
        store = rng.choice([0, capi.FLAG_FORCE_PLAIN_STORE])
        ldd = n + (rng.choice([0, 8, 24]) if store == 0 else rng.choice([0, 1, 3]))
        a, sfa, _ = _fp4_operand(smb, m, k, 5, 0)
        b, sfb, _ = _fp4_operand(smb, n, k, 5, 1)
        base = torch.empty((m, n), device=cuda_device, dtype=torch.bfloat16)
        plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, base, m, n, k, flags=capi.FLAG_TILE_N_256 | capi.FLAG_NO_DECODE)
        plan.run()
        plan.check()
        plan.close()
        variants = [capi.FLAG_TILE_N_384] + ([capi.FLAG_TILE_N_192] if k <= 2048 else [])
        for tile in variants:
            d = torch.full((m, ldd), float("nan"), device=cuda_device, dtype=torch.bfloat16)
            plan = smb.gemm.Fp4Plan(a, sfa, b, sfb, d, m, n, k, ldd=ldd, flags=tile | capi.FLAG_NO_DECODE | store)
            plan.tune(0, clusters, -1)
            plan.run()
            plan.run()
            plan.check()
            plan.close()
            assert torch.equal(d[:, :n], base), (m, n, k, clusters, store, ldd, tile)
            assert ldd == n or bool(torch.isnan(d[:, n:].float()).all()), (m, n, k, ldd, tile)


@pytest.mark.parametrize("seed", [1, 2])
def test_bf16_last_wave_cut_on_random_shapes(smb, oracle, cuda_device, seed):
    """SMB_FLAG_STREAM_K on seeded random shapes and cluster counts, three launches per plan: full
    fp64 check each time."""
    import random
    torch = _torch()
    rng = random.Random(seed)
    for _ in range(12):
        m = rng.choice([256, 300, 512, 1000, 2048])
        n = rng.choice([264, 512, 520, 1024, 1104, 2048, 3000])
        k = 64 * rng.randint(1, 64) + rng.choice([0, 0, 8, 32])
        clusters = rng.choice([0, 0, 1, 2, 3, 5, 7, 20, 37, 74])
        ldd = (n + rng.choice([0, 8, 24]) + 7) // 8 * 8
        a = torch.empty(m, k, device=cuda_device, dtype=torch.bfloat16)
        bt = torch.empty(n, k, device=cuda_device, dtype=torch.bfloat16)
        smb.gemm.bf16_operands_device(a, bt, m, n, k, 5)
        d = torch.full((m, ldd), float("nan"), device=cuda_device, dtype=torch.bfloat16)
        plan = smb.gemm.Bf16Plan(a, bt, d, m, n, k, ldd=ldd, flags=smb.capi.FLAG_STREAM_K)
        plan.tune(0, clusters)
        for _ in range(3):
            plan.run()
        plan.check()
        plan.close()
        assert ldd == n or bool(torch.isnan(d[:, n:].float()).all()), (m, n, k, clusters, ldd)
        _check_bf16_full(oracle, a, bt, d, n, k)
