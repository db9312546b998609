"""The oracle against the golden vectors produced by the reference's own verifier code
(tests/golden/make_golden.py), plus self-consistency of the parts the reference does not pin."""
import numpy as np
import pytest


def test_bf16_rounding_matches_reference(oracle, golden):
    f32 = golden["f32_samples"]
    np.testing.assert_array_equal(oracle.f32_to_bf16(f32), golden["f32_to_bf16"])
    np.testing.assert_array_equal(oracle.bf16_to_f32(golden["f32_to_bf16"]).view(np.uint32),
                                  golden["bf16_to_f32"].view(np.uint32))


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
@pytest.mark.parametrize("seed", [1, 2])
def test_bf16_fill_matches_reference(oracle, golden, mode, seed):
    idx = golden["fill_indices"]
    want = golden[f"bf16_fill_m{mode}_s{seed}"]
    got = oracle.bf16_to_f32(oracle.bf16_fill(idx, mode, seed))
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("shape", [(256, 128, 64), (14080, 5120, 64), (8192, 8192, 256), (7, 5, 100)])
def test_sample_coordinates_match_reference(oracle, golden, shape):
    m, n, count = shape
    rows, cols = oracle.sample_coordinates(m, n, count)
    np.testing.assert_array_equal(rows, golden[f"sample_rows_{m}_{n}_{count}"])
    np.testing.assert_array_equal(cols, golden[f"sample_cols_{m}_{n}_{count}"])


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
def test_bf16_smoke_output_matches_reference(oracle, golden, mode):
    a, bt = oracle.bf16_operands(256, 128, 64, mode)
    got = oracle.gemm_bf16_reference(a, bt)
    want = golden[f"bf16_smoke_out_m{mode}"]
    # Same fp32 matmul up to summation order: allow one bf16 ulp, require most to be identical.
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1
    assert (diff == 0).mean() > 0.99
    ref64 = oracle.gemm_f64(oracle.bf16_to_f32(a), oracle.bf16_to_f32(bt))
    ok, ratio, bad = oracle.check_north_star(want, ref64, 64)
    assert ok, (ratio, bad)


@pytest.mark.parametrize("name", ["und-qkv", "gen-o"])
@pytest.mark.parametrize("mode", [1, 2])
def test_bf16_sampled_references_match(oracle, golden, name, mode):
    m, k, n = (int(x) for x in golden[f"bf16_{name}_shape"])
    rows, cols = golden[f"bf16_{name}_rows"], golden[f"bf16_{name}_cols"]
    ks = np.arange(k, dtype=np.uint64)
    a = oracle.bf16_to_f32(oracle.bf16_fill(rows.astype(np.uint64)[:, None] * np.uint64(k) + ks, mode, 1))
    b = oracle.bf16_to_f32(oracle.bf16_fill(ks[None, :] * np.uint64(n) + cols.astype(np.uint64)[:, None], mode, 2))
    ref64 = np.einsum("ik,ik->i", a.astype(np.float64), b.astype(np.float64))
    want = golden[f"bf16_{name}_ref_m{mode}"]
    np.testing.assert_allclose(ref64, want, rtol=2e-5, atol=2e-4)


@pytest.mark.parametrize("name", ["bf16_8192", "bf16_ragged", "bf16_large"])
def test_bf16_config_references_match(oracle, golden, name):
    """Every BF16 benchmark configuration, fill 2, at the reference verifier's own sample
    coordinates (its CASES extended at run time when the vectors were made): the oracle's operands
    and float64 product against the reference's sampled fp32 dot products."""
    m, k, n = (int(x) for x in golden[f"cfg_{name}_shape"])
    rows, cols = golden[f"cfg_{name}_rows"], golden[f"cfg_{name}_cols"]
    assert rows.size >= 200 and rows.max() < m and cols.max() < n
    ks = np.arange(k, dtype=np.uint64)
    a = oracle.bf16_to_f32(oracle.bf16_fill(rows.astype(np.uint64)[:, None] * np.uint64(k) + ks, 2, 1))
    b = oracle.bf16_to_f32(oracle.bf16_fill(ks[None, :] * np.uint64(n) + cols.astype(np.uint64)[:, None], 2, 2))
    ref64 = np.einsum("ik,ik->i", a.astype(np.float64), b.astype(np.float64))
    np.testing.assert_allclose(ref64, golden[f"cfg_{name}_ref_m2"], rtol=5e-5, atol=2e-3)


@pytest.mark.parametrize("name", ["nvfp4_8192", "decode_m16", "decode_m64", "decode_m128"])
def test_fp4_config_references_match(oracle, golden, name):
    m, k, n = (int(x) for x in golden[f"cfg_{name}_shape"])
    rows, cols = golden[f"cfg_{name}_rows"], golden[f"cfg_{name}_cols"]
    want = golden[f"cfg_{name}_ref_m2"]
    ks = np.arange(k, dtype=np.uint64)
    kb = np.arange(k // 32, dtype=np.uint64)
    for i in range(0, rows.size, 4):     # every fourth sample keeps the CPU suite short
        r, c = rows[i], cols[i]
        a = oracle.e2m1_decode(oracle.fp4_fill_codes(np.uint64(r) * np.uint64(k) + ks, 2, oracle.SEED_FP4_A))
        b = oracle.e2m1_decode(oracle.fp4_fill_codes(np.uint64(c) * np.uint64(k) + ks, 2, oracle.SEED_FP4_B))
        sa = np.exp2(oracle.fp4_fill_scale_exp(np.uint64(r), kb, 2, 0).astype(np.float64))
        sb = np.exp2(oracle.fp4_fill_scale_exp(np.uint64(c), kb, 2, 1).astype(np.float64))
        ref = float(np.sum(a.astype(np.float64) * np.repeat(sa, 32) * b * np.repeat(sb, 32)))
        assert abs(ref - float(want[i])) <= max(16.0, 0.008 * abs(ref))


def test_hash_matches_reference(oracle, golden):
    np.testing.assert_array_equal(oracle.hash32(golden["hash_inputs"]), golden["hash32"])


def test_e2m1_table_matches_reference(oracle, golden):
    np.testing.assert_array_equal(oracle.E2M1_TABLE.view(np.uint32), golden["e2m1_table"].view(np.uint32))


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
def test_fp4_fill_values_match_reference(oracle, golden, mode):
    idx = golden["fill_indices"]
    for name, seed in (("A", oracle.SEED_FP4_A), ("B", oracle.SEED_FP4_B)):
        got = oracle.e2m1_decode(oracle.fp4_fill_codes(idx, mode, seed))
        want = golden[f"fp4_data_m{mode}_{name}"]
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
@pytest.mark.parametrize("which", [0, 1])
def test_fp4_scales_match_reference(oracle, golden, mode, which):
    e = oracle.fp4_fill_scale_exp(golden["scale_rows"], golden["scale_blocks"], mode, which)
    np.testing.assert_array_equal(np.exp2(e.astype(np.float32)), golden[f"fp4_scale_m{mode}_w{which}"])


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
def test_fp4_smoke_output_matches_reference(oracle, golden, mode):
    a_codes, a_sf = oracle.fp4_operand(256, 256, mode, 0)
    b_codes, b_sf = oracle.fp4_operand(128, 256, mode, 1)
    got = oracle.gemm_nvfp4_reference(a_codes, a_sf, b_codes, b_sf)
    want = golden[f"fp4_smoke_out_m{mode}"]
    diff = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert diff.max() <= 1
    assert (diff == 0).mean() > 0.98
    if mode in (1, 3):
        # Closed form of the constant fills: D = p K 2^((m%5)-2) 2^((n%3)-1), p = 16 or 1.
        p = 16.0 if mode == 1 else 1.0
        m = np.arange(256)[:, None]
        n = np.arange(128)[None, :]
        exact = p * 256 * np.exp2((m % 5) - 2.0) * np.exp2((n % 3) - 1.0)
        np.testing.assert_array_equal(oracle.bf16_to_f32(want), exact.astype(np.float32))
        np.testing.assert_array_equal(oracle.bf16_to_f32(got), exact.astype(np.float32))


@pytest.mark.parametrize("mode", [2, 4])
def test_fp4_flagship_samples_match_reference(oracle, golden, mode):
    m, k, n = (int(x) for x in golden["fp4_flagship_shape"])
    rows, cols = golden["fp4_flagship_rows"], golden["fp4_flagship_cols"]
    want = golden[f"fp4_flagship_ref_m{mode}"]
    ks = np.arange(k, dtype=np.uint64)
    kb = np.arange(k // 32, dtype=np.uint64)
    for i, (r, c) in enumerate(zip(rows, cols)):
        a = oracle.e2m1_decode(oracle.fp4_fill_codes(np.uint64(r) * np.uint64(k) + ks, mode, oracle.SEED_FP4_A))
        b = oracle.e2m1_decode(oracle.fp4_fill_codes(np.uint64(c) * np.uint64(k) + ks, mode, oracle.SEED_FP4_B))
        sa = np.exp2(oracle.fp4_fill_scale_exp(np.uint64(r), kb, mode, 0).astype(np.float64))
        sb = np.exp2(oracle.fp4_fill_scale_exp(np.uint64(c), kb, mode, 1).astype(np.float64))
        ref = float(np.sum(a.astype(np.float64) * np.repeat(sa, 32) * b * np.repeat(sb, 32)))
        # The reference rounds an fp32 sum to bf16: within its own tolerance of the exact value.
        assert abs(ref - float(want[i])) <= max(16.0, 0.008 * abs(ref))


# ---------------------------------------------------------------------------------------
# Parts with no reference counterpart: self-consistency.
# ---------------------------------------------------------------------------------------
def test_gauss12_moments(oracle):
    g = oracle.gauss12(np.arange(1 << 20), 1)
    assert abs(float(g.mean())) < 5e-3
    assert abs(float(g.var()) - 1.0) < 1e-2
    assert float(np.abs(g).max()) < 6.0
    assert np.all(g * 65536 == np.round(g * 65536))
    # Different seeds decorrelate.
    h = oracle.gauss12(np.arange(1 << 20), 2)
    assert abs(float(np.corrcoef(g, h)[0, 1])) < 5e-3


def test_e2m1_encode_ties_and_roundtrip(oracle):
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], dtype=np.float32)
    want = np.array([0.0, 1.0, 1.0, 2.0, 2.0, 4.0, 4.0], dtype=np.float32)
    np.testing.assert_array_equal(oracle.e2m1_decode(oracle.e2m1_encode(ties)), want)
    np.testing.assert_array_equal(oracle.e2m1_decode(oracle.e2m1_encode(-ties)), -want)
    codes = np.arange(16, dtype=np.uint8)
    np.testing.assert_array_equal(oracle.e2m1_encode(oracle.e2m1_decode(codes)) & 7, codes & 7)
    # Nearest: brute force against the table.
    x = np.linspace(-7, 7, 5601).astype(np.float32)
    dec = oracle.e2m1_decode(oracle.e2m1_encode(x))
    inside = np.abs(x) <= 6
    best = np.min(np.abs(x[:, None].astype(np.float64) - oracle.E2M1_TABLE[None, :]), axis=1)
    np.testing.assert_allclose(np.abs(dec - x)[inside], best[inside], atol=1e-7)
    np.testing.assert_array_equal(dec[~inside], np.sign(x[~inside]) * 6)


def test_ue8m0_exponent_is_smallest_cover(oracle):
    rng = np.random.default_rng(3)
    amax = np.concatenate([np.exp2(rng.uniform(-30, 30, 4000)).astype(np.float32),
                           np.array([6.0, 6.0000005, 3.0, 0.75, 1.5, 12.0, 1e-45, 3.0e38], dtype=np.float32)])
    e = oracle.ue8m0_exponent(amax).astype(np.float64)
    inside = (e > -126) & (e < 127)
    assert np.all(6.0 * np.exp2(e[inside]) >= amax[inside].astype(np.float64))
    assert np.all(6.0 * np.exp2(e[inside] - 1) < amax[inside].astype(np.float64))
    assert oracle.ue8m0_exponent(np.float32(0.0)) == 0


def test_quantizer_roundtrip_and_error(oracle):
    rng = np.random.default_rng(5)
    x = rng.standard_normal((64, 256)).astype(np.float32)
    codes, sf = oracle.quantize_mx(x)
    assert sf.min() >= 1 and sf.max() <= 254
    deq = oracle.dequantize(codes, sf)
    scale = np.repeat(np.exp2(sf.astype(np.float32) - 127), 32, axis=1)
    # Error at most half the widest E2M1 gap (2.0 between 4 and 6) times the block scale.
    assert np.all(np.abs(deq - x) <= 1.0 * scale + 1e-7)
    # The largest element of every block lands in the top binade of E2M1: |code value| >= 4
    # unless rounding pulled it down from (3.5, 4); never saturated beyond 6.
    top = np.abs(oracle.e2m1_decode(codes)).reshape(64, -1, 32).max(axis=2)
    assert np.all(top >= 3.0) and np.all(top <= 6.0)
    # Idempotent: quantising the dequantised values reproduces codes (up to -0) and scales.
    codes2, sf2 = oracle.quantize_mx(deq)
    np.testing.assert_array_equal(oracle.dequantize(codes2, sf2), deq)
    # Packing round trip, nibble order: even k low.
    packed = oracle.pack_codes(codes)
    assert packed.shape == (64, 128)
    np.testing.assert_array_equal(oracle.unpack_codes(packed), codes)
    assert packed[0, 0] == (codes[0, 0] | (codes[0, 1] << 4))


def test_sf_pack_layout(oracle):
    rows, kb = 300, 10
    sf = (np.arange(rows * kb) % 251).astype(np.uint8).reshape(rows, kb)
    packed = oracle.sf_pack(sf)
    assert packed.size == oracle.sf_packed_size(rows, kb) == 3 * 3 * 512
    for r, j in [(0, 0), (1, 0), (31, 3), (32, 0), (95, 7), (127, 9), (128, 0), (299, 9), (200, 4)]:
        band, rr = divmod(r, 128)
        off = (band * 3 + j // 4) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + j % 4
        assert packed[off] == sf[r, j]
    # Padding rows / k-blocks read as scale 1.
    assert packed[(2 * 3 + 0) * 512 + (50 % 32) * 16 + (50 // 32) * 4 + 0] == 127  # row 306
    assert packed[(0 * 3 + 2) * 512 + 0 * 16 + 0 * 4 + 2] == 127                    # k-block 10


def test_tile_raster_is_a_permutation(oracle):
    for tiles_m, tiles_n, gm in [(32, 16, 16), (32, 32, 8), (5, 7, 8), (17, 3, 4), (1, 1, 8), (128, 14, 16)]:
        seen = {oracle.tile_coords(t, tiles_m, tiles_n, gm) for t in range(tiles_m * tiles_n)}
        assert len(seen) == tiles_m * tiles_n
        assert all(0 <= m < tiles_m and 0 <= n < tiles_n for m, n in seen)


def test_swiglu_definition(oracle):
    acc = np.array([[2.0, 0.0, -3.0, 1.0, 0.5, 40.0, 7.0, -40.0]])
    out = oracle.swiglu(acc)
    # up = (2, -3, 0.5, 7), gate = (0, 1, 40, -40)
    want = np.array([[0.0, -3.0 / (1.0 + np.exp(-1.0)), 0.5 * 40.0, 7.0 * -40.0 / (1.0 + np.exp(40.0))]])
    np.testing.assert_allclose(out, want, rtol=1e-12, atol=1e-300)
    assert out.shape == (1, 4)
    # The tanh form the device uses is the same function.
    z = np.linspace(-20, 20, 4001)
    np.testing.assert_allclose(0.5 * z * (1 + np.tanh(z / 2)), z / (1 + np.exp(-z)), rtol=1e-12, atol=1e-15)
    assert np.all(oracle.swiglu_bound(acc, 64) > 0)
