"""CPU-side checks of the C ABI: the library loads, exports what the header declares, its
host-side generators agree with the oracle bit for bit, its descriptor bit patterns match the
known answers, and argument errors come back as status codes.  No kernel is launched here."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(smb):
    lib = smb.capi.lib()
    header = (ROOT / "include" / "strata_masonry_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(smb_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations parsed"
    bound = {name for name, _, _ in smb.capi.DECLARED}
    assert declared == bound, (declared - bound, bound - declared)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.smb_version() >= 1000


def test_product_never_reaches_into_the_oracle():
    # The oracle is test infrastructure: nothing under the package may import, include or open it.
    for p in (ROOT / "strata-masonry_b200").rglob("*"):
        if p.suffix == ".py":
            for line in p.read_text().splitlines():
                assert not re.match(r"\s*(from|import)\s+\S*oracle", line), (p, line)
                assert "oracle/" not in line and "oracle.py" not in line, (p, line)
        elif p.suffix in (".cu", ".cuh", ".cpp", ".h"):
            for line in p.read_text().splitlines():
                if line.lstrip().startswith("#include"):
                    assert "oracle" not in line, (p, line)


@pytest.mark.parametrize("fill", [1, 2, 3, 4, 5, 6, 7])
def test_bf16_host_fill_matches_oracle(smb, oracle, fill):
    m, k, n = 37, 72, 29
    a = smb.gemm.fill_bf16_host(m, k, fill, 1, 0, k, 1)
    bt = smb.gemm.fill_bf16_host(n, k, fill, 2, 0, 1, n)
    wa, wbt = oracle.bf16_operands(m, n, k, fill)
    np.testing.assert_array_equal(a, wa)
    np.testing.assert_array_equal(bt, wbt)
    # A slab of a wider BT (N-sharding) uses the global column index.
    slab = smb.gemm.fill_bf16_host(8, k, fill, 2, 13, 1, 64)
    _, wslab = oracle.bf16_operands(1, 8, k, fill, n0=13, n_total=64)
    np.testing.assert_array_equal(slab, wslab)


@pytest.mark.parametrize("fill", [1, 2, 3, 4])
def test_bf16_host_fill_matches_reference_vectors(smb, oracle, golden, fill):
    idx = golden["fill_indices"]
    for seed in (1, 2):
        want = oracle.f32_to_bf16(golden[f"bf16_fill_m{fill}_s{seed}"])
        got = np.empty(idx.size, dtype=np.uint16)
        lib = smb.capi.lib()
        for i, v in enumerate(idx[:: max(1, idx.size // 512)]):
            one = np.empty(1, dtype=np.uint16)
            assert lib.smb_fill_bf16_host(one.ctypes.data, 1, 1, 1, int(v) & 0xFFFFFFFFFFFFFFFF, 0, 0, fill, seed) == 0
            assert one[0] == want[i * max(1, idx.size // 512)]


def test_bf16_fill_wraps_at_32_bits(smb, oracle):
    # Index arithmetic wraps modulo 2^32 as in the reference driver.
    big = (1 << 32) + 12345
    a = smb.gemm.fill_bf16_host(1, 8, 2, 1, big, 8, 1)
    b = smb.gemm.fill_bf16_host(1, 8, 2, 1, 12345, 8, 1)
    np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("fill", [1, 2, 3, 4, 5, 6])
@pytest.mark.parametrize("which", [0, 1])
def test_fp4_host_fill_matches_oracle(smb, oracle, fill, which):
    rows, k, row0 = 150, 320, 7
    data, sf_packed, sf_rm = smb.gemm.fill_fp4_host(rows, k, fill, which, row0)
    codes, sf = oracle.fp4_operand(rows, k, fill, which, row0)
    np.testing.assert_array_equal(data, oracle.pack_codes(codes))
    np.testing.assert_array_equal(sf_rm, sf)
    np.testing.assert_array_equal(sf_packed, oracle.sf_pack(sf))


def test_quantizer_matches_oracle(smb, oracle):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((70, 256)).astype(np.float32)
    x[0, :32] = 0.0                       # all-zero block
    x[1, :32] = 6.0                       # exactly the top code
    x[2, :32] = np.float32(6.0000005)     # just above: next exponent
    x[3, :8] = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0]   # ties at scale 1
    x[3, 8:32] = 0.0
    x[4, :32] = 1e-41                     # subnormal block
    x[5, :32] *= 1e30
    data, sf_packed, sf_rm = smb.gemm.quantize_mx_host(x)
    codes, sf = oracle.quantize_mx(x)
    np.testing.assert_array_equal(sf_rm, sf)
    np.testing.assert_array_equal(data, oracle.pack_codes(codes))
    np.testing.assert_array_equal(sf_packed, oracle.sf_pack(sf))
    assert sf_rm.min() >= 1 and sf_rm.max() <= 254


def test_sf_pack_matches_oracle(smb, oracle):
    sf = (np.arange(300 * 10) * 7 % 251).astype(np.uint8).reshape(300, 10)
    np.testing.assert_array_equal(smb.gemm.sf_pack_host(sf), oracle.sf_pack(sf))
    lib = smb.capi.lib()
    assert lib.smb_sf_packed_bytes(300, 10) == oracle.sf_packed_size(300, 10)
    assert lib.smb_debug_sf_offset(95, 7, 10) == (7 // 4) * 512 + (95 % 32) * 16 + (95 // 32) * 4 + 3


def test_descriptor_known_answers(smb):
    lib = smb.capi.lib()
    # Shared-memory descriptor: addr 0x4000, SBO 256, LBO 128, 128-byte swizzle (the case pinned
    # by the reference's tests/42_smem_desc_blackwell_test.cu).
    want = (0x4000 >> 4) | ((128 >> 4) << 16) | ((256 >> 4) << 32) | (1 << 46) | (2 << 61)
    assert lib.smb_debug_smem_desc(0x4000, 256, 128, 2) == want
    assert (lib.smb_debug_smem_desc(0x4000, 256, 128, 0) >> 61) == 0
    # The operand descriptors the kernels build: SBO 1024, LBO 16.
    d = lib.smb_debug_smem_desc(0x8400, 1024, 16, 2)
    assert d & 0x3FFF == 0x840 and (d >> 16) & 0x3FFF == 1 and (d >> 32) & 0x3FFF == 64
    # kind::f16 instruction descriptor (layout pinned by tests/8_tcgen05_mma_idesc_test.cu):
    # D = F32 at bit 4, A/B = BF16 at bits 7/10, N >> 3 at 17, M >> 4 at 24.
    assert lib.smb_debug_idesc_bf16(128, 64) == (1 << 4) | (1 << 7) | (1 << 10) | (8 << 17) | (8 << 24)
    assert lib.smb_debug_idesc_bf16(256, 256) == (1 << 4) | (1 << 7) | (1 << 10) | (32 << 17) | (16 << 24)
    # kind::mxf4nvf4: E2M1 at bits 7/10, N >> 3 at 17, UE8M0 at 23, M >> 7 at 27, scale ids at 4/29.
    base = (1 << 7) | (1 << 10) | (16 << 17) | (1 << 23) | (2 << 27)
    assert lib.smb_debug_idesc_mxf4(256, 128, 0, 0, 1) == base
    assert lib.smb_debug_idesc_mxf4(256, 128, 2, 2, 1) == base | (2 << 4) | (2 << 29)
    assert lib.smb_debug_idesc_mxf4(128, 128, 0, 0, 0) == (1 << 7) | (1 << 10) | (16 << 17) | (1 << 27)


def test_tile_raster_matches_oracle(smb, oracle):
    lib = smb.capi.lib()
    tm, tn = C.c_int(), C.c_int()
    for tiles_m, tiles_n, gm in [(32, 16, 16), (5, 7, 8), (17, 3, 4), (128, 14, 16)]:
        for t in range(tiles_m * tiles_n):
            lib.smb_debug_tile_coords(t, tiles_m, tiles_n, gm, C.byref(tm), C.byref(tn))
            assert (tm.value, tn.value) == oracle.tile_coords(t, tiles_m, tiles_n, gm)


def test_argument_errors_are_status_codes(smb):
    lib = smb.capi.lib()
    capi = smb.capi
    plan = C.c_void_p()
    buf = np.zeros(64, dtype=np.uint16)
    p = buf.ctypes.data
    assert lib.smb_bf16_plan_create(C.byref(plan), None, p, p, 256, 128, 64, 64, 64, 128, 0) == capi.SMB_ERR_INVALID
    assert "null" in capi.last_error()
    assert lib.smb_bf16_plan_create(C.byref(plan), p, p, p, 0, 128, 64, 64, 64, 128, 0) == capi.SMB_ERR_INVALID
    assert lib.smb_bf16_plan_create(C.byref(plan), p, p, p, 256, 128, 60, 64, 64, 128, 0) == capi.SMB_ERR_UNSUPPORTED
    assert lib.smb_bf16_plan_create(C.byref(plan), p, p, p, 256, 128, 64, 32, 64, 128, 0) == capi.SMB_ERR_INVALID
    assert lib.smb_bf16_plan_run(None, None) == capi.SMB_ERR_INVALID
    assert lib.smb_bf16_plan_destroy(None) == capi.SMB_OK
    assert lib.smb_fill_bf16_host(p, 2, 2, 2, 0, 2, 1, 9, 1) == capi.SMB_ERR_INVALID
    assert lib.smb_fill_bf16_host(None, 2, 2, 2, 0, 2, 1, 1, 1) == capi.SMB_ERR_INVALID
    assert lib.smb_fill_fp4_host(p, 16, None, None, 1, 48, 0, 2, 0) == capi.SMB_ERR_INVALID   # K % 32
    assert lib.smb_fill_fp4_host(p, 16, None, None, 1, 32, 0, 9, 0) == capi.SMB_ERR_INVALID   # fill id
    assert lib.smb_dense_gemm_bf16_host(None, p, p, 1, 1, 8) == capi.SMB_ERR_INVALID
    with pytest.raises(capi.SmbError):
        capi.check(capi.SMB_ERR_INVALID)


def test_missing_library_is_loud(smb, tmp_path, monkeypatch):
    capi = smb.capi
    monkeypatch.setattr(capi, "_lib", None)
    monkeypatch.setattr(capi, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(ImportError, match="no CPU fallback"):
        capi.lib()


# ------------------------------------------------------------------------------- NVFP4 proper
def test_nvf4_host_quantizer_matches_oracle(smb, oracle):
    """E4M3 scale per 16 values + caller's per-tensor factor: the C++ quantiser against the NumPy
    definition, on random data of many magnitudes and on crafted blocks whose maximum sits on
    every E4M3 grid point and every midpoint between neighbours (ties go to the even code)."""
    import ctypes as C
    lib = smb.capi.lib()
    rng = np.random.default_rng(11)
    x = (rng.standard_normal((40, 256)) * np.exp2(rng.integers(-12, 6, (40, 16)).repeat(16, axis=1))).astype(np.float32)
    x[0, :16] = 0
    grid = oracle.e4m3_decode(np.arange(0x7F)).astype(np.float64)
    probes = np.concatenate([grid, (grid[:-1] + grid[1:]) / 2, [448.0, 460.0, 464.0, 500.0, 1e6, 2.0 ** -10, 2.0 ** -11]])
    crafted = np.zeros((len(probes), 16), dtype=np.float32)
    crafted[:, 0] = probes.astype(np.float32)
    crafted[:, 1] = -probes.astype(np.float32) / 3
    for data_in, gs in ((x, 37.5), (x, 0.01), (crafted, 6.0)):
        rows, k = data_in.shape
        data = np.zeros((rows, k // 2), dtype=np.uint8)
        sfr = np.zeros((rows, k // 16), dtype=np.uint8)
        sfp = np.zeros(lib.smb_sf_packed_bytes(rows, k // 16), dtype=np.uint8)
        src = np.ascontiguousarray(data_in)
        if k // 2 % 16 != 0:      # rows of codes must be 16-byte aligned: pad K to 32
            src = np.zeros((rows, 32), dtype=np.float32); src[:, :k] = data_in; k = 32
            data = np.zeros((rows, 16), dtype=np.uint8); sfr = np.zeros((rows, 2), dtype=np.uint8)
            sfp = np.zeros(lib.smb_sf_packed_bytes(rows, 2), dtype=np.uint8)
        smb.capi.check(lib.smb_quantize_nvf4_host(src.ctypes.data, k, C.c_float(gs), data.ctypes.data, k // 2,
                                                  sfp.ctypes.data, sfr.ctypes.data, rows, k))
        codes, sb = oracle.quantize_nvf4(src, gs)
        np.testing.assert_array_equal(sfr, sb)
        np.testing.assert_array_equal(data, oracle.pack_codes(codes))
        np.testing.assert_array_equal(sfp, oracle.sf_pack(sb, pad=0))
        assert sb.max() <= 0x7E
    # Round trip: the represented values are within half an E2M1 step of the block maximum.
    gs = 448.0 * 6.0 / float(np.abs(x).max())      # the usual choice: the largest block scale is 448
    codes, sb = oracle.quantize_nvf4(x, gs)
    back = oracle.dequantize_nvf4(codes, sb, gs)
    amax = np.abs(x.reshape(40, 16, 16)).max(axis=2).repeat(16, axis=1)
    assert np.all(np.abs(back - x) <= 0.26 * np.maximum(amax, 1e-30) + 2.0 ** -9 / gs * 6)
    assert lib.smb_quantize_nvf4_host(None, 0, C.c_float(1.0), None, 0, None, None, 1, 32) == smb.capi.SMB_ERR_INVALID
    assert lib.smb_fp4_plan_set_alpha(None, C.c_float(1.0)) == smb.capi.SMB_ERR_INVALID


def test_new_entry_points_validate_their_arguments(smb):
    """Host-side rules of the entry points added for the sharded path, the self test and the
    allocation-free decode call: all of them answer with status codes before touching a device."""
    lib, capi = smb.capi.lib(), smb.capi
    # All-gather shape rules (no device, no NCCL needed).
    assert lib.smb_allgather_check(8, 32768, 7168, 57344) == capi.SMB_OK
    assert lib.smb_allgather_check(8, 32768, 7168, 0) == capi.SMB_OK          # no full-D copy asked for
    assert lib.smb_allgather_check(0, 16, 8, 8) == capi.SMB_ERR_INVALID
    assert lib.smb_allgather_check(2, 16, 12, 24) == capi.SMB_ERR_INVALID     # slab rows not 16-byte multiples
    assert "multiple of 8" in capi.last_error()
    assert lib.smb_allgather_check(2, 16, 8, 8) == capi.SMB_ERR_INVALID       # pitch below world * n_local
    assert lib.smb_allgather_check(2, 0, 8, 16) == capi.SMB_ERR_INVALID
    assert lib.smb_allgather_columns(None, None, None, None, 16, 8, 16, None) == capi.SMB_ERR_INVALID
    assert lib.smb_comm_create(None, None, 2, 0) == capi.SMB_ERR_INVALID
    assert lib.smb_comm_destroy(None) == capi.SMB_OK
    # Contexts and probes.
    ctx = C.c_void_p()
    assert lib.smb_fp4_host_ctx_create(C.byref(ctx), 16, 128, 48) == capi.SMB_ERR_INVALID   # K % 32
    assert lib.smb_fp4_host_ctx_run(None, None, None, None, None, None) == capi.SMB_ERR_INVALID
    assert lib.smb_fp4_host_ctx_destroy(None) == capi.SMB_OK
    assert lib.smb_bf16_host_ctx_create_sharded(C.byref(ctx), 16, 128, 64, None) == capi.SMB_ERR_INVALID
    assert lib.smb_fp4_host_ctx_create_sharded(C.byref(ctx), 16, 128, 64, None) == capi.SMB_ERR_INVALID
    assert lib.smb_bf16_plan_wait_probe(None, 1000, None) == capi.SMB_ERR_INVALID
    assert lib.smb_fp4_plan_wait_probe(None, 1000, None) == capi.SMB_ERR_INVALID
    assert lib.smb_bf16_plan_describe(None, None, 0) == capi.SMB_ERR_INVALID
    # Allocation-free decode call: the split is a process-wide setting with a range.
    assert lib.smb_decode_noalloc_set_split(-1) == capi.SMB_ERR_INVALID
    assert lib.smb_decode_noalloc_set_split(4097) == capi.SMB_ERR_INVALID
    assert lib.smb_decode_noalloc_set_split(0) == capi.SMB_OK
    assert lib.smb_decode_noalloc_scratch_limit() == (2 << 20) - 256


@pytest.mark.parametrize("shape", [(8192, 8192, 8192), (14080, 5120, 2048), (30720, 2048, 4096), (300, 1000, 256),
                                   (256, 384, 256), (8192, 1024, 8192), (512, 130, 512)])
def test_fp4_tile_list_covers_every_column_once(smb, shape):
    """The FP4 kernel with 256 x 384 tiles hands out full tiles first and 256-wide tiles after them;
    together they must cover every 128-column unit of every tile row exactly once, whatever the
    split, and the split must never be worse than uniform tiles under its own cost model."""
    lib = smb.capi.lib()
    m, n, k = shape
    tiles_m = (m + 255) // 256
    units = (n + 127) // 128
    for clusters in (74, 66, 1):
        wide, narrow = C.c_int(), C.c_int()
        lib.smb_debug_fp4_phases(m, n, k, clusters, C.byref(wide), C.byref(narrow))
        a, b = wide.value, narrow.value
        assert a >= 0 and b >= 0 and a * 384 + b * 256 >= n
        assert a * 384 < n + 384 and (b == 0 or a * 384 + (b - 1) * 256 < n)
        seen = np.zeros((tiles_m, units), dtype=np.int32)
        tm, col0, full = C.c_int(), C.c_int(), C.c_int()
        for t in range(tiles_m * (a + b)):
            lib.smb_debug_fp4_tile(t, tiles_m, a, b, 12, C.byref(tm), C.byref(col0), C.byref(full))
            assert 0 <= tm.value < tiles_m and col0.value % 128 == 0 and col0.value < n
            width = 384 if full.value else 256
            u0 = col0.value // 128
            seen[tm.value, u0:min(units, u0 + width // 128)] += 1
        assert (seen == 1).all(), (a, b)
    # 8192^3 on 74 clusters: a few 256-wide tiles at the end of every group of tile rows leave the
    # clusters more evenly loaded than 21 full tiles and a 128-column remainder per row.
    wide, narrow = C.c_int(), C.c_int()
    lib.smb_debug_fp4_phases(8192, 8192, 8192, 74, C.byref(wide), C.byref(narrow))
    assert narrow.value >= 2 and wide.value * 384 + narrow.value * 256 == 8192


def test_fp4_a_resident_run_split_covers_every_tile_once(smb):
    """Runs of the A-resident schedule: chunks x run_len covers the tile row, no run is empty, and
    the shapes outside its range are refused (K > 2048, N < 384)."""
    lib = smb.capi.lib()
    for (m, n, k) in [(512, 768, 512), (14080, 5120, 2048), (30720, 5120, 2048), (8192, 8192, 256), (300, 400, 96),
                      (256, 100000, 1024)]:
        for clusters in (74, 7, 1):
            chunks, run_len = C.c_int(-1), C.c_int(-1)
            assert lib.smb_debug_fp4_arun_split(m, n, k, clusters, C.byref(chunks), C.byref(run_len)) == 1
            tiles_n = (n + 191) // 192
            assert chunks.value >= 1 and run_len.value >= 1
            assert chunks.value * run_len.value >= tiles_n
            assert (chunks.value - 1) * run_len.value < tiles_n
    chunks, run_len = C.c_int(-1), C.c_int(-1)
    assert lib.smb_debug_fp4_arun_split(512, 768, 4096, 74, C.byref(chunks), C.byref(run_len)) == 0
    assert lib.smb_debug_fp4_arun_split(512, 256, 512, 74, C.byref(chunks), C.byref(run_len)) == 0
    assert chunks.value == -1
    # One cluster: nothing to balance, one run per tile row.
    assert lib.smb_debug_fp4_arun_split(2048, 3840, 2048, 1, C.byref(chunks), C.byref(run_len)) == 1
    assert (chunks.value, run_len.value) == (1, 20)


def test_bf16_last_wave_cut_covers_every_k_block_once(smb):
    """The walk of SMB_FLAG_STREAM_K: whole-tile waves, then the last wave either as [0, cut) on one
    cluster per tile plus [cut, end) on the spare clusters, or as equal K slices.  Every K block of
    every tile is covered exactly once, no cluster gets more than one owner part, and the choice
    for the column shards of 8192^3 is what was measured to pay (2 GPUs) or not (4, 8 GPUs, 1 GPU)."""
    lib = smb.capi.lib()
    out = (C.c_int * 5)()
    for tiles, kb, clusters in [(64, 128, 74), (128, 128, 74), (256, 128, 74), (512, 128, 74), (1792, 128, 74),
                                (4, 64, 3), (1, 128, 5), (12, 33, 7), (32, 16, 74), (4, 16, 74), (74, 128, 74), (75, 128, 74)]:
        lib.smb_debug_bf16_streamk_plan(tiles, kb, clusters, out)
        full, rem, cut, tails, parts = list(out)
        assert full == tiles // clusters and rem == tiles % clusters
        spare = clusters - rem
        covered = 0
        if rem:
            if parts > 0:
                assert spare >= rem * parts and parts <= 7
                bounds = [kb * i // (parts + 1) for i in range(parts + 2)]
                assert bounds[0] == 0 and bounds[-1] == kb and all(b1 > b0 for b0, b1 in zip(bounds, bounds[1:]))
                covered = rem * kb
            elif cut < kb:
                assert 1 <= cut and tails >= 1 and spare * tails >= rem      # every tile's tail has a cluster
                covered = rem * cut + rem * (kb - cut)
            else:
                covered = rem * kb                                             # left whole
        assert covered == rem * kb
    assert lib.smb_debug_bf16_streamk_plan(256, 128, 74, out) == 1    # 8192 x 4096 x 8192: one long slice per spare cluster
    assert list(out) == [3, 34, 128, 0, 1]
    assert lib.smb_debug_bf16_streamk_plan(64, 128, 74, out) == 0     # 8192 x 1024 x 8192: seven tails per spare cluster
    assert lib.smb_debug_bf16_streamk_plan(128, 128, 74, out) == 0
    assert lib.smb_debug_bf16_streamk_plan(512, 128, 74, out) == 0
