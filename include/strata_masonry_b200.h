/*
 * strata_masonry_b200 -- C ABI of the B200 (sm_100a) dense GEMM path.
 *
 * The reference project (strata-masonry) exposes this path only as two executables,
 * kernel_sm100a_dense_gemm_bf16 and kernel_sm100a_dense_gemm_nvfp4, each a single .cu
 * with its own main().  This header declares the library those drivers sit on here;
 * each entry point names the reference code it stands in for.
 *
 * Conventions: every function returns SMB_OK (0) or a negative smb_status; nothing
 * calls exit() or throws across this boundary; smb_last_error() returns a thread-local
 * message for the last failure.  Device entry points are stream-ordered and never
 * synchronise; the caller owns all operand buffers.  `stream` is a cudaStream_t passed
 * as void* (NULL = the default stream).  A missing GPU is an error, never a silent CPU
 * path.
 */
#ifndef STRATA_MASONRY_B200_H_
#define STRATA_MASONRY_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum smb_status {
  SMB_OK = 0,
  SMB_ERR_INVALID = -1,      /* bad shape, null pointer, misaligned pointer or stride */
  SMB_ERR_UNSUPPORTED = -2,  /* valid request that this build cannot serve */
  SMB_ERR_CUDA = -3,         /* a CUDA runtime / driver call failed */
  SMB_ERR_DEVICE = -4,       /* a kernel reported a non-zero status word */
  SMB_ERR_IO = -5,           /* file could not be written */
  SMB_ERR_NOMEM = -6
} smb_status;

/* Library version, major * 1000 + minor. */
int smb_version(void);

/* Message describing the last error on the calling thread ("" if none). */
const char* smb_last_error(void);

/* ------------------------------------------------------------------------------------
 * Input generators.  Bit-identical to the reference drivers' host fills; `index0` lets a
 * caller generate a slab of a larger logical tensor (N-sharding) with the global indices.
 * ---------------------------------------------------------------------------------- */

/* BF16 fills 1..4 of the reference driver (fill_random_bf16, dense_gemm_bf16.cu:268-279;
 * verifier fill(), dense_gemm_bf16_cpu_verifier.py:32-44), plus fills 5..7: a Gaussian
 * stand-in (sum of twelve 16-bit uniform fields of a counter hash, mean 0, variance 1)
 * scaled by 0.1, 0.05 and 1.0.  Element (r, c) of the [rows, cols] output takes the value
 * of flat index  index0 + r * index_row_stride + c * index_col_stride  (32-bit wrap-around
 * as in the reference): A[M,K] uses strides (K, 1) and seed 1; BT[N,K], the transpose of the
 * reference's B[K,N], uses strides (1, N) and seed 2.
 * `out` is device memory, row-major, `ld` elements between rows. */
int smb_fill_bf16_device(uint16_t* out, int64_t rows, int64_t cols, int64_t ld, uint64_t index0,
                         uint64_t index_row_stride, uint64_t index_col_stride, int fill,
                         uint32_t seed, void* stream);
/* Same on the host (single thread; for tests and small shapes). */
int smb_fill_bf16_host(uint16_t* out, int64_t rows, int64_t cols, int64_t ld, uint64_t index0,
                       uint64_t index_row_stride, uint64_t index_col_stride, int fill,
                       uint32_t seed);

/* E2M1 operands with one UE8M0 scale per 32 K (the reference's "NVFP4" format).
 * `data` receives rows x K/2 bytes (two codes per byte, even k in the low nibble, `ld_bytes`
 * between rows, 16-byte aligned); `sf_packed` (optional) receives the scales in the packed
 * layout the kernels read, smb_sf_packed_bytes(rows, K/32) bytes; `sf_rowmajor` (optional)
 * receives them as plain [rows, K/32] bytes (exponent + 127).  `row0` is the global index of
 * the first row (N-sharding); `which` is 0 for A (seed 0x9E3779B9, scale rule of SFA) and 1
 * for B (seed 0x7F4A7C15, SFB).  Fills 1..4 are the reference's direct code/scale fills
 * (k1_e2m1_nibble / k1_generic_sf_exp, nvfp4/dense_gemm_nvfp4.cu:2279-2290, :2394-2398,
 * :2436-2437; verifier data_values / scale_values, dense_gemm_nvfp4_cpu_verifier.py:46-77).
 * Fills 5 and 6 have no reference counterpart: Gaussian FP32 source values (6: rounded to
 * bf16 first) pushed through the quantiser below. */
int smb_fill_fp4_device(uint8_t* data, int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor,
                        int64_t rows, int64_t K, uint64_t row0, int fill, int which, void* stream);
int smb_fill_fp4_host(uint8_t* data, int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor,
                      int64_t rows, int64_t K, uint64_t row0, int fill, int which);

/* FP32 -> E2M1 + UE8M0 quantiser, per row and per 32 consecutive k: scale exponent = the
 * smallest e with 6 * 2^e >= max|v| (0 for an all-zero block, clamped to [-126, 127]), each
 * value times 2^-e rounded to the nearest E2M1 code with ties to the even code.  No reference
 * counterpart (the reference generates codes directly); outputs as for the fills. */
int smb_quantize_mx_device(const float* src, int64_t ld_src, uint8_t* data, int64_t ld_bytes,
                           uint8_t* sf_packed, uint8_t* sf_rowmajor, int64_t rows, int64_t K,
                           void* stream);
int smb_quantize_mx_host(const float* src, int64_t ld_src, uint8_t* data, int64_t ld_bytes,
                         uint8_t* sf_packed, uint8_t* sf_rowmajor, int64_t rows, int64_t K);
/* NVFP4 proper (no counterpart in the reference, which documents the layout it would need,
 * nvfp4/dense_gemm_nvfp4.cu:109-129, but builds only the block-32 UE8M0 form): E2M1 codes with
 * one E4M3 scale per 16 consecutive k and a per-tensor factor chosen by the caller (typically
 * 448 * 6 / max|tensor|).  scale = e4m3_rne(max|v| * global_scale / 6), saturating at 448;
 * code = e2m1(v * global_scale / scale); the represented value is e2m1 * e4m3 / global_scale.
 * K % 32 == 0 (16-byte rows of codes); scales as [rows, K/16] bytes row-major and/or in the
 * packed layout of smb_sf_packed_bytes(rows, K/16), padding 0.  A GEMM over such operands is a
 * plan created with SMB_FLAG_SCALE_BLOCK16 and smb_fp4_plan_set_alpha(1 / (gs_a * gs_b)). */
int smb_quantize_nvf4_device(const float* src, int64_t ld_src, float global_scale, uint8_t* data,
                             int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor, int64_t rows,
                             int64_t K, void* stream);
int smb_quantize_nvf4_host(const float* src, int64_t ld_src, float global_scale, uint8_t* data,
                           int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor, int64_t rows,
                           int64_t K);
/* The same quantiser on BF16 bit patterns (every bf16 is an fp32: same rule, same result). */
int smb_quantize_mx_bf16_device(const uint16_t* src, int64_t ld_src, uint8_t* data, int64_t ld_bytes,
                                uint8_t* sf_packed, uint8_t* sf_rowmajor, int64_t rows, int64_t K,
                                void* stream);

/* Packed scale layout (sf_pack, nvfp4/dense_gemm_nvfp4.cu:2418-2435): bands of 128 rows, each
 * band (K/32 + 3) / 4 chunks of 512 bytes, byte (r, j) of a band at
 * (j / 4) * 512 + (r % 32) * 16 + (r / 32) * 4 + j % 4.  Padding holds 127 (scale 1). */
size_t smb_sf_packed_bytes(int64_t rows, int64_t kblocks);
int smb_sf_pack_host(const uint8_t* sf_rowmajor, int64_t rows, int64_t kblocks, uint8_t* packed);

/* Bit-pattern helpers, exported so that host-side known-answer tests can pin them the way the
 * reference's tests/8_tcgen05_mma_idesc_test.cu and tests/42_smem_desc_blackwell_test.cu do. */
uint64_t smb_debug_smem_desc(uint32_t smem_addr, uint32_t sbo_bytes, uint32_t lbo_bytes,
                             uint32_t swizzle_mode);
uint32_t smb_debug_idesc_bf16(int mma_m, int mma_n);
uint32_t smb_debug_idesc_mxf4(int mma_m, int mma_n, uint32_t sf_id_a, uint32_t sf_id_b, int ue8m0);
void smb_debug_tile_coords(int t, int tiles_m, int tiles_n, int group_m, int* tm, int* tn);
uint64_t smb_debug_sf_offset(uint32_t row, uint32_t kblock, uint32_t kblocks);
/* The tile list of the FP4 kernel with 256 x 384 tiles: `wide_tiles_n` full tiles per 256-row tile
 * row followed by `narrow_tiles_n` tiles of 256 columns (chosen so that the round-robin walk of
 * `clusters` clusters ends soonest), and tile t of that list (first column, full width or not).
 * Counterpart of the reference's static tile orders (nvfp4/dense_gemm_nvfp4.cu:380-434). */
void smb_debug_fp4_phases(int M, int N, int K, int clusters, int* wide_tiles_n, int* narrow_tiles_n);
void smb_debug_fp4_tile(int t, int tiles_m, int wide_tiles_n, int narrow_tiles_n, int group_m, int* tm,
                        int* col0, int* full_width);
/* The run split of the A-resident FP4 schedule (SMB_FLAG_TILE_N_192): every 256-row tile row is cut
 * into `chunks` runs of `run_len` tiles of 192 columns (the last run may be shorter); a cluster
 * loads the row's A panel once per run.  Returns 1 if the shape has that schedule (K <= 2048,
 * N >= 384), else 0 and leaves the outputs alone.  Counterpart of the reference's same-row runs
 * (nvfp4/dense_gemm_nvfp4.cu:372-434). */
int smb_debug_fp4_arun_split(int M, int N, int K, int clusters, int* chunks, int* run_len);
/* The cut of the last wave of the BF16 walk of SMB_FLAG_STREAM_K for `tiles` tiles of `kb` K blocks
 * on `clusters` clusters: out[0] whole-tile waves, out[1] tiles of the last wave, out[2] first K
 * block of the spare clusters' parts, out[3] such parts per spare cluster, out[4] equal K slices
 * per tile beyond the first (0: the form of out[2], out[3]).  Returns 1 if bf16_streamk_pays would
 * choose the walk for an M x N x K with that many tiles, else 0. */
int smb_debug_bf16_streamk_plan(long long tiles, int kb, int clusters, int* out);

/* ------------------------------------------------------------------------------------
 * Dense BF16 GEMM:  D[M,N] = bf16_rne( sum_k A[M,K] * BT[N,K] ), FP32 accumulate.
 * Stands in for dense_gemm_bf16_k0_impl + run_one_impl
 * (src/kernels/gemm/sm100a/dense_gemm_bf16.cu:86-234, :281-445).
 * A is row-major [M,K] (lda elements between rows), BT row-major [N,K] (ldb), D row-major
 * [M,N] (ldd).  Any M, N >= 1; K >= 8 and K % 8 == 0 (rows of A and BT must start on
 * 16-byte boundaries: lda % 8 == 0, ldb % 8 == 0, base pointers 16-byte aligned).
 * A D that is 16-byte aligned with ldd % 8 == 0 is written in whole 16-byte chunks: when the
 * row length is not a multiple of 8 elements, the row's padding up to the next multiple of 8
 * (always inside the pitch) is overwritten too.  Any other D is written element by element.
 * The same holds for the FP4 GEMM.
 * ---------------------------------------------------------------------------------- */
typedef struct smb_bf16_plan smb_bf16_plan;

/* Encode tensor maps and pick the tile configuration for one (A, BT, D) buffer set on the
 * current device.  `flags`: 0, or SMB_FLAG_* below. */
int smb_bf16_plan_create(smb_bf16_plan** plan, const void* a, const void* bt, void* d, int M, int N,
                         int K, int64_t lda, int64_t ldb, int64_t ldd, unsigned flags);
/* Launch the GEMM on `stream`.  Returns after enqueueing. */
int smb_bf16_plan_run(smb_bf16_plan* plan, void* stream);
/* Synchronise `stream` and translate the kernels' status word: SMB_OK, or SMB_ERR_DEVICE with
 * the role that gave up in smb_last_error(). */
int smb_bf16_plan_check(smb_bf16_plan* plan, void* stream);
int smb_bf16_plan_destroy(smb_bf16_plan* plan);
/* One line naming the kernel configuration the plan launches (tile shape, store path, CTAs per
 * SM), e.g. "bf16 tile 256x512 store=tma resident=1": what measurements are keyed by. */
int smb_bf16_plan_describe(smb_bf16_plan* plan, char* out, size_t capacity);
/* Self test of the bounded device waits: launches one CTA that waits `budget_cycles` SM clocks
 * (1 .. 2 000 000, i.e. at most about a millisecond) on an mbarrier nobody arrives at, gives up,
 * writes the "bounded-wait probe" status into the plan's status word and returns normally.  The
 * next smb_bf16_plan_check() therefore returns SMB_ERR_DEVICE with that message and clears the
 * word; the plan, the stream and the context stay usable.  The reference's wait helper spins
 * without a limit (src/primitives/33_mbarrier_try_wait.cuh:90-114) and has no such path. */
int smb_bf16_plan_wait_probe(smb_bf16_plan* plan, long long budget_cycles, void* stream);
/* Grouped GEMM for mixture-of-experts layers ("shared N and K, varying M", the case of the
 * reference's tile map composites/83_grouped_gemm_tile_map.cuh:71-101, which no kernel of its
 * tree uses): A [M_total, K] holds the rows of all groups back to back, every group padded to a
 * multiple of 256 rows; BT is [groups, N, K] stacked as [groups * N, K]; D is [M_total, N];
 * mtile_group_dev[t] (device memory, M_total / 256 ints, valid for the life of the plan) is the
 * group of rows [256 t, 256 t + 256).  Row r of D is A[r] times the BT of r's group.  Contiguous
 * operands (lda = ldb = K, ldd = N); run, check, destroy, peer copies and the gated epilogue as
 * for any other plan. */
int smb_bf16_grouped_plan_create(smb_bf16_plan** plan, const void* a, const void* bt_stacked, void* d,
                                 int M_total, int N, int K, int groups, const int* mtile_group_dev,
                                 unsigned flags);
/* The same for groups of ANY row count, the layout a token permutation yields without padding
 * (the tile map the reference describes, composites/83_grouped_gemm_tile_map.cuh:71-101, cuts
 * every group into tiles of its own): group g owns rows [group_offsets[g], group_offsets[g + 1]) of
 * A and D (host array of groups + 1 ints, offsets[0] = 0, M_total = offsets[groups]; empty groups
 * allowed).  The plan builds the row-tile table itself; the last tile of a group stores only the
 * group's own rows.  Contiguous operands (lda = ldb = K, ldd = N, or N / 2 with the gated epilogue). */
int smb_bf16_grouped_plan_create_offsets(smb_bf16_plan** plan, const void* a, const void* bt_stacked, void* d,
                                         int N, int K, int groups, const int* group_offsets, unsigned flags);
/* Tuning knobs (tests and sweeps): raster group height in tiles (0 = default), cap on
 * clusters (0 = all that fit). */
int smb_bf16_plan_tune(smb_bf16_plan* plan, int group_m, int max_clusters);

/* Role timers (the reference's counterpart is its WARP_PROF region markers, of which only a
 * no-op stub ships: src/primitives/_warp_prof_noop.cuh).  `counters` is device memory of
 * 8 int64 per CTA (2 CTAs per cluster, at most 2 * SM count CTAs), or NULL to switch the
 * timers off.  Per CTA: [0] load role cycles waiting for a free slot, [1] load role total,
 * [2] MMA role waiting for data, [3] MMA role waiting for an accumulator, [4] MMA role
 * total, [5] epilogue waiting for an accumulator, [6] epilogue total, [7] tiles done. */
int smb_bf16_plan_set_profile(smb_bf16_plan* plan, long long* counters);

/* One-shot convenience: plan + run + check + destroy on device pointers. */
int smb_dense_gemm_bf16(const void* a, const void* bt, void* d, int M, int N, int K, void* stream);

/* Host-buffer entry point, what a caller without device memory of its own uses:
 * allocates, copies A and BT to the device, runs, copies D back.  The reference driver does
 * these steps inline (dense_gemm_bf16.cu:293-307, :401-404). */
int smb_dense_gemm_bf16_host(const uint16_t* a, const uint16_t* bt, uint16_t* d, int M, int N, int K);

/* The same with the device buffers, plan and stream kept between calls: create once for a
 * shape, then every run uploads A and BT, launches, downloads D and synchronises.  Pass pinned
 * host memory for full copy bandwidth. */
typedef struct smb_bf16_host_ctx smb_bf16_host_ctx;
int smb_bf16_host_ctx_create(smb_bf16_host_ctx** ctx, int M, int N, int K);
int smb_bf16_host_ctx_run(smb_bf16_host_ctx* ctx, const uint16_t* a, const uint16_t* bt, uint16_t* d);
int smb_bf16_host_ctx_destroy(smb_bf16_host_ctx* ctx);

/* ------------------------------------------------------------------------------------
 * Dense block-scaled FP4 GEMM ("NVFP4" in the reference):
 *   D[M,N] = bf16_rne( sum_k (A[m,k] SFA[m,k/32]) (B[n,k] SFB[n,k/32]) ), FP32 accumulate.
 * Stands in for dense_gemm_nvfp4_k1_impl + run_one_k1
 * (src/kernels/gemm/sm100a/nvfp4/dense_gemm_nvfp4.cu:1705-2250, :2353-2700).
 * A: [M, K/2] bytes (two E2M1 codes per byte, even k low), B: [N, K/2] bytes, row pitches in
 * bytes (multiples of 16); SFA / SFB: UE8M0 bytes in the packed layout of
 * smb_sf_packed_bytes(); D: bf16 row-major.  Any M, N >= 1; K a multiple of 32.
 * Shapes with M <= 128 (decode: few activation rows against a large weight matrix B) run a
 * separate HBM-bound kernel that streams B once.  By default every CTA owns whole pairs of
 * 128-row weight tiles and needs no scratch memory; when a CTA count is forced
 * (smb_fp4_plan_tune) the (tile, K block) pairs are cut into equal ranges over those CTAs and
 * the fp32 partial sums of tiles shared between CTAs travel through plan-owned scratch.
 * ---------------------------------------------------------------------------------- */
typedef struct smb_fp4_plan smb_fp4_plan;
int smb_fp4_plan_create(smb_fp4_plan** plan, const void* a, const void* sfa, const void* b,
                        const void* sfb, void* d, int M, int N, int K, int64_t lda_bytes,
                        int64_t ldb_bytes, int64_t ldd, unsigned flags);
/* The same GEMM fed with BF16 activations [M, K] (row pitch ldx elements), as a model hands them
 * to a decode step: the plan owns the E2M1 codes and packed scales of A, and every
 * smb_fp4_plan_run first quantises `x_bf16` into them (the rule of smb_quantize_mx_*) and then
 * multiplies.  For M <= 128 this is ONE kernel.  From 17 rows up the decode kernel starts
 * streaming its weights at once, its CTAs share the quantisation of the activations between them
 * (each converts 1 / grid of the blocks after the previous kernel on the stream has completed),
 * meet on a counter, and only then load activations (SMB_FLAG_ACT_QUANT_SHARED forces this form
 * for fewer rows too).  Up to 16 rows every CTA converts all activations straight into its own
 * ring instead (SMB_FLAG_ACT_QUANT_PER_CTA; cheaper than the meeting for so few rows).
 * SMB_FLAG_ACT_QUANT_CHAINED selects a quantiser kernel chained in front, which is also what
 * runs above 128 rows.  All forms give the same bits.  The reference has no quantiser; its drivers generate codes and
 * scales directly (nvfp4/dense_gemm_nvfp4.cu:2279-2290). */
int smb_fp4_plan_create_bf16_activations(smb_fp4_plan** plan, const void* x_bf16, int64_t ldx,
                                         const void* b, const void* sfb, void* d, int M, int N, int K,
                                         int64_t ldb_bytes, int64_t ldd, unsigned flags);
/* Factor applied to every accumulator before the result is rounded to bf16; plans created with
 * SMB_FLAG_SCALE_BLOCK16 only (the product of the operands' inverse per-tensor factors). */
int smb_fp4_plan_set_alpha(smb_fp4_plan* plan, float alpha);
/* Grouped FP4 GEMM, the FP4 twin of smb_bf16_grouped_plan_create: B [groups * N, K/2] and its
 * scales (packed over all groups * N rows) stacked, N % 128 == 0, every group of A padded to a
 * multiple of 256 rows; SMB_FLAG_SCALE_BLOCK16 and the gated epilogue apply as usual. */
int smb_fp4_grouped_plan_create(smb_fp4_plan** plan, const void* a, const void* sfa, const void* b_stacked,
                                const void* sfb_stacked, void* d, int M_total, int N, int K, int groups,
                                const int* mtile_group_dev, unsigned flags);
/* Groups of any row count for the FP4 GEMM, with one restriction: every group starts on a multiple
 * of 128 rows (the packed scales of A come in bands of 128 rows), i.e. groups are padded to 128, not
 * to 256, and the last tile of a group stores only the group's own rows. */
int smb_fp4_grouped_plan_create_offsets(smb_fp4_plan** plan, const void* a, const void* sfa, const void* b_stacked,
                                        const void* sfb_stacked, void* d, int N, int K, int groups,
                                        const int* group_offsets, unsigned flags);
int smb_fp4_plan_run(smb_fp4_plan* plan, void* stream);
int smb_fp4_plan_check(smb_fp4_plan* plan, void* stream);
int smb_fp4_plan_destroy(smb_fp4_plan* plan);
int smb_fp4_plan_describe(smb_fp4_plan* plan, char* out, size_t capacity);
/* The bounded-wait self test on an FP4 plan's status word; see smb_bf16_plan_wait_probe. */
int smb_fp4_plan_wait_probe(smb_fp4_plan* plan, long long budget_cycles, void* stream);
/* Tuning: raster group height (0 = default), cluster cap (0 = all), L2 prefetch distance in
 * 256-wide K blocks (0 = off, negative = keep). */
int smb_fp4_plan_tune(smb_fp4_plan* plan, int group_m, int max_clusters, int prefetch);
/* Role timers, same layout as smb_bf16_plan_set_profile. */
int smb_fp4_plan_set_profile(smb_fp4_plan* plan, long long* counters);

/* One-shot on device pointers (packed scales). */
int smb_dense_gemm_nvfp4(const void* a, const void* sfa, const void* b, const void* sfb, void* d,
                         int M, int N, int K, void* stream);
/* Host buffers; the scales are given in their logical form, [rows, K/32] bytes row-major, and
 * are packed here (sf_pack in the reference driver, nvfp4/dense_gemm_nvfp4.cu:2418-2435). */
int smb_dense_gemm_nvfp4_host(const uint8_t* a, const uint8_t* sfa_rowmajor, const uint8_t* b,
                              const uint8_t* sfb_rowmajor, uint16_t* d, int M, int N, int K);

/* Host-buffer context, the FP4 twin of smb_bf16_host_ctx (the reference driver does these steps
 * inline: nvfp4/dense_gemm_nvfp4.cu:2418-2468 sf_pack and uploads, :2594-2610 download): create
 * once for a shape; every run uploads the E2M1 codes of A [M, K/2] and B [N, K/2] and their UE8M0
 * scales in logical form ([rows, K/32] bytes row-major), packs the scales on the device,
 * multiplies and downloads D [M, N] (bf16).  Uploads, GEMMs and downloads of row chunks of A
 * overlap.  With b == NULL and sfb_rowmajor == NULL a run reuses the B of the previous run on this
 * context (a decode step: weights stay on the device, activations travel).  Pass pinned host
 * memory for full copy bandwidth.  Synchronises before it returns. */
typedef struct smb_fp4_host_ctx smb_fp4_host_ctx;
int smb_fp4_host_ctx_create(smb_fp4_host_ctx** ctx, int M, int N, int K);
int smb_fp4_host_ctx_run(smb_fp4_host_ctx* ctx, const uint8_t* a, const uint8_t* sfa_rowmajor,
                         const uint8_t* b, const uint8_t* sfb_rowmajor, uint16_t* d);
int smb_fp4_host_ctx_destroy(smb_fp4_host_ctx* ctx);

/* Decode-shape FP4 GEMM (M <= 128) for callers that cannot allocate device memory where the
 * GEMM runs: a server whose start-up pool owns all of HBM, or a plugin living inside another
 * framework's allocator, where a cudaMalloc on the request path either fails or stalls every
 * stream of the device.  It has no counterpart in the reference.  Same operands and result as smb_dense_gemm_nvfp4 (packed scales, lda =
 * ldb = K/2 bytes, ldd = N); what the kernel needs besides its operands (a status word, and for
 * its stream-K work split tile counters and partial-sum slots) lives in a 2 MiB array built
 * into the library, so the call performs no cudaMalloc / cudaFree of any kind.
 *   - Work split: by default every CTA owns whole pairs of weight tiles and only the status
 *     word is used.  After smb_decode_noalloc_set_split(ctas > 0) the (tile, K block) pairs are
 *     cut into equal ranges over `ctas` CTAs (at most one per SM); the array must then hold one
 *     4-byte counter per 128 columns of N and two fp32 partial-tile slots (round_up(M,16) * 512
 *     bytes each) per CTA within smb_decode_noalloc_scratch_limit() bytes (2 MiB - 256): the CTA
 *     count is lowered to what fits, and a shape whose counters leave room for no CTA returns
 *     SMB_ERR_UNSUPPORTED.  The setting is process-wide, like the array.  The splits agree up
 *     to the order of a few fp32 additions.
 *   - The first call on a device looks up the array's device address; make that call outside
 *     any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents: what must start
 *     at zero (status word; counters for the stream-K split) is cleared on `stream` before each
 *     launch, and two calls that overlap on the GPU (different streams) corrupt each other.
 *   - Enqueues and returns.  smb_decode_noalloc_check(stream) synchronises `stream`, reads the
 *     status word into a host variable (no allocation) and returns SMB_ERR_DEVICE if the last
 *     call's kernel gave up a bounded wait. */
int smb_dense_gemm_nvfp4_decode_noalloc(const void* a, const void* sfa, const void* b,
                                        const void* sfb, void* d, int M, int N, int K, void* stream);
int smb_decode_noalloc_set_split(int ctas);
int smb_decode_noalloc_check(void* stream);
size_t smb_decode_noalloc_scratch_limit(void);

/* ----------------------------------------------------------------------------------
 * Column-sharded GEMM across the GPUs of one box (one process per GPU).  The reference is
 * single-GPU: nothing below has a counterpart there.  Rank r of g holds rows
 * [r N/g, (r+1) N/g) of BT and computes D[:, r N/g : (r+1) N/g].
 *
 * Fused all-gather: with peer copies set, the epilogue of a plan writes every box of D it
 * stores also into `count` (<= 7) further buffers with plain 16-byte stores, normally the
 * same [M, N/g] column slab inside the full row-major D of every other GPU, mapped into this
 * process with smb_peer_open().  dst[i] is the address of element (0, 0) of this plan's D in
 * destination i, `ld` the row pitch (elements) of all destinations.  Needs the aligned store
 * path (D 16-byte aligned, ldd % 8 == 0), N % 8 == 0, dst[i] 16-byte aligned, ld % 8 == 0.
 * The kernel waits on no other GPU; a destination is complete once the writing kernel has
 * completed (synchronise the stream, then tell the owner, e.g. with a barrier).
 * count = 0 switches the copies off.  Decode-path FP4 plans (M <= 128) refuse them. */
int smb_bf16_plan_set_peer_copies(smb_bf16_plan* plan, int count, void* const* dst, int64_t ld);
int smb_fp4_plan_set_peer_copies(smb_fp4_plan* plan, int count, void* const* dst, int64_t ld);

/* Fused scatter of a reduce-scatter: for the K-sharded (row-parallel) form, where every rank
 * computes a partial product over its slice of K and rank b is to own rows [b R, (b + 1) R) of
 * the sum.  With a row route set the plan does not write its D: rows of block b go to dst[b]
 * (<= 8 blocks), at their row inside the block, with plain 16-byte stores, dst[b] normally a
 * slot reserved for this rank inside rank b's receive buffer, mapped with smb_peer_open().
 * rows_per_block R % 256 == 0, blocks * R >= M; ld, N, alignment as for peer copies.
 * The kernel's walk over the tiles starts at row block `first_block`: give every rank a
 * different one (rank + 1, say), or all ranks deliver to the same owner at the same time and
 * its NVLink port is the bottleneck (measured at 8 GPUs: 206 GB/s sent per GPU with equal
 * starts, 526 GB/s with rotated ones).  blocks = 0 switches the route off.  Once all ranks' kernels have completed, rank b adds its
 * g slots up with smb_sum_slots_bf16_device (fp32 accumulation in slot order, one bf16
 * rounding; the partial products themselves were rounded to bf16 when they were stored). */
int smb_bf16_plan_set_row_route(smb_bf16_plan* plan, int blocks, void* const* dst, int rows_per_block,
                                int64_t ld, int first_block);
int smb_fp4_plan_set_row_route(smb_fp4_plan* plan, int blocks, void* const* dst, int rows_per_block,
                               int64_t ld, int first_block);
/* d[i] = bf16(sum_s slots[s][i]) for `count` consecutive slots of `elems` bf16 each (elems % 8
 * == 0, 16-byte-aligned buffers).  Stream-ordered. */
int smb_sum_slots_bf16_device(const void* slots, void* d, int count, int64_t elems, void* stream);

/* Device memory that other processes of the box can map: allocate, export a 64-byte handle
 * (send it to the peers by any host channel), map a peer's handle into this process, unmap,
 * free.  A mapped pointer is valid for kernels and copies of this process; peer access over
 * NVLink is switched on by the mapping. */
#define SMB_PEER_HANDLE_BYTES 64
int smb_peer_alloc(void** ptr, size_t bytes);
int smb_peer_export(void* ptr, unsigned char handle[SMB_PEER_HANDLE_BYTES]);
int smb_peer_open(const unsigned char handle[SMB_PEER_HANDLE_BYTES], void** ptr);
int smb_peer_close(void* ptr);
int smb_peer_free(void* ptr);
/* Waits for all work this process has queued on the current device.  Call it before telling the
 * other ranks that a peer-mapped buffer may be unmapped or freed: a GEMM with peer copies or a
 * row route may still be storing into it. */
int smb_device_synchronize(void);

/* The column slab of rank `rank` of `world`: an equal split of N whose slabs keep 16-byte
 * aligned bf16 rows (N % world == 0 and (N / world) % 8 == 0, else SMB_ERR_INVALID).  Pure
 * arithmetic, no device needed; the drivers' --shard=RANK/WORLD uses it. */
int smb_column_shard(int n_total, int world, int rank, int* n0, int* n_local);

/* Unfused path: an all-gather of the [M, N/g] slabs (NCCL concatenates them rank-major as
 * [g, M, N/g]) followed by this copy into row-major [M, g * n_local] (pitch ldd elements).
 * n_local % 8 == 0, both buffers 16-byte aligned, ldd % 8 == 0.  Stream-ordered. */
int smb_unshard_columns_device(const void* gathered, void* d, int g, int M, int n_local, int64_t ldd,
                               void* stream);

/* The all-gather itself behind the C ABI: NCCL over NVLink, resolved at run time (libnccl.so.2;
 * SMB_ERR_UNSUPPORTED when it cannot be loaded).  A communicator is either one rank of a
 * one-process-per-GPU job (rank 0 makes an id with smb_comm_unique_id, hands it to the others by
 * any host channel, every rank calls smb_comm_create with its device current), or one of `ndev`
 * communicators of a single process that drives several devices (smb_comm_create_all; devices
 * == NULL means 0 .. ndev - 1), which is what the drivers' --gpus=G --allgather uses.
 * smb_allgather_columns: `slab` is this rank's [M, n_local] bf16 result, `gathered` receives
 * all ranks' slabs rank-major as [world, M, n_local]; if d_full is not NULL the unshard copy
 * into row-major [M, world * n_local] (pitch ldd) follows on the same stream.  The _multi form
 * makes the calls of all devices of one process inside one NCCL group.  Stream-ordered; same
 * alignment rules as smb_unshard_columns_device.  smb_allgather_check applies the shape rules
 * only (no device or NCCL needed). */
#define SMB_COMM_ID_BYTES 128
typedef struct smb_comm smb_comm;
int smb_comm_unique_id(unsigned char id[SMB_COMM_ID_BYTES]);
int smb_comm_create(smb_comm** comm, const unsigned char id[SMB_COMM_ID_BYTES], int world, int rank);
int smb_comm_create_all(smb_comm** comms, int ndev, const int* devices);
int smb_comm_destroy(smb_comm* comm);
int smb_allgather_check(int world, int M, int n_local, int64_t ldd);
int smb_allgather_columns(smb_comm* comm, const void* slab, void* gathered, void* d_full, int M,
                          int n_local, int64_t ldd, void* stream);
int smb_allgather_columns_multi(smb_comm* const* comms, int ndev, const void* const* slabs,
                                void* const* gathered, void* const* d_full, int M, int n_local,
                                int64_t ldd, void* const* streams);

/* Host-buffer contexts of a column-sharded job (one process per GPU, `comm` from
 * smb_comm_create, kept by the caller for the life of the context): the context's N is this
 * rank's n_local columns, and every run takes only this rank's M / world rows of A (rows
 * [rank M / world, (rank + 1) M / world); for FP4 also of its row-major scales), its own shard
 * of BT / B, and returns its [M, n_local] slab of D.  The ranks complete A on every GPU with an
 * NCCL all-gather over NVLink inside the run, so the host sends every byte of A once per step
 * instead of once per GPU.  M % world == 0.  All ranks must call run together. */
int smb_bf16_host_ctx_create_sharded(smb_bf16_host_ctx** ctx, int M, int n_local, int K, smb_comm* comm);
int smb_fp4_host_ctx_create_sharded(smb_fp4_host_ctx** ctx, int M, int n_local, int K, smb_comm* comm);

#define SMB_FLAG_NONE 0u
#define SMB_FLAG_FORCE_PLAIN_STORE 1u /* use the non-TMA epilogue even when D is aligned */
#define SMB_FLAG_TILE_N_128 2u        /* force 256 x 128 tiles */
#define SMB_FLAG_TILE_N_64 4u         /* force 256 x 64 tiles */
#define SMB_FLAG_TILE_N_256 8u        /* force 256 x 256 tiles, two accumulator banks */
#define SMB_FLAG_TILE_N_512 16u       /* force 256 x 512 tiles, one accumulator set */
#define SMB_FLAG_TILE_N_384 32u       /* FP4 only: force 256 x 384 tiles */
#define SMB_FLAG_STREAM_K 524288u     /* BF16 only: 256 x 512 tiles with their K loops cut where the clusters' shares
                                         end, partial sums through a workspace the plan owns (chosen by itself where
                                         whole tiles would leave much of the last wave idle) */
#define SMB_FLAG_TILE_N_192 262144u   /* FP4 only: force the A-resident schedule (256 x 192 tiles, two accumulator
                                         sets, K <= 2048, N >= 384); SMB_ERR_UNSUPPORTED where it has no form */
 /* Hand tiles out through the hardware work queue (clusterlaunchcontrol.try_cancel, the
  * reference's CLC scheduler, blocks/97_sched_warp_clc.cuh) instead of the static stride walk. */
#define SMB_FLAG_DYNAMIC_TILES 256u
/* The GEMM kernels are launched with programmatic stream serialisation: their prologue overlaps
 * the tail of the previous kernel on the stream and by default they wait for that kernel before
 * loading anything.  With this flag the caller vouches that the operand (and scale) buffers are
 * not written by that previous kernel; then only the stores to D wait, and loads and MMAs of
 * this launch overlap the previous kernel's tail (what the reference drivers' timing loops do:
 * dense_gemm_bf16.cu:355-361, blocks/97_sched_warp_clc.cuh:118-129). */
#define SMB_FLAG_OPERANDS_STATIC 1024u
/* Stronger: the previous kernel on the stream neither writes this plan's operands nor reads or
 * writes its D, so this launch waits for nothing and consecutive launches may run side by side
 * and finish in any order (later stream operations still wait for all of them).  This is the
 * launch behaviour of the reference kernels, whose only wait is compiled out
 * (blocks/97_sched_warp_clc.cuh:108, USE_GRIDDEP_WAIT = false); the drivers here use it in their
 * timing loops, which launch the same GEMM repeatedly.  Implies SMB_FLAG_OPERANDS_STATIC.  Tiled
 * kernels only; the decode kernel ignores it (its scratch protocol needs the order). */
#define SMB_FLAG_LAUNCH_INDEPENDENT 4096u
/* Gated-activation epilogue, the reference's SwiGLU epilogue block
 * (blocks/93_epi_warp_blackwell.cuh:439-596, composites/130_swiglu_act.cuh): the rows of BT (B
 * for FP4) are interleaved, row 2n = up projection n, row 2n + 1 = gate projection n, and the
 * kernel stores D[m, n] = bf16(silu(acc[m, 2n + 1]) * acc[m, 2n]) with silu(z) = 0.5 z (1 +
 * tanh(z / 2)) on the hardware tanh approximation.  D is [M, N / 2] (ldd >= N / 2, 16-byte
 * aligned, ldd % 8 == 0), N even; the plan uses 256-wide tiles.  Tiled kernels only. */
#define SMB_FLAG_EPILOGUE_SWIGLU 8192u
/* FP4 plans: the scale buffers hold one E4M3 byte per 16 K (NVFP4 proper, issued as
 * kind::mxf4nvf4.block_scale.scale_vec::4X) instead of one UE8M0 byte per 32 K, packed with
 * smb_sf_packed_bytes(rows, K / 16).  K % 64 == 0; 256-wide tiles, or for M <= 128 the
 * dual-tile form of the decode kernel. */
#define SMB_FLAG_SCALE_BLOCK16 16384u
#define SMB_FLAG_NO_DECODE 64u        /* FP4 only: M <= 128 through the tiled kernel, not the decode kernel */
#define SMB_FLAG_NO_LAUNCH_OVERLAP 128u /* decode kernel: no programmatic dependent launch */
/* Decode kernel (FP4, M <= 128).  By default a CTA multiplies two adjacent weight tiles against
 * one copy of the activations; up to 64 rows the weights are the rows of the instruction and the
 * activations its columns, above 64 rows (and N <= 256 x SMs) the other way round.  DECODE_DUAL
 * forces the two-tile form with the weights as rows for every M, DECODE_SINGLE the form with one
 * weight tile per activation box.  All forms give the same bits. */
#define SMB_FLAG_DECODE_DUAL 512u
#define SMB_FLAG_DECODE_SINGLE 2048u
/* Plans created from BF16 activations, M <= 128: how the activations are quantised (default: once
 * per launch, shared by the CTAs of the decode kernel); see smb_fp4_plan_create_bf16_activations. */
#define SMB_FLAG_ACT_QUANT_PER_CTA 32768u
#define SMB_FLAG_ACT_QUANT_CHAINED 65536u
#define SMB_FLAG_ACT_QUANT_SHARED 131072u

#ifdef __cplusplus
}
#endif

#endif /* STRATA_MASONRY_B200_H_ */
