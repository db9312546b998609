// Skinny ("decode") block-scaled FP4 GEMM for sm_100a:  D[M,N] = bf16( X[M,K] . W[N,K]^T ) with
// M <= 128 activation rows and a large weight matrix W.  The work is one pass over W (N*K/2 bytes
// plus scales), so the bound is HBM bandwidth, not the tensor pipe.
//
// The reference has no kernel for this shape class (its NVFP4 driver requires M % 256 == 0,
// src/kernels/gemm/sm100a/nvfp4/dense_gemm_nvfp4.cu:2976-2985); numerics and operand formats
// are those of dense_gemm_nvfp4_k1_impl (same file, :1705-2250).
//
// Design: operands are swapped so that the weights fill the 128 rows of a 1-CTA tcgen05.mma
// (M_mma = 128 weight rows, N_mma = padded activation rows, K = 64 per instruction); the
// accumulator of a weight tile is 128 lanes x M_pad fp32 columns in tensor memory.
// The (weight tile, 256-wide K block) pairs are numbered n_tile * KB + kb and cut into one
// contiguous range per CTA ("stream-K"): every SM streams the same number of bytes from HBM
// whatever the tile count.  A range covers parts of up to three tiles:
//   * a tile covered completely by one CTA is converted to bf16 and stored directly;
//   * of a partly covered tile every contributor but the last to arrive writes its fp32 partial
//     sums into a scratch slot of its own and raises a per-tile counter by the K blocks it
//     contributed; the CTA that completes the count adds the other parts to its own, converts,
//     stores, and resets the counter for the next call.
// Warp roles (256 threads): warp 0 TMA producer, warp 1 MMA issue + TMEM owner, warp 2 scale
// copies (tcgen05.cp, issued apart from the MMAs so that they overlap them), warp 3 idle,
// warps 4-7 epilogue (warp w reads TMEM lanes 32 (w % 4) .. +31).
//
// That is the single-tile form, kept for callers that ask for a CTA count.  The default is the
// dual-tile form further down (two weight tiles per activation box, whole tile pairs per CTA, no
// scratch; 384 threads: a second group of epilogue warps), with two variants of its own: above 64
// activation rows the operands are not swapped (one 128 x 256 instruction per K step), and up to
// 16 rows BF16 activations are quantised by extra warps of the kernel itself (640 threads).
#include "epilogue.cuh"
#include "formats.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace smb {

namespace fp4d {

constexpr int kThreads = 256;
constexpr int kDualThreads = 384;    // dual-tile form: a second group of four epilogue warps
constexpr int kQuantWarps = 8;
constexpr int kFusedThreads = kDualThreads + 32 * kQuantWarps;   // + warps that quantise BF16 activations into the ring
constexpr int kBlockKBytes = 128;     // 256 E2M1 values
constexpr int kBlockK = 256;
constexpr int kWBytes = 128 * kBlockKBytes;   // 16 KiB weight box
constexpr int kSfBytes = 1024;        // one 128-row band x 8 scales (two 512-byte cells)
constexpr int kSlotCols = 16;         // SFW cells (8 columns) + SFX cells (8 columns) per stage
constexpr int kMaxStages = 16;
constexpr int kDefaultStages = 6;
constexpr int kDualFromPad = 16;      // padded activation rows from which two tiles share one activation box
constexpr int kWholeTileStages = 8;
constexpr int kMaxPad = 128;         // activation rows, padded
constexpr int kStageRows = 64;       // activation rows of D staged in shared memory per TMA store
constexpr int kBarrierBytes = 1024;

struct Params {
  int M, N, K;
  int m_pad;          // activation rows rounded up to 16
  int stages;
  int stage_bytes;
  int tmem_cols;      // 512 with one CTA per SM, 256 with two
  int bank_stride;    // columns between the two accumulator banks (128 or 64)
  int ldd;
  uint16_t* d;
  float* scratch;     // [2 * CTAs][m_pad / 4][128] float4 partial sums (need no clearing)
  int* counters;      // [tiles] K blocks accumulated so far (zero between calls)
  int d_tma;          // 1: D is written by TMA from a transposed staging buffer
  int tiles_per_cta;  // > 0: CTA b owns the whole tiles [b t, (b+1) t); 0: stream-K ranges
  int* status;
  int activations_dynamic;  // 1: X and SFX are written by the previous kernel on the stream
};

// Tensor memory read-back of 16 columns.
__device__ __forceinline__ void ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  tmem_ld_32x32b_x16(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ uint16_t to_bf16(float v) {
  uint32_t b = __float_as_uint(v);
  return static_cast<uint16_t>((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}

__device__ __forceinline__ void decode_body(const CUtensorMap& tmap_w, const CUtensorMap& tmap_x,
                                            const CUtensorMap& tmap_sfw, const CUtensorMap& tmap_sfx,
                                            const CUtensorMap& tmap_d, const Params& p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int stages = p.stages;
  const uint32_t ring_base = smem_base;
  const uint32_t stage_base = ring_base + static_cast<uint32_t>(stages * p.stage_bytes);   // D staging
  const uint32_t bar_base = stage_base + static_cast<uint32_t>((p.m_pad < kStageRows ? p.m_pad : kStageRows) * 256);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto sf_full_bar = [&](int s) { return bar_base + 8u * (2 * kMaxStages + s); };
  auto sf_ready_bar = [&](int s) { return bar_base + 8u * (3 * kMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (4 * kMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (4 * kMaxStages + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (4 * kMaxStages + 4);
  const uint32_t last_flag = tmem_slot + 8;   // epilogue broadcast: 1 = this CTA completes the tile

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int tiles = (p.N + 127) / 128;
  const long long units = static_cast<long long>(tiles) * num_kb;
  // Work split.  Default: whole tiles, t per CTA, on ceil(tiles / t) CTAs: no tile is shared, so
  // nothing goes through the scratch.  HBM is saturated by far fewer than all SMs (112 CTAs with
  // two tiles each: 18.0 us at M = 16, N = 28672; 148 CTAs with 1.51 tiles each and the fix-up
  // that implies: 19.4 us; the gap grows with M and for small N), so idle SMs cost nothing.
  // Stream-K ranges over all CTAs remain for callers that ask for a CTA count.
  const long long t_first = static_cast<long long>(blockIdx.x) * p.tiles_per_cta;
  const long long t_last = t_first + p.tiles_per_cta;
  const long long u_begin = p.tiles_per_cta > 0 ? (t_first < tiles ? t_first : tiles) * num_kb
                                                : units * blockIdx.x / gridDim.x;
  const long long u_end = p.tiles_per_cta > 0 ? (t_last < tiles ? t_last : tiles) * num_kb
                                              : units * (blockIdx.x + 1) / gridDim.x;
  const uint32_t x_off = kWBytes;
  const uint32_t sfw_off = kWBytes + static_cast<uint32_t>(p.m_pad) * kBlockKBytes;
  const uint32_t sfx_off = sfw_off + kSfBytes;

  // Let the next launch on the stream start its prologue and its (read-only) operand loads
  // while this grid is still running; it waits before it touches D or the scratch.
  griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(sf_full_bar(s), 1);
      mbar_init(sf_ready_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4);
    }
    fence_mbar_init_cluster();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_sfw);
    tma_prefetch_desc(&tmap_sfx);
    if (p.d_tma) tma_prefetch_desc(&tmap_d);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, static_cast<uint32_t>(p.tmem_cols));
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    // (All role loops are walked by the whole warp with one elected lane issuing: warp-uniform
    // control flow keeps descriptors and addresses in uniform registers.)
    {
      const uint64_t stream_once = l2_policy_evict_first();   // weights: read exactly once
      const uint64_t keep = l2_policy_evict_last();           // activations: re-read by every CTA
      int s = 0;
      uint32_t ph = 0;
      long long u = u_begin;
      const uint32_t op_bytes = kWBytes + static_cast<uint32_t>(p.m_pad) * kBlockKBytes;
      if (p.activations_dynamic) {
        // The activations (codes and scales) come from the kernel launched just before this one
        // (the quantiser): fill the whole ring with weights and weight scales first, they do not
        // depend on it, then wait for that kernel and add the activation boxes to the same
        // stages.  Each barrier expects the bytes of both parts, so a stage is full only when
        // both have landed.
        const int pre = (u_end - u_begin) < stages ? static_cast<int>(u_end - u_begin) : stages;
        for (int i = 0; i < pre; ++i) {
          const long long uu = u_begin + i;
          const int tile = static_cast<int>(uu / num_kb);
          const int kb = static_cast<int>(uu - static_cast<long long>(tile) * num_kb);
          const uint32_t dst = ring_base + static_cast<uint32_t>(i * p.stage_bytes);
          if (elect_one()) {
            mbar_arrive_expect_tx(sf_full_bar(i), 2 * kSfBytes);
            tma_load_2d_cta_hint(dst + sfw_off, &tmap_sfw, sf_full_bar(i), kb * 128, tile, stream_once);
            mbar_arrive_expect_tx(full_bar(i), op_bytes);
            tma_load_2d_cta_hint(dst, &tmap_w, full_bar(i), kb * kBlockKBytes, tile * 128, stream_once);
          }
          __syncwarp();
        }
        griddep_wait();
        for (int i = 0; i < pre; ++i) {
          const long long uu = u_begin + i;
          const int kb = static_cast<int>(uu % num_kb);
          const uint32_t dst = ring_base + static_cast<uint32_t>(i * p.stage_bytes);
          if (elect_one()) {
            tma_load_2d_cta_hint(dst + sfx_off, &tmap_sfx, sf_full_bar(i), kb * 128, 0, keep);
            tma_load_2d_cta_hint(dst + x_off, &tmap_x, full_bar(i), kb * kBlockKBytes, 0, keep);
          }
          __syncwarp();
        }
        u += pre;
        if (pre == stages) ph ^= 1u; else s = pre;
      }
      for (; u < u_end; ++u) {
        const int tile = static_cast<int>(u / num_kb);
        const int kb = static_cast<int>(u - static_cast<long long>(tile) * num_kb);
        if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
          report_status(p.status, kDevTimeoutProducer);
          for (int i = 0; i < 64; ++i) __nanosleep(1000);
          break;
        }
        const uint32_t dst = ring_base + static_cast<uint32_t>(s * p.stage_bytes);
        if (elect_one()) {
          mbar_arrive_expect_tx(sf_full_bar(s), 2 * kSfBytes);
          tma_load_2d_cta_hint(dst + sfw_off, &tmap_sfw, sf_full_bar(s), kb * 128, tile, stream_once);
          tma_load_2d_cta_hint(dst + sfx_off, &tmap_sfx, sf_full_bar(s), kb * 128, 0, keep);
          mbar_arrive_expect_tx(full_bar(s), op_bytes);
          tma_load_2d_cta_hint(dst, &tmap_w, full_bar(s), kb * kBlockKBytes, tile * 128, stream_once);
          tma_load_2d_cta_hint(dst + x_off, &tmap_x, full_bar(s), kb * kBlockKBytes, 0, keep);
        }
        __syncwarp();
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issue
    {
      int s = 0;
      uint32_t ph = 0;
      int seg = 0;
      bool ok = true;
      long long u = u_begin;
      while (u < u_end && ok) {
        const int tile = static_cast<int>(u / num_kb);
        const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * num_kb);
        const long long seg_end = (static_cast<long long>(tile) + 1) * num_kb < u_end
                                      ? (static_cast<long long>(tile) + 1) * num_kb : u_end;
        const int count = static_cast<int>(seg_end - u);
        const int bank = seg & 1;
        if (!mbar_wait(acc_empty_bar(bank), (static_cast<uint32_t>(seg >> 1) & 1u) ^ 1u)) {
          report_status(p.status, kDevTimeoutMmaAcc);
          break;
        }
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + static_cast<uint32_t>(bank * p.bank_stride);
        for (int i = 0; i < count; ++i) {
          if (!mbar_wait(full_bar(s), ph) || !mbar_wait(sf_ready_bar(s), ph)) {
            report_status(p.status, kDevTimeoutMmaFull);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t stage = ring_base + static_cast<uint32_t>(s * p.stage_bytes);
          const uint32_t sf_t = tmem_base + static_cast<uint32_t>(2 * p.bank_stride + s * kSlotCols);
          const uint64_t desc_w = make_smem_desc(stage, 1024, 16, kSwizzle128B);
          const uint64_t desc_x = make_smem_desc(stage + x_off, 1024, 16, kSwizzle128B);
          if (elect_one()) {
#pragma unroll
            for (int ki = 0; ki < 4; ++ki) {
              const uint32_t sf_id = (ki & 1) ? 2u : 0u;
              const uint32_t cell = static_cast<uint32_t>(ki >> 1);
              const uint32_t idesc = make_idesc_mxf4(128, p.m_pad, sf_id, sf_id, true);
              mma_mxf4_ss<1>(acc, desc_w + 2u * ki, desc_x + 2u * ki, idesc, sf_t + 4u * cell,
                             sf_t + 8u + 4u * cell, (i > 0 || ki > 0) ? 1u : 0u);
            }
            mma_commit_1cta(empty_bar(s));
          }
          __syncwarp();
          if (++s == stages) { s = 0; ph ^= 1u; }
        }
        (void)kb0;
        if (ok && elect_one()) mma_commit_1cta(acc_full_bar(bank));
        __syncwarp();
        u = seg_end;
        ++seg;
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------- scale copies
    {
      int s = 0;
      uint32_t ph = 0;
      for (long long u = u_begin; u < u_end; ++u) {
        if (!mbar_wait(sf_full_bar(s), ph)) {
          report_status(p.status, kDevTimeoutSched);
          break;
        }
        tc_fence_after_sync();
        const uint32_t stage = ring_base + static_cast<uint32_t>(s * p.stage_bytes);
        const uint32_t sf_t = tmem_base + static_cast<uint32_t>(2 * p.bank_stride + s * kSlotCols);
        const uint64_t sfw_desc = make_smem_desc(stage + sfw_off, 128, 16, kSwizzleNone);
        const uint64_t sfx_desc = make_smem_desc(stage + sfx_off, 128, 16, kSwizzleNone);
        if (elect_one()) {
#pragma unroll
          for (int cell = 0; cell < 2; ++cell) {
            tmem_cp_32x128b_warpx4<1>(sf_t + 4u * cell, sfw_desc + cell * 32);
            tmem_cp_32x128b_warpx4<1>(sf_t + 8u + 4u * cell, sfx_desc + cell * 32);
          }
          mma_commit_1cta(sf_ready_bar(s));
        }
        __syncwarp();
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------- epilogue (4 warps)
    // Thread `row` (0..127) owns weight row `row` of the tile = output column n, and reads its
    // m_pad accumulator columns (one per activation row) from tensor memory.
    //
    // Output: the tile's [m_pad x 128] block of D is transposed through shared memory (at most 64
    // activation rows at a time) and written with one TMA store per chunk; where D is not
    // 16-byte aligned every thread writes its own 2-byte elements instead.
    //
    // Tiles shared by several CTAs: every contributor but the last to arrive writes its fp32
    // partial sums into a slot of its own (two per CTA: slot 0 for the segment its range starts
    // with, slot 1 for any other), raises the tile's counter by the K blocks it added, and the
    // CTA that completes the count adds the others' slots to its own part and stores the tile.
    // Plain 16-byte stores and loads, no atomics on the data and nothing to clear afterwards;
    // slot layout [m_pad / 4][128 rows] float4, so that a warp moves 512 contiguous bytes.
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const bool first_thread = (threadIdx.x == 128);
    const int groups = p.m_pad / 4;
    float4* const slots = reinterpret_cast<float4*>(p.scratch);
    const long long n_ctas = gridDim.x;
    auto range_begin = [&](long long cta) { return units * cta / n_ctas; };
    // Slot that CTA `cta` uses for its segment starting at unit `seg_start`.
    auto slot_of = [&](long long cta, long long seg_start) {
      const long long which = (seg_start == range_begin(cta)) ? 0 : 1;
      return slots + (cta * 2 + which) * groups * 128;
    };
    const int chunk_rows = p.m_pad < kStageRows ? p.m_pad : kStageRows;
    int seg = 0;
    bool waited_for_previous_grid = false;
    bool store_pending = false;     // first_thread: a TMA store may still be reading the staging buffer
    long long u = u_begin;

    // Writes the finished tile.  fetch(c, v) delivers the final fp32 values of columns c..c+15.
    auto store_tile = [&](int tile, auto&& fetch) {
      const int n = tile * 128 + row;
      if (p.d_tma) {
        for (int c0 = 0; c0 < p.m_pad; c0 += chunk_rows) {
          if (first_thread && store_pending) bulk_wait_group_read<0>();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          for (int c = c0; c < c0 + chunk_rows && c < p.m_pad; c += 16) {
            float v[16];
            fetch(c, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const uint32_t dst = stage_base + static_cast<uint32_t>((c - c0 + j) * 256 + row * 2);
              asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst), "h"(to_bf16(v[j])) : "memory");
            }
          }
          fence_proxy_async_smem();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (first_thread) {
            // Rows >= M and columns >= N of the box are clipped by the tensor map.
            tma_store_2d(&tmap_d, stage_base, tile * 128, c0);
            bulk_commit_group();
            store_pending = true;
          }
        }
      } else {
        for (int c = 0; c < p.m_pad; c += 16) {
          float v[16];
          fetch(c, v);
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c + j < p.M) p.d[static_cast<size_t>(c + j) * p.ldd + n] = to_bf16(v[j]);
            }
          }
        }
      }
    };

    while (u < u_end) {
      const int tile = static_cast<int>(u / num_kb);
      const long long tile_begin = static_cast<long long>(tile) * num_kb;
      const long long tile_end = tile_begin + num_kb;
      const long long seg_end = tile_end < u_end ? tile_end : u_end;
      const int count = static_cast<int>(seg_end - u);
      const int bank = seg & 1;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(bank * p.bank_stride);
      const bool whole = (count == num_kb);
      // CTAs whose ranges meet this tile: c_lo .. c_hi (this CTA among them).
      long long c_lo = 0, c_hi = 0;
      bool early = false;
      float pre[kMaxPad];
      if (!whole) {
        c_lo = tile_begin * n_ctas / units;
        while (c_lo + 1 < n_ctas && range_begin(c_lo + 1) <= tile_begin) ++c_lo;
        while (c_lo > 0 && range_begin(c_lo) > tile_begin) --c_lo;
        c_hi = (tile_end - 1) * n_ctas / units;
        while (c_hi + 1 < n_ctas && range_begin(c_hi + 1) < tile_end) ++c_hi;
        while (c_hi > 0 && range_begin(c_hi) >= tile_end) --c_hi;
        if (!waited_for_previous_grid) {
          // First touch of the counters and slots: the previous launch on the stream (which may
          // be this same kernel, started early under programmatic dependent launch) must be done.
          griddep_wait();
          waited_for_previous_grid = true;
        }
        // If every other part of the tile has been published already (the usual case for the
        // segment at the END of a range: the neighbour handled its part at the start of its own
        // range), add those parts up in registers while the MMAs of this segment are running.
        if (first_thread) {
          const int seen = atomicAdd(p.counters + tile, 0);
          const uint32_t f = (seen + count == num_kb) ? 1u : 0u;
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(last_flag), "r"(f) : "memory");
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t f;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(f) : "r"(last_flag) : "memory");
        early = (f != 0u);
        asm volatile("bar.sync 1, 128;" ::: "memory");   // everyone has read the flag word
        if (early) {
          __threadfence();
#pragma unroll
          for (int c = 0; c < kMaxPad; ++c) pre[c] = 0.0f;
          for (long long c = c_lo; c <= c_hi; ++c) {
            if (c == static_cast<long long>(blockIdx.x)) continue;
            const long long rb = range_begin(c);
            const float4* src = slot_of(c, rb > tile_begin ? rb : tile_begin);
#pragma unroll
            for (int g = 0; g < kMaxPad / 4; ++g) {
              if (g < groups) {
                const float4 q = __ldcg(src + g * 128 + row);
                pre[4 * g] += q.x; pre[4 * g + 1] += q.y; pre[4 * g + 2] += q.z; pre[4 * g + 3] += q.w;
              }
            }
          }
        }
      }
      if (!mbar_wait(acc_full_bar(bank), static_cast<uint32_t>(seg >> 1) & 1u)) {
        if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      if (!waited_for_previous_grid) {
        griddep_wait();   // first store to D
        waited_for_previous_grid = true;
      }
      if (whole || early) {
        if (early) {
          // Static register indexing: the column loop of store_tile is not unrolled, so add the
          // other parts here, 16 columns at a time, with a fully unrolled selector.
          store_tile(tile, [&](int c, float (&v)[16]) {
            ld16(taddr + c, v);
#pragma unroll
            for (int cc = 0; cc < kMaxPad; cc += 16) {
              if (cc == c) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += pre[cc + j];
              }
            }
          });
        } else {
          store_tile(tile, [&](int c, float (&v)[16]) { ld16(taddr + c, v); });
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(bank));
        if (early && first_thread) p.counters[tile] = 0;
      } else {
        // Publish this part, then find out whether it was the last one after all.
        float4* mine = slot_of(blockIdx.x, u);
        for (int c = 0; c < p.m_pad; c += 16) {
          float v[16];
          ld16(taddr + c, v);
#pragma unroll
          for (int q = 0; q < 4; ++q)
            __stcg(mine + (c / 4 + q) * 128 + row, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(bank));
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (first_thread) {
          const int before = atomicAdd(p.counters + tile, count);
          const uint32_t last = (before + count == num_kb) ? 1u : 0u;
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(last_flag), "r"(last) : "memory");
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t last;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(last) : "r"(last_flag) : "memory");
        if (last) {
          // All parts, this CTA's included, are in their slots: add them in CTA order.
          __threadfence();
          store_tile(tile, [&](int c, float (&v)[16]) {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            for (long long cc = c_lo; cc <= c_hi; ++cc) {
              const long long rb = range_begin(cc);
              const float4* src = slot_of(cc, rb > tile_begin ? rb : tile_begin);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float4 x = __ldcg(src + (c / 4 + q) * 128 + row);
                v[4 * q] += x.x; v[4 * q + 1] += x.y; v[4 * q + 2] += x.z; v[4 * q + 3] += x.w;
              }
            }
          });
          if (first_thread) p.counters[tile] = 0;
        }
        // The flag word is reused by the next partial segment.
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      u = seg_end;
      ++seg;
    }
    if (first_thread && store_pending) bulk_wait_group<0>();
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}


__global__ void __launch_bounds__(kThreads, 1)
gemm_nvfp4_decode_kernel(const __grid_constant__ CUtensorMap tmap_w,
                         const __grid_constant__ CUtensorMap tmap_x,
                         const __grid_constant__ CUtensorMap tmap_sfw,
                         const __grid_constant__ CUtensorMap tmap_sfx,
                         const __grid_constant__ CUtensorMap tmap_d,
                         const __grid_constant__ Params p) {
  decode_body(tmap_w, tmap_x, tmap_sfw, tmap_sfx, tmap_d, p);
}

// -----------------------------------------------------------------------------------
// Dual-tile form: one CTA multiplies TWO adjacent weight tiles per K block against one copy of the
// activations.  At M = 128 the activation box of a stage is as large as a weight box, and loaded
// once per weight tile it made the kernel L2 -> SM bound (250 MB per launch through that path at
// 112 CTAs, 100 GB/s per SM, for 125 MB of HBM traffic); loaded once per tile PAIR it is a third of
// the stage.  Whole tile pairs only: CTA b owns the pairs [b t, (b+1) t), nothing is shared between
// CTAs, so there is no scratch and no hand-over.  Roles as in the single form.
//   stage:  [W tile 0 16 KiB][W tile 1 16 KiB][X m_pad x 128 B][SFW0 1 KiB][SFW1 1 KiB][SFX 1 KiB]
//   TMEM :  banks of 2 x m_pad accumulator columns (two banks when they fit beside the scale
//           slots, else one), then per stage 24 scale columns (SFW0 | SFW1 | SFX).
// -----------------------------------------------------------------------------------
// Eight fp32 values -> eight E2M1 codes in one word (value 0 in the low nibble of byte 0), by the
// hardware conversion: round to nearest, ties to the even code, saturating at 6 -- what
// fmt::e2m1_encode computes with comparisons.  The first source of the instruction lands in the
// high nibble.
__device__ __forceinline__ uint32_t e2m1x8_from_f32(float f0, float f1, float f2, float f3, float f4,
                                                    float f5, float f6, float f7) {
  uint32_t out;
  asm("{\n\t"
      ".reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t"
      "}"
      : "=r"(out)
      : "f"(f0), "f"(f1), "f"(f2), "f"(f3), "f"(f4), "f"(f5), "f"(f6), "f"(f7));
  return out;
}

// One block of 32 BF16 values (sixteen words, even element in the low half) -> sixteen code bytes
// and the UE8M0 scale byte; the same result as fmt::quantize_mx_block on the widened values for
// finite inputs, in about four instructions per value instead of twenty-five: every CTA of the
// decode kernel quantises all activations again, so the conversion has to be cheap.
__device__ __forceinline__ void quantize_mx_block_bf16(const uint4 (&raw)[4], uint4* codes, uint32_t* scale_byte) {
  const uint32_t w[16] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w,
                          raw[2].x, raw[2].y, raw[2].z, raw[2].w, raw[3].x, raw[3].y, raw[3].z, raw[3].w};
  uint32_t m = 0u;
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t a = w[i] & 0x7FFF7FFFu;   // |x| of both halves
    asm("max.bf16x2 %0, %1, %2;" : "=r"(m) : "r"(m), "r"(a));
  }
  const float hi = __uint_as_float(m & 0xFFFF0000u), lo = __uint_as_float(m << 16);
  const int e = fmt::ue8m0_exponent(hi > lo ? hi : lo);
  const float inv = fmt::exp2i(-e);
  uint32_t out[4];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float f[8];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      // + 0 in the same rounding turns a negative zero into the positive one, as the comparison
      // form does; every other product is unchanged.
      f[2 * t] = __fmaf_rn(__uint_as_float(w[4 * q + t] << 16), inv, 0.0f);
      f[2 * t + 1] = __fmaf_rn(__uint_as_float(w[4 * q + t] & 0xFFFF0000u), inv, 0.0f);
    }
    out[q] = e2m1x8_from_f32(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7]);
  }
  *codes = make_uint4(out[0], out[1], out[2], out[3]);
  *scale_byte = static_cast<uint32_t>(e + 127);
}

struct DualParams {
  int M, N, K;
  int m_pad;
  int stages;
  int stage_bytes;
  int banks;            // 1 or 2 accumulator banks of 2 * m_pad columns
  int pairs_per_cta;
  int ldd;
  uint16_t* d;
  int* status;
  int d_tma;
  int activations_dynamic;
  float alpha;          // factor on every accumulator (block-16 scales: 1 / (global scale X x W))
  const uint16_t* x_src;   // kFused / act_spread: BF16 activations [M, K], quantised by the kernel itself
  long long ldx;           // elements between their rows
  // act_spread: the CTAs of the grid share the quantisation of x_src into act_codes / act_sf
  // (the buffers tmap_x / tmap_sfx read) and meet on act_counter before any of them loads
  // activations; see the comment at the top of decode_dual_body.
  int act_spread;
  // Gated epilogue (the tiled kernels' kSwiglu store mode): weight rows are interleaved, row 2n =
  // up projection n, row 2n + 1 = gate projection n; D is [M, N / 2] = silu(gate) * up.
  int swiglu;
  uint8_t* act_codes;                 // [M, K/2] E2M1 codes
  uint8_t* act_sf;                    // packed UE8M0 scales of X
  unsigned long long* act_counter;    // arrivals of all launches so far (never reset)
};


// act_spread: thread `t` of `threads` in this CTA converts its share of the M * K / 32 blocks
// of the BF16 activations; the grid's threads walk the blocks with a grid-wide stride, so that
// consecutive threads read consecutive 64-byte blocks of a row and write consecutive 16-byte
// code groups.
__device__ __forceinline__ void spread_quantize(const DualParams& p, int t, int threads) {
  const long long kblocks = p.K / 32;
  const long long total = static_cast<long long>(p.M) * kblocks;
  const long long stride = static_cast<long long>(gridDim.x) * threads;
  for (long long i = static_cast<long long>(blockIdx.x) * threads + t; i < total; i += stride) {
    const long long r = i / kblocks;
    const long long j = i - r * kblocks;
    const uint4* src = reinterpret_cast<const uint4*>(p.x_src + r * p.ldx + j * 32);
    uint4 raw[4] = {__ldg(src), __ldg(src + 1), __ldg(src + 2), __ldg(src + 3)};
    uint4 codes;
    uint32_t sb;
    quantize_mx_block_bf16(raw, &codes, &sb);
    *reinterpret_cast<uint4*>(p.act_codes + r * (p.K / 2) + j * 16) = codes;
    p.act_sf[fmt::sf_packed_offset(static_cast<uint32_t>(r), static_cast<uint32_t>(j),
                                   static_cast<uint32_t>(kblocks))] = static_cast<uint8_t>(sb);
  }
}

// V4: one E4M3 scale per 16 K (scale_vec::4X): four 4-byte scale cells per band and stage
// instead of two, 2 KiB of scales per band, 48 instead of 24 tensor-memory columns per slot.
//
// kWide (more than 64 activation rows, one tile pair per CTA): the operands are NOT swapped.  The
// activations are the 128 rows of the instruction and the two weight tiles its 256 columns, one
// instruction per K = 64 instead of two.  Why: the tensor core reads its operands from shared
// memory at about 64 bytes per clock, and two 128 x 128 instructions read 2 x (4 + 4) KiB where
// one 128 x 256 instruction reads 4 + 8 KiB; at M = 128 the swapped form spent 1024 cycles per
// stage on operand reads (17 us for K = 8192, more than the HBM time), this form 768.  The
// accumulator is then [m][n] as D is, and the epilogue is the tiled kernels' (32 x 64 boxes,
// staged in the ring, which is free once the only tile pair of the CTA is complete).
//   stage:  [W tile 0][W tile 1][X 128 x 128 B (rows >= m_pad never loaded, never stored)][SFW0][SFW1][SFX]
//   TMEM :  256 accumulator columns, then per stage [SFX cells][cell 0: SFW0 SFW1][cell 1: ...]
//
// kFused (swapped form, UE8M0 scales): the activations arrive as BF16 and eight extra warps
// quantise them straight into the ring: for every stage one warp reads the stage's 256 K values of
// all rows from global memory (L2-resident after the first CTA), computes scale and codes per 32
// values exactly as quantize_mx_bf16_kernel does, and writes the codes in the 128-byte-swizzled
// layout a TMA load would have produced and the scale bytes in the packed cell layout, then
// arrives on the stage's barriers beside the TMA producer.  Saves the separate quantiser launch
// of a decode step (M = 16, N = 28672, K = 8192: 21.9 us per step against 23.2 us chained).
//
// act_spread (any form with UE8M0 scales, run-time switch): the activations arrive as BF16 and
// the grid quantises them ONCE, every CTA a 1 / gridDim share, instead of once per CTA (kFused) or
// in a kernel of its own chained in front: the eight epilogue warps, idle until the first
// accumulator is complete, wait for the previous kernel on the stream (which may have written
// x_src, and whose CTAs may still be reading the code buffer), convert their share of the
// 32-value blocks into the plan's code and scale buffers, fence, and count the CTA in on a global
// counter.  The TMA producer, which has meanwhile filled the ring with weights, waits until all
// CTAs of this launch are counted in (bounded), orders the async proxy behind that, and loads the
// activation boxes like any others.  The counter only grows: a CTA that arrives as number `old`
// waits for (old / gridDim + 1) * gridDim, which every CTA of one launch computes alike because
// the arrivals of consecutive launches never mix (each waits for its predecessor's completion).
// All CTAs of the grid are resident at once (one per SM, grid <= SM count), so nobody waits for
// a CTA that cannot start.
template <bool V4, bool kWide, bool kFused>
__device__ __forceinline__ void decode_dual_body(const CUtensorMap& tmap_w, const CUtensorMap& tmap_x,
                                                 const CUtensorMap& tmap_sfw, const CUtensorMap& tmap_sfx,
                                                 const CUtensorMap& tmap_d, const DualParams& p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr int kCells = V4 ? 4 : 2;
  constexpr uint32_t kBandBytes = kCells * 512;            // scales of one 128-row band, one stage
  constexpr uint32_t kOperandCols = kCells * 4;            // tensor-memory columns of one band
  constexpr uint32_t kSlotCols = 3 * kOperandCols;         // SFW0 | SFW1 | SFX
  constexpr int kSfBox = kCells * 64;                      // 64-bit words per band and stage
  const int stages = p.stages;
  const uint32_t ring_base = smem_base;
  const uint32_t stage_base = ring_base + static_cast<uint32_t>(stages * p.stage_bytes);   // D staging
  const int chunk_rows = p.m_pad < kStageRows ? p.m_pad : kStageRows;
  const uint32_t bar_base = stage_base + static_cast<uint32_t>(chunk_rows * 256);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto sf_full_bar = [&](int s) { return bar_base + 8u * (2 * kMaxStages + s); };
  auto sf_ready_bar = [&](int s) { return bar_base + 8u * (3 * kMaxStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (4 * kMaxStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (4 * kMaxStages + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (4 * kMaxStages + 4);
  const uint32_t quant_bar = bar_base + 8u * (4 * kMaxStages + 6);      // act_spread: this CTA's share is done
  const uint32_t quant_target = bar_base + 8u * (4 * kMaxStages + 7);   // counter value to wait for (u64)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;
  const int tiles = (p.N + 127) / 128;
  const int pairs = (tiles + 1) / 2;
  const int q_begin = min(static_cast<int>(blockIdx.x) * p.pairs_per_cta, pairs);
  const int q_end = min(q_begin + p.pairs_per_cta, pairs);
  const uint32_t w1_off = kWBytes;
  const uint32_t x_off = 2 * kWBytes;
  const uint32_t sfw0_off = x_off + static_cast<uint32_t>(kWide ? kMaxPad : p.m_pad) * kBlockKBytes;
  const uint32_t sfw1_off = sfw0_off + kBandBytes;
  const uint32_t sfx_off = sfw1_off + kBandBytes;
  const uint32_t bank_cols = kWide ? 256u : 2u * static_cast<uint32_t>(p.m_pad);
  const uint32_t slot_base = static_cast<uint32_t>(p.banks) * bank_cols;
  // Epilogue warps 4-7 (group 0) and 8-11 (group 1) share the accumulator columns (= rows of D) of
  // every tile: group 0 takes the first half in units of 16, group 1 the rest.  With 16 columns
  // there is nothing to share and group 1 stays out of every barrier.
  const int epi_groups = p.m_pad >= 32 ? 2 : 1;
  const int cols_group0 = ((p.m_pad / 16 + 1) / 2) * 16;

  griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar(s), kFused ? 2 : 1);      // TMA producer (+ the quantising warp of the stage)
      mbar_init(empty_bar(s), 1);
      mbar_init(sf_full_bar(s), kFused ? 2 : 1);
      mbar_init(sf_ready_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4 * epi_groups);   // one arrival per working epilogue warp
    }
    mbar_init(quant_bar, 1);
    fence_mbar_init_cluster();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_w);
    tma_prefetch_desc(&tmap_x);
    tma_prefetch_desc(&tmap_sfw);
    tma_prefetch_desc(&tmap_sfx);
    if (p.d_tma) tma_prefetch_desc(&tmap_d);
  }
  if (warp == 1) {
    tmem_alloc<1>(tmem_slot, 512);
    tmem_relinquish<1>();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    const uint64_t stream_once = l2_policy_evict_first();
    const uint64_t keep = l2_policy_evict_last();
    const uint32_t op_bytes = 2 * kWBytes + (kFused ? 0u : static_cast<uint32_t>(p.m_pad) * kBlockKBytes);
    int s = 0;
    uint32_t ph = 0;
    bool waited = kFused || !p.activations_dynamic;
    int issued = 0;
    // Until the activations exist: the quantiser kernel launched just before this one has
    // completed, or (act_spread) every CTA of this grid has converted its share.
    auto wait_activations = [&]() -> bool {
      if (!p.act_spread) {
        griddep_wait();
        return true;
      }
      if (!mbar_wait(quant_bar, 0u)) return false;
      unsigned long long target;
      asm volatile("ld.shared.u64 %0, [%1];" : "=l"(target) : "r"(quant_target) : "memory");
      const long long t0 = clock64();
      while (true) {
        unsigned long long seen;
        asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(seen) : "l"(p.act_counter) : "memory");
        if (seen >= target) break;
        if (clock64() - t0 > SMB_WAIT_BUDGET_CYCLES) return false;
        __nanosleep(20);
      }
      // The codes and scales were written with ordinary stores by other CTAs; the loads below
      // go through the async proxy.
      asm volatile("fence.proxy.async;" ::: "memory");
      return true;
    };
    bool acts_ok = true;
    for (int q = q_begin; q < q_end && acts_ok; ++q) {
      for (int kb = 0; kb < num_kb; ++kb, ++issued) {
        // Activations written by the kernel launched just before this one (the quantiser): the
        // first ring of weight boxes goes out before the wait, the activation boxes after it.
        if (!waited && issued == stages) {
          if (!wait_activations()) {
            report_status(p.status, kDevTimeoutActivations);
            acts_ok = false;
            break;
          }
          waited = true;
          for (int j = 0; j < stages; ++j) {
            const int kbj = (j) % num_kb;
            const uint32_t dstj = ring_base + static_cast<uint32_t>(j * p.stage_bytes);
            if (elect_one()) {
              tma_load_2d_cta_hint(dstj + sfx_off, &tmap_sfx, sf_full_bar(j), kbj * kSfBox, 0, keep);
              tma_load_2d_cta_hint(dstj + x_off, &tmap_x, full_bar(j), kbj * kBlockKBytes, 0, keep);
            }
            __syncwarp();
          }
        }
        if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
          report_status(p.status, kDevTimeoutProducer);
          for (int i = 0; i < 64; ++i) __nanosleep(1000);
          q = q_end;
          break;
        }
        const uint32_t dst = ring_base + static_cast<uint32_t>(s * p.stage_bytes);
        if (elect_one()) {
          mbar_arrive_expect_tx(sf_full_bar(s), (kFused ? 2 : 3) * kBandBytes);
          tma_load_2d_cta_hint(dst + sfw0_off, &tmap_sfw, sf_full_bar(s), kb * kSfBox, 2 * q, stream_once);
          tma_load_2d_cta_hint(dst + sfw1_off, &tmap_sfw, sf_full_bar(s), kb * kSfBox, 2 * q + 1, stream_once);
          mbar_arrive_expect_tx(full_bar(s), op_bytes);
          tma_load_2d_cta_hint(dst, &tmap_w, full_bar(s), kb * kBlockKBytes, (2 * q) * 128, stream_once);
          tma_load_2d_cta_hint(dst + w1_off, &tmap_w, full_bar(s), kb * kBlockKBytes, (2 * q + 1) * 128,
                               stream_once);
          if (waited && !kFused) {
            tma_load_2d_cta_hint(dst + sfx_off, &tmap_sfx, sf_full_bar(s), kb * kSfBox, 0, keep);
            tma_load_2d_cta_hint(dst + x_off, &tmap_x, full_bar(s), kb * kBlockKBytes, 0, keep);
          }
        }
        __syncwarp();
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
    }
    if (!waited && acts_ok && !wait_activations()) {
      report_status(p.status, kDevTimeoutActivations);
      acts_ok = false;
    }
    if (!waited && acts_ok) {
      // Fewer units than ring slots: the activation boxes of everything issued are still owed.
      for (int j = 0; j < issued; ++j) {
        const int kbj = j % num_kb;
        const uint32_t dstj = ring_base + static_cast<uint32_t>(j * p.stage_bytes);
        if (elect_one()) {
          tma_load_2d_cta_hint(dstj + sfx_off, &tmap_sfx, sf_full_bar(j), kbj * kSfBox, 0, keep);
          tma_load_2d_cta_hint(dstj + x_off, &tmap_x, full_bar(j), kbj * kBlockKBytes, 0, keep);
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issue
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    int seg = 0;
    for (int q = q_begin; q < q_end && ok; ++q, ++seg) {
      const int bank = p.banks == 2 ? (seg & 1) : 0;
      const uint32_t use = static_cast<uint32_t>(p.banks == 2 ? (seg >> 1) : seg) & 1u;
      if (!mbar_wait(acc_empty_bar(bank), use ^ 1u)) {
        report_status(p.status, kDevTimeoutMmaAcc);
        break;
      }
      tc_fence_after_sync();
      const uint32_t acc0 = tmem_base + static_cast<uint32_t>(bank) * bank_cols;
      const uint32_t acc1 = acc0 + static_cast<uint32_t>(p.m_pad);
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(full_bar(s), ph) || !mbar_wait(sf_ready_bar(s), ph)) {
          report_status(p.status, kDevTimeoutMmaFull);
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t stage = ring_base + static_cast<uint32_t>(s * p.stage_bytes);
        const uint32_t sf_t = tmem_base + slot_base + static_cast<uint32_t>(s) * kSlotCols;
        const uint64_t desc_w0 = make_smem_desc(stage, 1024, 16, kSwizzle128B);
        const uint64_t desc_w1 = make_smem_desc(stage + w1_off, 1024, 16, kSwizzle128B);
        const uint64_t desc_x = make_smem_desc(stage + x_off, 1024, 16, kSwizzle128B);
        if (elect_one()) {
#pragma unroll
          for (int ki = 0; ki < 4; ++ki) {
            const uint32_t sf_id = V4 ? 0u : ((ki & 1) ? 2u : 0u);
            const uint32_t cell = static_cast<uint32_t>(V4 ? ki : (ki >> 1));
            const uint32_t accum = (kb > 0 || ki > 0) ? 1u : 0u;
            if (kWide) {
              // One instruction over both weight tiles: rows = activations, 256 columns = the 128
              // rows of W0 followed by those of W1 (adjacent in the stage), scales of cell c at
              // [SFX cell c] and [cell c: SFW0, SFW1].
              const uint32_t idesc = make_idesc_mxf4(128, 256, sf_id, sf_id, !V4);
              const uint32_t sx = sf_t + 4u * cell;
              const uint32_t sw = sf_t + kOperandCols + 8u * cell;
              if (V4) mma_nvf4_ss<1>(acc0, desc_x + 2u * ki, desc_w0 + 2u * ki, idesc, sx, sw, accum);
              else mma_mxf4_ss<1>(acc0, desc_x + 2u * ki, desc_w0 + 2u * ki, idesc, sx, sw, accum);
              continue;
            }
            const uint32_t idesc = make_idesc_mxf4(128, p.m_pad, sf_id, sf_id, !V4);
            const uint32_t s0 = sf_t + 4u * cell, s1 = sf_t + kOperandCols + 4u * cell;
            const uint32_t sx = sf_t + 2u * kOperandCols + 4u * cell;
            if (V4) {
              mma_nvf4_ss<1>(acc0, desc_w0 + 2u * ki, desc_x + 2u * ki, idesc, s0, sx, accum);
              mma_nvf4_ss<1>(acc1, desc_w1 + 2u * ki, desc_x + 2u * ki, idesc, s1, sx, accum);
            } else {
              mma_mxf4_ss<1>(acc0, desc_w0 + 2u * ki, desc_x + 2u * ki, idesc, s0, sx, accum);
              mma_mxf4_ss<1>(acc1, desc_w1 + 2u * ki, desc_x + 2u * ki, idesc, s1, sx, accum);
            }
          }
          mma_commit_1cta(empty_bar(s));
        }
        __syncwarp();
        if (++s == stages) { s = 0; ph ^= 1u; }
      }
      if (ok && elect_one()) mma_commit_1cta(acc_full_bar(bank));
      __syncwarp();
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------- scale copies
    int s = 0;
    uint32_t ph = 0;
    const int total = (q_end - q_begin) * num_kb;
    for (int i = 0; i < total; ++i) {
      if (!mbar_wait(sf_full_bar(s), ph)) {
        report_status(p.status, kDevTimeoutSched);
        break;
      }
      tc_fence_after_sync();
      const uint32_t stage = ring_base + static_cast<uint32_t>(s * p.stage_bytes);
      const uint32_t sf_t = tmem_base + slot_base + static_cast<uint32_t>(s) * kSlotCols;
      const uint64_t d0 = make_smem_desc(stage + sfw0_off, 128, 16, kSwizzleNone);
      const uint64_t d1 = make_smem_desc(stage + sfw1_off, 128, 16, kSwizzleNone);
      const uint64_t dx = make_smem_desc(stage + sfx_off, 128, 16, kSwizzleNone);
      if (elect_one()) {
#pragma unroll
        for (int cell = 0; cell < kCells; ++cell) {
          if (kWide) {
            tmem_cp_32x128b_warpx4<1>(sf_t + 4u * cell, dx + cell * 32);
            tmem_cp_32x128b_warpx4<1>(sf_t + kOperandCols + 8u * cell, d0 + cell * 32);
            tmem_cp_32x128b_warpx4<1>(sf_t + kOperandCols + 8u * cell + 4u, d1 + cell * 32);
          } else {
            tmem_cp_32x128b_warpx4<1>(sf_t + 4u * cell, d0 + cell * 32);
            tmem_cp_32x128b_warpx4<1>(sf_t + kOperandCols + 4u * cell, d1 + cell * 32);
            tmem_cp_32x128b_warpx4<1>(sf_t + 2u * kOperandCols + 4u * cell, dx + cell * 32);
          }
        }
        mma_commit_1cta(sf_ready_bar(s));
      }
      __syncwarp();
      if (++s == stages) { s = 0; ph ^= 1u; }
    }
  } else if (warp >= 4 && (warp < 8 || (warp < 12 && epi_groups == 2))) {
    // ------------------------------------------------------------- epilogue (4 or 8 warps)
    // Thread (quarter, lane) owns weight row n = quarter * 32 + lane of a tile, i.e. one lane of
    // tensor memory, whose columns are the rows m of D: the tile comes out transposed and goes
    // through shared memory ([m][128 n] bf16, 256 bytes per m) to a TMA store.
    const int quarter = warp & 3;
    const int group = (warp - 4) >> 2;
    const int row = quarter * 32 + lane;
    const int col_begin = group == 0 ? 0 : cols_group0;
    const int col_end = (group == 0 && epi_groups == 2) ? cols_group0 : p.m_pad;
    const int epi_threads = 128 * epi_groups;
    const bool first_thread = (threadIdx.x == 128);
    bool store_pending = false;
    bool waited_for_previous_grid = false;
    int seg = 0;
    // Gated epilogue in the swapped forms: a thread holds one weight row, so the (up, gate) pair
    // of an output sits in two neighbouring lanes; the even lane gets the gate from its
    // neighbour, applies the activation and stores output column row / 2 of the tile's 64.
    const bool gated = p.swiglu != 0;
    const bool writer = !gated || (lane & 1) == 0;
    const int out_row = gated ? (row >> 1) : row;                 // column inside the tile's output block
    const uint32_t out_pitch = gated ? 128u : 256u;               // bytes per activation row in the staging block
    const int out_tile_cols = gated ? 64 : 128;
    const int n_out = gated ? p.N / 2 : p.N;
    auto finish = [&](float (&v)[16]) {
      if (V4) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= p.alpha;
      }
      if (gated) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float other = __shfl_xor_sync(0xffffffffu, v[j], 1);
          v[j] = swiglu_f32(other, v[j]);     // meaningful in even lanes: own = up, neighbour = gate
        }
      }
    };
    if (p.act_spread) {
      // This CTA's share of the activation quantiser (see the top of this function); the four
      // warps 8-11 take part even where they have no accumulator columns to drain.
      griddep_wait();
      waited_for_previous_grid = true;
      spread_quantize(p, static_cast<int>(threadIdx.x) - 128, 128 * epi_groups);
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");
      if (first_thread) {
        const unsigned long long old = atomicAdd(p.act_counter, 1ull);
        const unsigned long long target = (old / gridDim.x + 1ull) * gridDim.x;
        asm volatile("st.shared.u64 [%0], %1;" ::"r"(quant_target), "l"(target) : "memory");
        mbar_arrive(quant_bar);
      }
    }
    for (int q = q_begin; q < q_end; ++q, ++seg) {
      const int bank = p.banks == 2 ? (seg & 1) : 0;
      const uint32_t use = static_cast<uint32_t>(p.banks == 2 ? (seg >> 1) : seg) & 1u;
      if (!mbar_wait(acc_full_bar(bank), use)) {
        if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      if (!waited_for_previous_grid) {
        griddep_wait();   // first store to D
        waited_for_previous_grid = true;
      }
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(bank) * bank_cols;
      if constexpr (kWide) {
        // Lanes are rows of D, columns are columns of D: warp group g takes weight tile 2 q + g.
        // The CTA has this one tile pair, so the ring is free and stages the 32 x 64 boxes.
        PeerCopies none;
        none.count = 0;
        none.route_rows = 0;
        StoreTarget out;
        out.tmap_d = &tmap_d;
        out.d_ptr = p.d;
        out.ldd = p.ldd;
        out.M = p.M;
        out.N = p.swiglu ? p.N / 2 : p.N;
        out.peers = &none;
        out.alpha = p.alpha;
        out.row_end = p.M;
        const uint32_t sbuf = ring_base + static_cast<uint32_t>((warp - 4) * kStoreBufBytes);
        const uint32_t release = mapa_u32(acc_empty_bar(bank), 0);
        const int col0 = (2 * q + group) * 128;
        if (p.d_tma && p.swiglu) {
          // 128 accumulator columns = one weight tile = 64 gated outputs = one store box.
          drain_and_store<128, true, true, V4>(tbase + static_cast<uint32_t>(group * 128), sbuf, out,
                                               quarter * 32, col0, release, lane);
          drain_store_groups<true>(lane);
        } else if (p.d_tma) {
          drain_and_store<128, true, false, V4>(tbase + static_cast<uint32_t>(group * 128), sbuf, out,
                                                quarter * 32, col0, release, lane);
          drain_store_groups<true>(lane);
        } else {
          drain_and_store<128, false, false, V4>(tbase + static_cast<uint32_t>(group * 128), sbuf, out,
                                                 quarter * 32, col0, release, lane);
        }
        continue;
      }
      if (p.d_tma && q == q_end - 1) {
        // Last tile pair of this CTA: every load has been consumed (the accumulators are
        // complete), so the whole ring is free and takes both transposed tiles at once,
        // [sub][m][128 n]; no chunking, one barrier, then all stores.
        for (int sub = 0; sub < 2; ++sub) {
          if (2 * q + sub >= tiles) break;
          for (int c = col_begin; c < col_end; c += 16) {
            float v[16];
            ld16(tbase + static_cast<uint32_t>(sub * p.m_pad + c), v);
            finish(v);
            if (writer) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const uint32_t dst = ring_base + static_cast<uint32_t>((sub * p.m_pad + c + j)) * out_pitch +
                                     static_cast<uint32_t>(out_row * 2);
                asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst), "h"(to_bf16(v[j])) : "memory");
              }
            }
          }
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");
        if (first_thread) {
          for (int sub = 0; sub < 2; ++sub) {
            const int tile = 2 * q + sub;
            if (tile >= tiles) break;
            for (int c0 = 0; c0 < p.m_pad; c0 += chunk_rows) {
              tma_store_2d(&tmap_d, ring_base + static_cast<uint32_t>(sub * p.m_pad + c0) * out_pitch,
                           tile * out_tile_cols, c0);
            }
          }
          bulk_commit_group();
          store_pending = true;
        }
      } else {
        for (int sub = 0; sub < 2; ++sub) {
          const int tile = 2 * q + sub;
          if (tile >= tiles) break;
          const int n = tile * 128 + row;
          const uint32_t taddr = tbase + static_cast<uint32_t>(sub * p.m_pad);
          if (p.d_tma) {
            for (int c0 = 0; c0 < p.m_pad; c0 += chunk_rows) {
              if (first_thread && store_pending) bulk_wait_group_read<0>();
              asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");
              const int lo = c0 > col_begin ? c0 : col_begin;
              const int hi = c0 + chunk_rows < col_end ? c0 + chunk_rows : col_end;
              for (int c = lo; c < hi; c += 16) {
                float v[16];
                ld16(taddr + c, v);
                finish(v);
                if (writer) {
#pragma unroll
                  for (int j = 0; j < 16; ++j) {
                    const uint32_t dst = stage_base + static_cast<uint32_t>(c - c0 + j) * out_pitch +
                                         static_cast<uint32_t>(out_row * 2);
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(dst), "h"(to_bf16(v[j])) : "memory");
                  }
                }
              }
              fence_proxy_async_smem();
              asm volatile("bar.sync 1, %0;" ::"r"(epi_threads) : "memory");
              if (first_thread) {
                tma_store_2d(&tmap_d, stage_base, tile * out_tile_cols, c0);
                bulk_commit_group();
                store_pending = true;
              }
            }
          } else {
            for (int c = col_begin; c < col_end; c += 16) {
              float v[16];
              ld16(taddr + c, v);
              finish(v);
              const int n_store = gated ? tile * 64 + out_row : n;
              if (writer && n_store < n_out) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  if (c + j < p.M) p.d[static_cast<size_t>(c + j) * p.ldd + n_store] = to_bf16(v[j]);
                }
              }
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty_bar(bank));
    }
    if (first_thread && store_pending) bulk_wait_group_read<0>();
  } else if (kFused && warp >= 12) {
    // ------------------------------------------------------------- activation quantiser (kQuantWarps warps)
    // Warp w takes the stages w, w + kQuantWarps, ...: a stage visit costs an L2 round trip, and
    // that many visits in flight keep up with the weight stream.  Lane l of a pass holds blocks l, l + 32, l + 64,
    // l + 96 of the stage (block = row * 8 + k-block: eight lanes read 512 contiguous bytes of a row).
    // No more warps than ring slots take part: a warp whose consecutive visits lay more than one
    // ring cycle apart could be two barrier phases ahead of a slot, and a parity wait cannot tell
    // "two phases ago" from "now" (it would pass early and arrive on a barrier that is still in
    // use).
    const int qw = warp - 12;
    const int q_active = stages < kQuantWarps ? stages : kQuantWarps;
    const int total = qw < q_active ? (q_end - q_begin) * num_kb : 0;
    const int kblocks = p.K / 32;
    const int stage_blocks = p.m_pad * 8;
    griddep_wait();   // the activations are the previous kernel's output
    for (int g = qw; g < total; g += q_active) {
      const int s = g % stages;
      const uint32_t ph = static_cast<uint32_t>(g / stages) & 1u;
      const int kb = g % num_kb;
      if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
        if (lane == 0) report_status(p.status, kDevTimeoutProducer);
        break;
      }
      const uint32_t dst = ring_base + static_cast<uint32_t>(s * p.stage_bytes);
      for (int b0 = 0; b0 < stage_blocks; b0 += 128) {
        uint4 raw[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int b = b0 + i * 32 + lane;
          const int r = b >> 3, gk = kb * 8 + (b & 7);
          if (b < stage_blocks && r < p.M && gk < kblocks) {
            const uint4* src = reinterpret_cast<const uint4*>(p.x_src + static_cast<long long>(r) * p.ldx + gk * 32);
#pragma unroll
            for (int j = 0; j < 4; ++j) raw[i][j] = __ldg(src + j);
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) raw[i][j] = make_uint4(0u, 0u, 0u, 0u);
          }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int b = b0 + i * 32 + lane;
          if (b >= stage_blocks) continue;
          const int r = b >> 3, j8 = b & 7;
          uint4 packed;
          uint32_t sb;
          quantize_mx_block_bf16(raw[i], &packed, &sb);   // an all-zero block (padding): codes 0, scale 127
          // Codes: row r, 16-byte chunk j8 of its 128 bytes, at chunk j8 ^ (r % 8) (128-byte swizzle).
          st_shared_v4(dst + x_off + static_cast<uint32_t>(r * 128 + ((j8 ^ (r & 7)) << 4)), packed.x, packed.y,
                       packed.z, packed.w);
          // Scale: cell j8 / 4, line r % 32, 4-byte group r / 32, byte j8 % 4.
          const uint32_t sf_dst = dst + sfx_off +
                                  static_cast<uint32_t>((j8 >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (j8 & 3));
          asm volatile("st.shared.u8 [%0], %1;" ::"r"(sf_dst), "r"(sb) : "memory");
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(sf_full_bar(s));
        mbar_arrive(full_bar(s));
      }
    }
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, 512);
  }
}

template <bool V4, bool kWide, bool kFused>
__global__ void __launch_bounds__(kFused ? kFusedThreads : kDualThreads, 1)
gemm_nvfp4_decode_dual_kernel(const __grid_constant__ CUtensorMap tmap_w,
                              const __grid_constant__ CUtensorMap tmap_x,
                              const __grid_constant__ CUtensorMap tmap_sfw,
                              const __grid_constant__ CUtensorMap tmap_sfx,
                              const __grid_constant__ CUtensorMap tmap_d,
                              const __grid_constant__ DualParams p) {
  static_assert(!kFused || (!V4 && !kWide), "the fused quantiser exists for the swapped UE8M0 form");
  decode_dual_body<V4, kWide, kFused>(tmap_w, tmap_x, tmap_sfw, tmap_sfx, tmap_d, p);
}

}  // namespace fp4d

int fp4_decode_stage_bytes(int m_pad) { return fp4d::kWBytes + m_pad * fp4d::kBlockKBytes + 2 * fp4d::kSfBytes; }

size_t fp4_decode_slot_bytes(int M) { return static_cast<size_t>((M + 15) / 16 * 16) * 128 * sizeof(float); }

size_t fp4_decode_scratch_bytes(int M, int N, int ctas) {
  return 2 * static_cast<size_t>(ctas) * fp4_decode_slot_bytes(M) + (static_cast<size_t>(N) + 127) / 128 * sizeof(int);
}

int fp4_decode_box_rows(int M) {
  const int m_pad = (M + 15) / 16 * 16;
  return m_pad < fp4d::kStageRows ? m_pad : fp4d::kStageRows;
}

namespace {

template <bool V4, bool kWide, bool kFused = false>
int fp4_decode_dual_launch(const Fp4DecodeLaunch& L, cudaStream_t stream) {
  constexpr int kBandBytes = V4 ? 2048 : 1024;
  constexpr int kSlotCols = V4 ? 48 : 24;
  auto kernel = fp4d::gemm_nvfp4_decode_dual_kernel<V4, kWide, kFused>;
  static thread_local int configured_device = -1;
  static thread_local int sm_count = 0;
  constexpr int kSmemBudget = 227 * 1024;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_error(SMB_ERR_CUDA, "cudaGetDevice failed");
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return set_cuda_error(e, "decode (dual) kernel setup");
    configured_device = dev;
  }
  fp4d::DualParams p;
  p.M = L.M;
  p.N = L.N;
  p.K = L.K;
  p.m_pad = (L.M + 15) / 16 * 16;
  // The wide form keeps room for all 128 rows of the instruction's first operand in every stage.
  p.stage_bytes = 2 * fp4d::kWBytes + (kWide ? fp4d::kMaxPad : p.m_pad) * fp4d::kBlockKBytes + 3 * kBandBytes;
  const int staging = fp4_decode_box_rows(L.M) * 256;
  int stages = (kSmemBudget - 1024 - fp4d::kBarrierBytes - staging) / p.stage_bytes;
  if (stages > fp4d::kMaxStages) stages = fp4d::kMaxStages;
  // Two accumulator banks (a tile pair is drained while the next one is multiplied) when they fit
  // beside at least three scale slots, else one.  The wide form has 256 accumulator columns.
  p.banks = (!kWide && 4 * p.m_pad + 3 * kSlotCols <= 512) ? 2 : 1;
  const int max_slots = (512 - (kWide ? 256 : p.banks * 2 * p.m_pad)) / kSlotCols;
  if (stages > max_slots) stages = max_slots;
  if (L.max_stages > 0 && stages > L.max_stages) stages = L.max_stages;
  if (stages < 2) return set_error(SMB_ERR_UNSUPPORTED, "decode (dual): activation tile too large");
  p.stages = stages;
  p.ldd = L.ldd;
  p.d = static_cast<uint16_t*>(L.d);
  p.status = L.status;
  p.d_tma = L.d_tma ? 1 : 0;
  p.activations_dynamic = L.activations_dynamic ? 1 : 0;
  p.alpha = L.alpha;
  p.x_src = static_cast<const uint16_t*>(L.act_src);
  p.ldx = L.act_ld;
  p.swiglu = L.swiglu ? 1 : 0;
  p.act_spread = (!kFused && fp4_decode_spreads_activations(L)) ? 1 : 0;
  p.act_codes = static_cast<uint8_t*>(L.act_codes);
  p.act_sf = static_cast<uint8_t*>(L.act_sf);
  p.act_counter = L.act_counter;
  const int pairs = ((L.N + 127) / 128 + 1) / 2;
  p.pairs_per_cta = (pairs + sm_count - 1) / sm_count;
  const int grid = (pairs + p.pairs_per_cta - 1) / p.pairs_per_cta;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(kFused ? fp4d::kFusedThreads : fp4d::kDualThreads, 1, 1);
  cfg.dynamicSmemBytes = 1024 + stages * p.stage_bytes + staging + fp4d::kBarrierBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = L.no_overlap ? 0 : 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (kWide && p.pairs_per_cta != 1)
    return set_error(SMB_ERR_INVALID, "decode (wide): one tile pair per CTA only");
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L.tmap_w, L.tmap_x, L.tmap_sfw, L.tmap_sfx,
                                     kWide ? L.tmap_d_rows : L.tmap_d, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "nvfp4 decode (dual) launch");
  return SMB_OK;
}

}  // namespace

bool fp4_decode_prefers_dual(int M) { return (M + 15) / 16 * 16 >= fp4d::kDualFromPad; }

// BF16 activations are quantised inside the GEMM kernel by the swapped dual form with UE8M0 scales
// and whole tile pairs, for at most 16 rows: every CTA quantises all activations again, one
// stage visit of a warp takes about 1.3 us per 16 rows, and with more rows the visits no longer
// keep up with the weight stream (N = 28672, K = 8192, us per step, fused / quantiser kernel
// chained in front: M = 1 20.6 / 22.8, 16 21.9 / 23.2, 32 30.2 / 23.8, 64 49.1 / 26.4).  Elsewhere
// the caller quantises first.
bool fp4_decode_fuses_activations(const Fp4DecodeLaunch& L) {
  return L.act_src != nullptr && L.act_mode == 1 && !L.block16 && L.dual && !L.narrow && L.max_ctas == 0 &&
         L.M <= 16;
}

// BF16 activations quantised once per launch by the grid as a whole (act_spread in
// decode_dual_body): any number of rows, the dual forms with UE8M0 scales and whole tile pairs,
// plans that own a code buffer and a counter.
bool fp4_decode_spreads_activations(const Fp4DecodeLaunch& L) {
  return L.act_src != nullptr && L.act_mode == 0 && L.act_counter != nullptr && L.act_codes != nullptr &&
         !L.block16 && L.dual && L.max_ctas == 0;
}

namespace {
// More than 64 activation rows and at most one tile pair per SM: the form with the activations as
// the instruction's rows (see decode_dual_body).
bool fp4_decode_wide_applies(const Fp4DecodeLaunch& L) {
  if (L.narrow || (L.M + 15) / 16 * 16 <= 64) return false;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return false;
  const int pairs = ((L.N + 127) / 128 + 1) / 2;
  return pairs <= sms;
}
}  // namespace

int fp4_decode_launch(const Fp4DecodeLaunch& L, cudaStream_t stream) {
  // The dual-tile form has whole tile pairs only: a caller that asks for a CTA count gets the
  // stream-K ranges of the single form.
  const bool wide = (L.block16 || (L.dual && L.max_ctas == 0)) && fp4_decode_wide_applies(L);
  if (fp4_decode_fuses_activations(L)) return fp4_decode_dual_launch<false, false, true>(L, stream);
  if (L.block16)   // this format has the dual forms only
    return wide ? fp4_decode_dual_launch<true, true>(L, stream) : fp4_decode_dual_launch<true, false>(L, stream);
  if (L.dual && L.max_ctas == 0)
    return wide ? fp4_decode_dual_launch<false, true>(L, stream) : fp4_decode_dual_launch<false, false>(L, stream);
  if (L.swiglu)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "decode: the gated epilogue exists for the tile-pair forms (no forced CTA count, not the "
                     "single-tile form)");
  static thread_local int configured_device = -1;
  static thread_local int sm_count = 0;
  constexpr int kSmemBudget = 227 * 1024;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_error(SMB_ERR_CUDA, "cudaGetDevice failed");
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(fp4d::gemm_nvfp4_decode_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaFuncSetAttribute(decode smem)");
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaDeviceGetAttribute(SM count)");
    configured_device = dev;
  }
  fp4d::Params p;
  p.M = L.M;
  p.N = L.N;
  p.K = L.K;
  p.m_pad = (L.M + 15) / 16 * 16;
  p.stage_bytes = fp4_decode_stage_bytes(p.m_pad);
  // One CTA per SM.  (Two co-resident CTAs with half the ring each were measured slower, 22.8
  // against 21.0-21.7 us at M = 16, and would let three CTAs share a tile.)
  const int staging = fp4_decode_box_rows(L.M) * 256;   // transposed [rows x 128] bf16 block of D
  const int budget = kSmemBudget - 1024 - fp4d::kBarrierBytes - staging;
  int stages = budget / p.stage_bytes;
  p.tmem_cols = 512;
  p.bank_stride = 128;
  const int max_slots = (p.tmem_cols - 2 * p.bank_stride) / fp4d::kSlotCols;
  if (stages > max_slots) stages = max_slots;
  if (stages > fp4d::kMaxStages) stages = fp4d::kMaxStages;
  // With stream-K ranges over all SMs, six stages (96 KiB of weights in flight per SM) cover the
  // HBM latency and deeper rings measured slower (M = 16: 19.4 us with 6 stages, 19.8 with 8,
  // 20.4 with 11).  With whole tiles on fewer CTAs each SM carries more of the stream: 8 stages
  // (M = 16, 112 CTAs: 17.8 us against 18.05 with 6 and 19.3 with 4).
  const bool whole_tiles = (L.max_ctas == 0);
  if (L.max_stages == 0 && stages > (whole_tiles ? fp4d::kWholeTileStages : fp4d::kDefaultStages))
    stages = whole_tiles ? fp4d::kWholeTileStages : fp4d::kDefaultStages;
  if (L.max_stages > 0 && stages > L.max_stages) stages = L.max_stages;
  if (stages < 2) return set_error(SMB_ERR_UNSUPPORTED, "decode: activation tile too large");
  p.stages = stages;
  p.ldd = L.ldd;
  p.d = static_cast<uint16_t*>(L.d);
  p.scratch = L.scratch;
  p.counters = L.counters;
  p.status = L.status;
  p.d_tma = L.d_tma ? 1 : 0;
  p.activations_dynamic = L.activations_dynamic ? 1 : 0;
  const int num_kb = (L.K + fp4d::kBlockK - 1) / fp4d::kBlockK;
  const long long units = static_cast<long long>((L.N + 127) / 128) * num_kb;
  int grid;
  if (whole_tiles) {
    const int tiles = (L.N + 127) / 128;
    p.tiles_per_cta = (tiles + sm_count - 1) / sm_count;
    grid = (tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;
  } else {
    p.tiles_per_cta = 0;
    grid = L.max_ctas;
    if (grid > sm_count) grid = sm_count;
    if (grid > L.scratch_ctas) grid = L.scratch_ctas;   // two scratch slots per CTA exist for so many
    if (units < grid) grid = static_cast<int>(units);
    if (grid < 1) return set_error(SMB_ERR_INVALID, "decode: no scratch slots");
  }
  const int smem = 1024 + stages * p.stage_bytes + staging + fp4d::kBarrierBytes;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(fp4d::kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = L.no_overlap ? 0 : 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, fp4d::gemm_nvfp4_decode_kernel, L.tmap_w, L.tmap_x, L.tmap_sfw,
                                     L.tmap_sfx, L.tmap_d, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "nvfp4 decode launch");
  return SMB_OK;
}

// Fills the output side of a decode launch: the TMA view of D when D allows one.
int fp4_decode_bind_output(Fp4DecodeLaunch* L, void* d, int M, int N, long long ldd, bool allow_tma) {
  L->d = d;
  L->ldd = static_cast<int>(ldd);
  L->d_tma = allow_tma && (ldd % 8 == 0) && (reinterpret_cast<uintptr_t>(d) % 16 == 0);
  if (L->d_tma) {
    // Gated epilogue: D is [M, N / 2] and a weight tile of 128 rows yields 64 output columns.
    const int n_out = L->swiglu ? N / 2 : N;
    int rc = encode_tmap_2d(&L->tmap_d, d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, n_out, ldd * 2,
                            fp4_decode_box_rows(M), L->swiglu ? 64 : 128, false);
    if (rc == SMB_OK)
      rc = encode_tmap_2d(&L->tmap_d_rows, d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, n_out, ldd * 2, 32, 64, true);
    return rc;
  }
  L->tmap_d = L->tmap_w;   // never dereferenced
  L->tmap_d_rows = L->tmap_w;
  return SMB_OK;
}

}  // namespace smb

// -----------------------------------------------------------------------------------
// Decode GEMM for callers that must not allocate
// -----------------------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc on the path that runs the GEMM: an
// inference server that has handed all device memory to its own pool at start-up, or a
// plugin running inside another framework's allocator: there a cudaMalloc on the request path
// fails, or succeeds and stalls every stream of the device while it runs.  For them the status word, the tile counters and the fp32 partial-sum slots
// of the decode kernel live in the fixed array below instead of in a plan-owned allocation.
// Which of them a call uses depends on the work split (smb_decode_noalloc_set_split): whole
// tile pairs per CTA share no tile between CTAs and use the status word only; the stream-K
// split over a fixed number of CTAs uses the counters of all tiles and two slots per CTA.  The
// array is part of the library image: every GPU that loads the library carries these 2 MiB until
// the process exits.
#include <atomic>

namespace {

constexpr size_t kStaticScratchBytes = size_t(2) << 20;
constexpr size_t kStaticStatusOffset = kStaticScratchBytes - 256;   // last 256 bytes: status word
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
// Device address of the array per device ordinal, published once it is known.  Two host threads
// that race here both look the same address up and store the same value.
std::atomic<void*> g_static_scratch_addr[kMaxDevices];
// CTAs of the stream-K split; 0 = whole tile pairs per CTA.  Process-wide, like the array.
std::atomic<int> g_noalloc_split_ctas{0};

// The array's name is only a host-side handle here; the kernel needs its device address,
// which differs per device.  Looked up once per device, with that device current.
int static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return smb::set_cuda_error(e, "no-alloc decode: cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices)
    return smb::set_error(SMB_ERR_UNSUPPORTED, "no-alloc decode: device ordinal %d out of range", dev);
  void* ptr = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (e != cudaSuccess) return smb::set_cuda_error(e, "no-alloc decode: cudaGetSymbolAddress");
    if (ptr == nullptr)
      return smb::set_error(SMB_ERR_CUDA, "no-alloc decode: cudaGetSymbolAddress returned null");
    g_static_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *out = ptr;
  return SMB_OK;
}

}  // namespace

extern "C" size_t smb_decode_noalloc_scratch_limit(void) { return kStaticStatusOffset; }

extern "C" int smb_decode_noalloc_set_split(int ctas) {
  if (ctas < 0 || ctas > 4096)
    return smb::set_error(SMB_ERR_INVALID, "no-alloc decode: split of %d CTAs outside 0..4096", ctas);
  g_noalloc_split_ctas.store(ctas, std::memory_order_relaxed);
  return SMB_OK;
}

extern "C" int smb_decode_noalloc_check(void* stream) {
  using namespace smb;
  void* base = nullptr;
  if (int rc = static_scratch_address(&base)) return rc;
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return set_cuda_error(e, "no-alloc decode check: stream synchronize");
  int status = 0;   // host stack: the copy below allocates nothing
  e = cudaMemcpy(&status, static_cast<char*>(base) + kStaticStatusOffset, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return set_cuda_error(e, "no-alloc decode check: status read");
  if (status != 0) {
    // The next call clears the word (and, for the stream-K split, the counters) before it launches.
    return set_error(SMB_ERR_DEVICE, "nvfp4 decode kernel reported status %d: %s", status,
                     device_status_name(status));
  }
  return SMB_OK;
}

extern "C" int smb_dense_gemm_nvfp4_decode_noalloc(const void* a, const void* sfa, const void* b,
                                                   const void* sfb, void* d, int M, int N, int K,
                                                   void* stream) {
  using namespace smb;
  if (a == nullptr || sfa == nullptr || b == nullptr || sfb == nullptr || d == nullptr)
    return set_error(SMB_ERR_INVALID, "no-alloc decode: null operand pointer");
  if (M <= 0 || N <= 0 || K <= 0)
    return set_error(SMB_ERR_INVALID, "no-alloc decode: dimensions must be positive");
  if (M > 128)
    return set_error(SMB_ERR_UNSUPPORTED, "no-alloc decode: M=%d exceeds 128 activation rows", M);
  if (K % 32 != 0)
    return set_error(SMB_ERR_UNSUPPORTED, "no-alloc decode: K=%d must be a multiple of 32", K);
  const int m_pad = (M + 15) / 16 * 16;
  // Stream-K split: one counter per tile and two slots per CTA must fit below the status word.
  // Whole tile pairs need neither, so any N is served.
  const int split = g_noalloc_split_ctas.load(std::memory_order_relaxed);
  const size_t counter_bytes = (static_cast<size_t>(N) + 127) / 128 * sizeof(int);
  const size_t per_cta = 2 * fp4_decode_slot_bytes(M);
  int ctas = 0;
  if (split > 0) {
    if (counter_bytes + per_cta > kStaticStatusOffset)
      return set_error(SMB_ERR_UNSUPPORTED,
                       "no-alloc decode: M=%d N=%d needs %zu bytes of scratch for its tile counters and "
                       "one CTA, the built-in array holds %zu",
                       M, N, counter_bytes + per_cta, kStaticStatusOffset);
    const size_t fit = (kStaticStatusOffset - counter_bytes) / per_cta;
    ctas = fit < static_cast<size_t>(split) ? static_cast<int>(fit) : split;
  }
  const size_t slot_bytes = static_cast<size_t>(ctas) * per_cta;
  void* base = nullptr;
  if (int rc = static_scratch_address(&base)) return rc;

  Fp4DecodeLaunch L;
  L.M = M;
  L.N = N;
  L.K = K;
  L.max_ctas = ctas;     // 0: whole tile pairs; else stream-K ranges over this many CTAs
  L.max_stages = 0;
  L.activations_dynamic = false;
  L.dual = fp4_decode_prefers_dual(M);
  L.narrow = false;
  L.act_src = nullptr;
  L.act_ld = 0;
  L.block16 = false;
  L.alpha = 1.0f;
  L.swiglu = false;
  L.act_mode = 0;
  L.act_codes = L.act_sf = nullptr;
  L.act_counter = nullptr;
  L.no_overlap = true;   // the clears below must be ordered before every access of this launch
  L.scratch = static_cast<float*>(base);
  L.scratch_ctas = ctas;
  L.counters = reinterpret_cast<int*>(static_cast<char*>(base) + slot_bytes);
  L.status = reinterpret_cast<int*>(static_cast<char*>(base) + kStaticStatusOffset);
  const uint64_t kchunks = (static_cast<uint64_t>(K) / 32 + 3) / 4;
  const uint64_t bands_a = (static_cast<uint64_t>(M) + 127) / 128;
  const uint64_t bands_b = (static_cast<uint64_t>(N) + 127) / 128;
  int rc = encode_tmap_2d(&L.tmap_w, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, K / 2, 128, 128, true);
  if (rc == SMB_OK)
    rc = encode_tmap_2d(&L.tmap_x, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K / 2, K / 2, m_pad, 128, true);
  if (rc == SMB_OK)
    rc = encode_tmap_2d(&L.tmap_sfw, sfb, CU_TENSOR_MAP_DATA_TYPE_UINT64, 8, bands_b, kchunks * 64,
                        kchunks * 512, 1, 128, false);
  if (rc == SMB_OK)
    rc = encode_tmap_2d(&L.tmap_sfx, sfa, CU_TENSOR_MAP_DATA_TYPE_UINT64, 8, bands_a, kchunks * 64,
                        kchunks * 512, 1, 128, false);
  if (rc == SMB_OK) rc = fp4_decode_bind_output(&L, d, M, N, N, true);
  if (rc != SMB_OK) return rc;
  // The array keeps whatever the last call left in it.  The status word always starts at zero.
  // The counters (used by the stream-K split only) are all zero after a call that ran to the
  // end and anything after one that was cut short, so that split clears them too.  The slots
  // need no clearing: a slot is read only after its writer has counted itself in.
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(L.status, 0, sizeof(int), st);
  if (e == cudaSuccess && ctas > 0) e = cudaMemsetAsync(L.counters, 0, counter_bytes, st);
  if (e != cudaSuccess) return set_cuda_error(e, "no-alloc decode: scratch clear");
  return fp4_decode_launch(L, st);
}
