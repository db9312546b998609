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
//   * a partly covered tile is added (red.global.add.f32) into a per-tile fp32 scratch slab, a
//     per-tile counter is raised by the K blocks contributed, and the CTA that completes the
//     count converts the slab to bf16, stores it, and zeroes slab and counter for the next call.
// Warp roles (256 threads): warp 0 TMA producer, warp 1 MMA issue + TMEM owner, warp 2 scale
// copies (tcgen05.cp, issued apart from the MMAs so that they overlap them), warp 3 idle,
// warps 4-7 epilogue (warp w reads TMEM lanes 32 (w % 4) .. +31).
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace smb {

namespace fp4d {

constexpr int kThreads = 256;
constexpr int kBlockKBytes = 128;     // 256 E2M1 values
constexpr int kBlockK = 256;
constexpr int kWBytes = 128 * kBlockKBytes;   // 16 KiB weight box
constexpr int kSfBytes = 1024;        // one 128-row band x 8 scales (two 512-byte cells)
constexpr int kSlotCols = 16;         // SFW cells (8 columns) + SFX cells (8 columns) per stage
constexpr int kMaxStages = 16;
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
  float* scratch;     // [tiles][m_pad][128] fp32 partial sums (zero between calls)
  int* counters;      // [tiles] K blocks accumulated so far (zero between calls)
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

__global__ void __launch_bounds__(kThreads, 1)
gemm_nvfp4_decode_kernel(const __grid_constant__ CUtensorMap tmap_w,
                         const __grid_constant__ CUtensorMap tmap_x,
                         const __grid_constant__ CUtensorMap tmap_sfw,
                         const __grid_constant__ CUtensorMap tmap_sfx, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int stages = p.stages;
  const uint32_t ring_base = smem_base;
  const uint32_t bar_base = ring_base + static_cast<uint32_t>(stages * p.stage_bytes);
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
  const long long u_begin = units * blockIdx.x / gridDim.x;
  const long long u_end = units * (blockIdx.x + 1) / gridDim.x;
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
    const int quarter = warp & 3;
    int seg = 0;
    bool waited_for_previous_grid = false;
    long long u = u_begin;
    while (u < u_end) {
      const int tile = static_cast<int>(u / num_kb);
      const long long seg_end = (static_cast<long long>(tile) + 1) * num_kb < u_end
                                    ? (static_cast<long long>(tile) + 1) * num_kb : u_end;
      const int count = static_cast<int>(seg_end - u);
      const int bank = seg & 1;
      if (!mbar_wait(acc_full_bar(bank), static_cast<uint32_t>(seg >> 1) & 1u)) {
        if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
        break;
      }
      tc_fence_after_sync();
      const int row = quarter * 32 + lane;            // weight row inside the tile
      const int n = tile * 128 + row;                 // output column
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                             static_cast<uint32_t>(bank * p.bank_stride);
      const bool whole = (count == num_kb);
      float* slab = p.scratch + static_cast<size_t>(tile) * p.m_pad * 128;
      if (!waited_for_previous_grid) {
        // First touch of D / scratch / counters: the previous launch on the stream (which may
        // be this same kernel, started early under programmatic dependent launch) must be done.
        griddep_wait();
        waited_for_previous_grid = true;
      }
      if (whole) {
        for (int c = 0; c < p.m_pad; c += 16) {
          float v[16];
          ld16(taddr + c, v);
          if (n < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c + j < p.M) p.d[static_cast<size_t>(c + j) * p.ldd + n] = to_bf16(v[j]);
            }
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty_bar(bank));
      } else {
        // Partly covered tile.  If every other contribution is already in the slab (the usual
        // case for the segment at the end of a CTA's range: its partner handled the other
        // part of the tile at the start of its own range), merge straight from registers.
        if (warp == 4 && lane == 0) {
          const int seen = atomicAdd(p.counters + tile, 0);
          const uint32_t f = (seen + count == num_kb) ? 2u : 0u;
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(last_flag), "r"(f) : "memory");
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        uint32_t flag;
        asm volatile("ld.shared.b32 %0, [%1];" : "=r"(flag) : "r"(last_flag) : "memory");
        if (flag == 2u) {
          __threadfence();
          for (int c = 0; c < p.m_pad; c += 16) {
            float v[16], o[16];
            ld16(taddr + c, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) o[j] = __ldcg(slab + (c + j) * 128 + row);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              if (c + j < p.M && n < p.N)
                p.d[static_cast<size_t>(c + j) * p.ldd + n] = to_bf16(v[j] + o[j]);
              __stcg(slab + (c + j) * 128 + row, 0.0f);
            }
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(bank));
          if (warp == 4 && lane == 0) p.counters[tile] = 0;
        } else {
          for (int c = 0; c < p.m_pad; c += 16) {
            float v[16];
            ld16(taddr + c, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) atomicAdd(slab + (c + j) * 128 + row, v[j]);
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(acc_empty_bar(bank));
          // Publish the partial sums, then find out whether this CTA completed the tile after all.
          __threadfence();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (warp == 4 && lane == 0) {
            const int before = atomicAdd(p.counters + tile, count);
            const uint32_t last = (before + count == num_kb) ? 1u : 0u;
            asm volatile("st.shared.b32 [%0], %1;" ::"r"(last_flag), "r"(last) : "memory");
          }
          asm volatile("bar.sync 1, 128;" ::: "memory");
          uint32_t last;
          asm volatile("ld.shared.b32 %0, [%1];" : "=r"(last) : "r"(last_flag) : "memory");
          if (last) {
            __threadfence();
            for (int c = 0; c < p.m_pad; c += 16) {
              float o[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) o[j] = __ldcg(slab + (c + j) * 128 + row);
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c + j < p.M && n < p.N)
                  p.d[static_cast<size_t>(c + j) * p.ldd + n] = to_bf16(o[j]);
                __stcg(slab + (c + j) * 128 + row, 0.0f);
              }
            }
            if (warp == 4 && lane == 0) p.counters[tile] = 0;
          }
        }
        // The flag word is reused by the next partial segment.
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      u = seg_end;
      ++seg;
    }
  }
  __syncwarp();
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<1>(tmem_base, static_cast<uint32_t>(p.tmem_cols));
  }
}

}  // namespace fp4d

int fp4_decode_stage_bytes(int m_pad) { return fp4d::kWBytes + m_pad * fp4d::kBlockKBytes + 2 * fp4d::kSfBytes; }

int fp4_decode_launch(const Fp4DecodeLaunch& L, cudaStream_t stream) {
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
  const int per_sm = 1;
  const int budget = (per_sm == 2 ? 113 * 1024 : kSmemBudget) - 1024 - fp4d::kBarrierBytes;
  int stages = budget / p.stage_bytes;
  p.tmem_cols = per_sm == 2 ? 256 : 512;
  p.bank_stride = per_sm == 2 ? 64 : 128;
  const int max_slots = (p.tmem_cols - 2 * p.bank_stride) / fp4d::kSlotCols;
  if (stages > max_slots) stages = max_slots;
  if (stages > fp4d::kMaxStages) stages = fp4d::kMaxStages;
  if (L.max_stages > 0 && stages > L.max_stages) stages = L.max_stages;
  if (stages < 2) return set_error(SMB_ERR_UNSUPPORTED, "decode: activation tile too large");
  p.stages = stages;
  p.ldd = L.ldd;
  p.d = static_cast<uint16_t*>(L.d);
  p.scratch = L.scratch;
  p.counters = L.counters;
  p.status = L.status;
  p.activations_dynamic = L.activations_dynamic ? 1 : 0;
  const int num_kb = (L.K + fp4d::kBlockK - 1) / fp4d::kBlockK;
  const long long units = static_cast<long long>((L.N + 127) / 128) * num_kb;
  int grid = L.max_ctas > 0 ? L.max_ctas : per_sm * sm_count;
  if (grid > per_sm * sm_count) grid = per_sm * sm_count;
  if (units < grid) grid = static_cast<int>(units);
  const int smem = 1024 + stages * p.stage_bytes + fp4d::kBarrierBytes;
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
  cudaError_t e = cudaLaunchKernelEx(&cfg, fp4d::gemm_nvfp4_decode_kernel, L.tmap_w, L.tmap_x,
                                     L.tmap_sfw, L.tmap_sfx, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "nvfp4 decode launch");
  return SMB_OK;
}

}  // namespace smb

// -----------------------------------------------------------------------------------
// Decode GEMM for callers that must not allocate
// -----------------------------------------------------------------------------------
// Some hosts of this library cannot call cudaMalloc on the path that runs the GEMM: an
// inference server that has handed all device memory to its own pool at start-up, a
// plugin running inside another framework's allocator, code between a stream capture's
// begin and end.  For them the fp32 partial-sum slabs and tile counters of the decode
// kernel live in the fixed array below instead of in a plan-owned allocation.  The array
// is part of the library image: every GPU that loads the library carries these 16 MiB
// until the process exits.
namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;
constexpr size_t kStaticStatusOffset = kStaticScratchBytes - 256;   // last 256 bytes: status word
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {nullptr};

// The array's name is only a host-side handle here; the kernel needs its device address,
// which differs per device.  Looked up once per device, with that device current.
int static_scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return smb::set_cuda_error(e, "no-alloc decode: cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices)
    return smb::set_error(SMB_ERR_UNSUPPORTED, "no-alloc decode: device ordinal %d out of range", dev);
  if (g_static_scratch_addr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (e != cudaSuccess) return smb::set_cuda_error(e, "no-alloc decode: cudaGetSymbolAddress");
    if (ptr == nullptr)
      return smb::set_error(SMB_ERR_CUDA, "no-alloc decode: cudaGetSymbolAddress returned null");
    g_static_scratch_addr[dev] = ptr;
  }
  *out = g_static_scratch_addr[dev];
  return SMB_OK;
}

}  // namespace

extern "C" size_t smb_decode_noalloc_scratch_limit(void) { return kStaticStatusOffset; }

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
  const size_t tiles = (static_cast<size_t>(N) + 127) / 128;
  const size_t slab_bytes = tiles * m_pad * 128 * sizeof(float);
  const size_t need = slab_bytes + tiles * sizeof(int);
  if (need > kStaticStatusOffset)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "no-alloc decode: M=%d N=%d needs %zu bytes of scratch, the built-in array "
                     "holds %zu (ceil(N/128) * (round_up(M,16) * 512 + 4) must not exceed it)",
                     M, N, need, kStaticStatusOffset);
  void* base = nullptr;
  if (int rc = static_scratch_address(&base)) return rc;

  Fp4DecodeLaunch L;
  L.M = M;
  L.N = N;
  L.K = K;
  L.d = d;
  L.ldd = N;
  L.max_ctas = 0;
  L.max_stages = 0;
  L.activations_dynamic = false;
  L.no_overlap = true;   // the memset below must be ordered before every access of this launch
  L.scratch = static_cast<float*>(base);
  L.counters = reinterpret_cast<int*>(static_cast<char*>(base) + slab_bytes);
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
  if (rc != SMB_OK) return rc;
  // The array keeps whatever the last call left in it (all zero after a call that ran to the
  // end, anything after one that was cut short): clear the part this call uses, and the status.
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(base, 0, need, st);
  if (e == cudaSuccess) e = cudaMemsetAsync(L.status, 0, sizeof(int), st);
  if (e != cudaSuccess) return set_cuda_error(e, "no-alloc decode: scratch clear");
  return fp4_decode_launch(L, st);
}
