// Dense BF16 GEMM for sm_100a whose LAST wave of tiles is cut along K ("stream-K" for the tail
// only): for shapes whose 256 x 512 tiles do not fill a whole number of waves.
//
// Same tile, ring, instructions and epilogue as gemm_bf16_kernel<256, 2> (gemm_bf16.cu), and the
// same walk for the full waves: cluster c takes tiles c, c + C, ... in raster order, so the
// clusters of a wave run their K loops in step and share A and B panels through L2.  (Cutting
// EVERY tile where the clusters' equal shares end was tried first: the clusters then sit at
// different K positions of far-apart tiles, nothing is shared, and 8192^3 took 806 us instead of
// 646, 8192 x 1024 x 8192 128 us instead of 90.)  Only the last, partial wave of R < C tiles is
// split, in one of two ways, both keeping the clusters of a kind in step:
//   * fewer spare clusters than tiles (E = C - R < R): clusters 0 .. R-1 take the K blocks
//     [0, cut) of one tile each, every spare cluster the K blocks [cut, end) of up to T tiles one
//     after the other, cut chosen so that cut ~ T (end - cut);
//   * at least as many: every tile is cut into P + 1 equal K slices, P = E / R, one cluster each.
// A cluster that holds a later part of a tile writes its fp32 partial sums to that part's slot
// of a workspace and publishes one flag per epilogue warp; the cluster with the first K blocks
// owns the tile: its epilogue warps wait for their counterparts' flags, add the sums and store.
// All clusters of the grid are resident together (the grid is at most the number of cluster
// slots), an owner only waits for work that started no later than its own, and every wait is
// bounded.  8192 x 1024 x 8192 (one of eight column shards of 8192^3): 64 tiles on 74 clusters
// would take 112/128 of a tile's time if the hand-over of partial sums were free; it is not (see
// bf16_streamk_plan), so plans take this walk on request or where the estimate says it pays.
//
// The reference has no counterpart: its BF16 kernel hands out whole tiles
// (src/kernels/gemm/sm100a/dense_gemm_bf16.cu:86-234, blocks/97 scheduler).
#include "epilogue.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace smb {

namespace bf16s {

constexpr int kBlockM = 128;
constexpr int kBlockK = 64;
constexpr int kThreads = 352;
constexpr int kEpiWarps = 8;
constexpr int kTN = 256;                 // one N sub-block = one accumulator slot
constexpr int kTileN = 512;
constexpr int kABytes = kBlockM * kBlockK * 2;          // 16 KiB
constexpr int kBBytes = (kTN / 2) * kBlockK * 2;        // 16 KiB: one sub-block, one CTA
constexpr int kStageBytes = kABytes + 2 * kBBytes;
constexpr int kStages = (192 * 1024) / kStageBytes;     // 4
constexpr int kRingBytes = kStages * kStageBytes;
constexpr int kStoreBytes = kEpiWarps * kStoreBufBytes;
constexpr int kTotal = 1024 + kRingBytes + kStoreBytes + 1024;
static_assert(kTotal <= 232448, "shared memory budget");

struct Params {
  int M, N, K;
  int tiles_m, tiles_n;
  int group_m;
  int ldd;
  uint16_t* d_ptr;
  int* status;
  long long* prof;        // optional role timers, as in gemm_bf16.cu
  PeerCopies peers;       // always empty; the shared store code reads it
  float* partial;         // [slots][2 CTAs][8 warps][8 chunks][32 columns][32 lanes] fp32
  unsigned* flags;        // [slots][2 CTAs][8 warps]: launch number whose partial sums are complete
  StreamKWalk walk;       // how the last wave is cut (bf16_streamk_plan)
  unsigned epoch;         // this launch's number (never 0, never repeated while the flags live)
  int operands_static;    // 0: loads wait for the previous kernel on the stream, else they do not
  int l2_a, l2_b;
};

enum { kProfLoadWait = 0, kProfLoadTotal, kProfMmaWaitFull, kProfMmaWaitAcc, kProfMmaTotal,
       kProfEpiWait, kProfEpiTotal, kProfTiles, kProfCount };

constexpr size_t kPartialFloatsPerWarp = 8u * 32u * 32u;            // 8 chunks x 32 lanes x 32 columns
constexpr size_t kPartialFloatsPerCluster = 2u * 8u * kPartialFloatsPerWarp;

struct Segment {
  int tile, kb0, kb1;
  int slot;         // >= 0: a later part of a tile, partial sums go to this workspace slot
  int owned_parts;  // > 0: the first part of a tile whose other parts are in slots first_slot ...
  int first_slot;
};

// Item i of cluster `cluster`'s work list; false when the list is used up.
__device__ __forceinline__ bool segment_at(const StreamKWalk& w, int cluster, int n_clusters, int num_kb, int i,
                                           Segment& sg) {
  sg.slot = -1;
  sg.owned_parts = 0;
  sg.first_slot = 0;
  if (i < w.full_waves) {
    sg.tile = i * n_clusters + cluster;
    sg.kb0 = 0;
    sg.kb1 = num_kb;
    return true;
  }
  const int j = i - w.full_waves;
  const int first = w.full_waves * n_clusters;
  if (cluster < w.rem_tiles) {
    if (j > 0) return false;
    sg.tile = first + cluster;
    sg.kb0 = 0;
    if (w.parts > 0) {
      sg.kb1 = num_kb / (w.parts + 1);
      sg.owned_parts = w.parts;
      sg.first_slot = cluster * w.parts;
    } else {
      sg.kb1 = w.cut;
      sg.owned_parts = w.cut < num_kb ? 1 : 0;
      sg.first_slot = cluster;
    }
    return true;
  }
  const int e = cluster - w.rem_tiles;
  if (w.parts > 0) {
    if (j > 0 || e >= w.rem_tiles * w.parts) return false;
    const int r = e % w.rem_tiles, part = e / w.rem_tiles;
    sg.tile = first + r;
    sg.kb0 = static_cast<int>(static_cast<long long>(num_kb) * (part + 1) / (w.parts + 1));
    sg.kb1 = static_cast<int>(static_cast<long long>(num_kb) * (part + 2) / (w.parts + 1));
    sg.slot = r * w.parts + part;
    return true;
  }
  const int r = e * w.tails_per_cluster + j;
  if (j >= w.tails_per_cluster || r >= w.rem_tiles || w.cut >= num_kb) return false;
  sg.tile = first + r;
  sg.kb0 = w.cut;
  sg.kb1 = num_kb;
  sg.slot = r;
  return true;
}

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_bf16_streamk_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring_base = smem_base;
  const uint32_t store_base = ring_base + kRingBytes;
  const uint32_t bar_base = store_base + kStoreBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  const uint32_t acc_full_bar = bar_base + 8u * (2 * kStages);
  auto acc_empty_bar = [&](int h) { return bar_base + 8u * (2 * kStages + 1 + h); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 3);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = static_cast<int>(cluster_id_x());
  const int n_clusters = static_cast<int>(num_clusters_x());
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;

  griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(acc_full_bar, 1);
    for (int h = 0; h < 2; ++h) mbar_init(acc_empty_bar(h), 2 * 4);   // the four warps of a group, both CTAs
    fence_mbar_init_cluster();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_d);
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, 512);
    tmem_relinquish<2>();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer (both CTAs)
    const uint32_t leader_full0 = mapa_u32(full_bar(0), 0);
    int s = 0;
    uint32_t ph = 0;
    bool ok = true;
    const bool prof = p.prof != nullptr;
    long long waited = 0;
    const long long t_begin = prof ? clock64() : 0;
    const uint64_t pol_a = p.l2_a == 2 ? l2_policy_evict_first() : l2_policy_evict_last();
    const uint64_t pol_b = p.l2_b == 2 ? l2_policy_evict_first() : l2_policy_evict_last();
    if (!p.operands_static) griddep_wait();
    Segment sg;
    for (int item = 0; ok && segment_at(p.walk, cluster, n_clusters, num_kb, item, sg); ++item) {
      int tm, tn;
      tile_coords(sg.tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      const int row_a = tm * 256 + static_cast<int>(rank) * kBlockM;
      const int row_b = tn * kTileN + static_cast<int>(rank) * (kTN / 2);
      for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
        const long long w0 = prof ? clock64() : 0;
        if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
          report_status(p.status, kDevTimeoutProducer);
          ok = false;
          break;
        }
        if (prof) waited += clock64() - w0;
        const uint32_t bar = leader_full0 + 8u * s;
        const uint32_t dst_a = ring_base + s * kStageBytes;
        if (elect_one()) {
          if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * kStageBytes);
          if (p.l2_a != 0) tma_load_2d_pair_hint(dst_a, &tmap_a, bar, kb * kBlockK, row_a, pol_a);
          else tma_load_2d_pair(dst_a, &tmap_a, bar, kb * kBlockK, row_a);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (p.l2_b != 0)
              tma_load_2d_pair_hint(dst_a + kABytes + h * kBBytes, &tmap_b, bar, kb * kBlockK, row_b + h * kTN, pol_b);
            else
              tma_load_2d_pair(dst_a + kABytes + h * kBBytes, &tmap_b, bar, kb * kBlockK, row_b + h * kTN);
          }
        }
        __syncwarp();
        if (++s == kStages) { s = 0; ph ^= 1u; }
      }
    }
    if (!ok) {
      for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if (prof && lane == 0) {
      p.prof[blockIdx.x * kProfCount + kProfLoadWait] = waited;
      p.prof[blockIdx.x * kProfCount + kProfLoadTotal] = clock64() - t_begin;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issue (leader CTA only)
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, kTN);
      int s = 0;
      uint32_t ph = 0;
      int local = 0;
      bool ok = true;
      const bool prof = p.prof != nullptr;
      long long wait_full = 0, wait_acc = 0;
      const long long t_begin = prof ? clock64() : 0;
      Segment sg;
      for (; ok && segment_at(p.walk, cluster, n_clusters, num_kb, local, sg); ++local) {
        const uint32_t use_parity = static_cast<uint32_t>(local) & 1u;
        for (int kb = sg.kb0; kb < sg.kb1 && ok; ++kb) {
          const long long w0 = prof ? clock64() : 0;
          if (!mbar_wait(full_bar(s), ph)) {
            report_status(p.status, kDevTimeoutMmaFull);
            ok = false;
            break;
          }
          if (prof) wait_full += clock64() - w0;
          tc_fence_after_sync();
          const uint32_t a_addr = ring_base + s * kStageBytes;
          const uint64_t desc_a = make_smem_desc(a_addr, 1024, 16, kSwizzle128B);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (kb == sg.kb0) {
              // Half h of the accumulator must have been read out (previous segment).
              const long long a0 = prof ? clock64() : 0;
              if (!mbar_wait(acc_empty_bar(h), use_parity ^ 1u)) {
                report_status(p.status, kDevTimeoutMmaAcc);
                ok = false;
                break;
              }
              if (prof) wait_acc += clock64() - a0;
              tc_fence_after_sync();
            }
            const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(h * kTN);
            const uint64_t desc_b = make_smem_desc(a_addr + kABytes + h * kBBytes, 1024, 16, kSwizzle128B);
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < kBlockK / 16; ++k)
                mma_bf16_ss<2>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
            }
            __syncwarp();
          }
          if (!ok) break;
          if (elect_one()) mma_commit_pair(empty_bar(s), 0x3);
          __syncwarp();
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        if (ok && elect_one()) mma_commit_pair(acc_full_bar, 0x3);
        __syncwarp();
      }
      if (prof && lane == 0) {
        p.prof[blockIdx.x * kProfCount + kProfMmaWaitFull] = wait_full;
        p.prof[blockIdx.x * kProfCount + kProfMmaWaitAcc] = wait_acc;
        p.prof[blockIdx.x * kProfCount + kProfMmaTotal] = clock64() - t_begin;
        p.prof[blockIdx.x * kProfCount + kProfTiles] = local;
      }
    }
  } else if (warp >= 2 && warp < 2 + kEpiWarps) {
    // ------------------------------------------------------------- epilogue (8 warps, both CTAs)
    // Warp group g (warps 2-5 / 6-9) owns accumulator half g = columns [256 g, 256 g + 256) of
    // the tile; each warp its lane quarter's 32 rows.
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const uint32_t leader_acc_empty = mapa_u32(acc_empty_bar(group), 0);
    const uint32_t sbuf = store_base + (warp - 2) * kStoreBufBytes;
    StoreTarget out;
    out.tmap_d = &tmap_d;
    out.d_ptr = p.d_ptr;
    out.ldd = p.ldd;
    out.M = p.M;
    out.N = p.N;
    out.peers = &p.peers;
    out.alpha = 1.0f;
    out.row_end = p.M;
    int local = 0;
    bool ok = true;
    // The workspace and the flags are shared with the previous launch of the same plan, D with
    // whatever ran before: nothing is written until that grid has completed.
    griddep_wait();
    const bool prof = p.prof != nullptr && warp == 2 && lane == 0;
    long long waited = 0;
    const long long t_begin = prof ? clock64() : 0;
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + static_cast<uint32_t>(group * kTN);
    // This warp's part of a cluster's workspace slot.
    const size_t warp_off = (static_cast<size_t>(rank) * kEpiWarps + static_cast<size_t>(warp - 2)) * kPartialFloatsPerWarp;
    const size_t flag_off = static_cast<size_t>(rank) * kEpiWarps + static_cast<size_t>(warp - 2);
    Segment sg;
    for (; ok && segment_at(p.walk, cluster, n_clusters, num_kb, local, sg); ++local) {
      int tm, tn;
      tile_coords(sg.tile, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
      const long long w0 = prof ? clock64() : 0;
      if (!mbar_wait(acc_full_bar, static_cast<uint32_t>(local) & 1u)) {
        if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
        ok = false;
        break;
      }
      if (prof) waited += clock64() - w0;
      tc_fence_after_sync();
      const int row0 = tm * 256 + static_cast<int>(rank) * kBlockM + quarter * 32;
      const int col0 = tn * kTileN + group * kTN;
      if (sg.slot < 0 && sg.owned_parts == 0) {
        drain_and_store<kTN, true>(taddr, sbuf, out, row0, col0, leader_acc_empty, lane);
      } else if (sg.slot >= 0) {
        // A later part of a tile another cluster owns: fp32 partial sums to the part's slot, one
        // coalesced 128-byte store per accumulator column, then the flag.
        float* dst = p.partial + static_cast<size_t>(sg.slot) * kPartialFloatsPerCluster + warp_off + lane;
#pragma unroll 1
        for (int g = 0; g < kTN / 32; ++g) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + g * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[g * 1024 + i * 32] = __uint_as_float(v[i]);
        }
        release_columns(leader_acc_empty, lane);
        __threadfence();
        __syncwarp();
        if (lane == 0)
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.flags + static_cast<size_t>(sg.slot) * 2 * kEpiWarps + flag_off),
                       "r"(p.epoch)
                       : "memory");
      } else {
        // The first K blocks of a tile: this cluster owns it.  Wait for this warp's counterparts
        // in the clusters that hold the other parts, add their sums chunk by chunk, store.
        const int parts = sg.owned_parts;
        for (int j = 0; j < parts && ok; ++j) {
          const unsigned* flag = p.flags + static_cast<size_t>(sg.first_slot + j) * 2 * kEpiWarps + flag_off;
          const long long t0 = clock64();
          unsigned spins = 0;
          while (ld_acquire_gpu_u32(flag) != p.epoch) {
            if ((++spins & 0xff) == 0 && clock64() - t0 > SMB_WAIT_BUDGET_CYCLES) {
              if (lane == 0) report_status(p.status, kDevTimeoutFixup);
              ok = false;
              break;
            }
            __nanosleep(64);
          }
        }
        if (!ok) break;
        uint32_t packed[kTN / 2];
#pragma unroll
        for (int g = 0; g < kTN / 32; ++g) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + g * 32, v);
          tmem_ld_wait();
          for (int j = 0; j < parts; ++j) {
            const float* src = p.partial + static_cast<size_t>(sg.first_slot + j) * kPartialFloatsPerCluster + warp_off +
                               lane + g * 1024;
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) + __ldcg(src + i * 32));
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) packed[g * 16 + i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
        }
        release_columns(leader_acc_empty, lane);
        store_columns<kTN, true>(packed, sbuf, out, row0, col0, lane);
      }
    }
    drain_store_groups<true>(lane);
    if (prof) {
      p.prof[blockIdx.x * kProfCount + kProfEpiWait] = waited;
      p.prof[blockIdx.x * kProfCount + kProfEpiTotal] = clock64() - t_begin;
    }
  }
  __syncwarp();

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<2>(tmem_base, 512);
  }
}

}  // namespace bf16s

size_t bf16_streamk_workspace_bytes(int clusters) {
  return static_cast<size_t>(clusters) * bf16s::kPartialFloatsPerCluster * sizeof(float);
}
size_t bf16_streamk_flag_bytes(int clusters) {
  return static_cast<size_t>(clusters) * 2 * bf16s::kEpiWarps * sizeof(unsigned);
}

// How the last wave of `tiles` tiles on `clusters` clusters is cut, and an estimate of what the
// whole GEMM then costs in K-block times (the whole-tile walk costs ceil(tiles / clusters) * kb).
// Every later part of a tile costs its cluster about 5 us on top of its K blocks (the fp32 sums of
// a 256 x 512 tile are 512 KB per cluster, written with ordinary stores while the accumulator is
// still held), and the owner about as much again to read them: kStreamKHandOver K-block times.
// Measured (us per launch, whole tiles / this walk): 8192 x 4096 x 8192 362 / 352,
// 32768 x 7168 x 8192 2388 / 2377, 8192 x 2048 x 8192 182 / 189, 4096^3 92 / 105,
// 8192 x 1024 x 8192 93 / 123 (seven 16-block tails per spare cluster), 8192^3 677 / 726.
constexpr double kStreamKHandOver = 40.0;
double bf16_streamk_plan(long long tiles, int kb, int clusters, StreamKWalk* w) {
  w->full_waves = static_cast<int>(tiles / clusters);
  w->rem_tiles = static_cast<int>(tiles % clusters);
  w->cut = kb;
  w->tails_per_cluster = 0;
  w->parts = 0;
  const int R = w->rem_tiles, E = clusters - R;
  double last = 0.0;
  if (R > 0) {
    last = kb;
    if (E >= R && kb >= 2) {
      int parts = E / R;
      if (parts > kb - 1) parts = kb - 1;
      if (parts > 7) parts = 7;
      w->parts = parts;
      last = (kb + parts) / (parts + 1) + kStreamKHandOver;   // the longest slice
    } else if (E > 0) {
      const int T = (R + E - 1) / E;
      int best_cut = kb;
      double best = kb;
      for (int cut = kb - 1; cut >= 1; --cut) {
        const double cost = (cut > T * (kb - cut) ? cut : T * (kb - cut)) + kStreamKHandOver;
        if (cost < best) {
          best = cost;
          best_cut = cut;
        }
      }
      w->cut = best_cut;
      w->tails_per_cluster = best_cut < kb ? T : 0;
      last = best;
    }
  }
  return static_cast<double>(w->full_waves) * kb + last;
}

// Whether cutting the last wave is expected to pay by at least 3 % of the whole GEMM.  With the
// measured hand-over cost that is rare (long K, a last wave less than half full); plans take the
// walk on request (SMB_FLAG_STREAM_K) or where this says so.
bool bf16_streamk_pays(int M, int N, int K, int clusters) {
  if (clusters < 1 || N <= 256) return false;
  const long long tiles = static_cast<long long>((M + 255) / 256) * ((N + 511) / 512);
  const int kb = (K + 63) / 64;
  if (kb < 16) return false;   // short K loops: the partial sums would cost as much as they save
  StreamKWalk w;
  const double cut = bf16_streamk_plan(tiles, kb, clusters, &w);
  const double whole = static_cast<double>((tiles + clusters - 1) / clusters) * kb;
  return (w.parts > 0 || w.cut < kb) && cut < whole * 0.97;
}

}  // namespace smb

// Host-side view of the cut, for known-answer tests (no device needed).
extern "C" int smb_debug_bf16_streamk_plan(long long tiles, int kb, int clusters, int* out) {
  if (out == nullptr || tiles < 1 || kb < 1 || clusters < 1) return 0;
  smb::StreamKWalk w;
  const double cut = smb::bf16_streamk_plan(tiles, kb, clusters, &w);
  out[0] = w.full_waves;
  out[1] = w.rem_tiles;
  out[2] = w.cut;
  out[3] = w.tails_per_cluster;
  out[4] = w.parts;
  const double whole = static_cast<double>((tiles + clusters - 1) / clusters) * kb;
  return ((w.parts > 0 || w.cut < kb) && kb >= 16 && cut < whole * 0.97) ? 1 : 0;
}

namespace smb {

int bf16_streamk_launch(const Bf16Launch& L, cudaStream_t stream) {
  auto kernel = bf16s::gemm_bf16_streamk_kernel;
  static thread_local int configured_device = -1;
  static thread_local int max_clusters = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_error(SMB_ERR_CUDA, "cudaGetDevice failed");
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bf16s::kTotal);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaFuncSetAttribute(bf16 stream-K smem)");
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2, 1, 1);
    probe.blockDim = dim3(bf16s::kThreads, 1, 1);
    probe.dynamicSmemBytes = bf16s::kTotal;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    probe.attrs = &attr;
    probe.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kernel, &probe);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaOccupancyMaxActiveClusters(bf16 stream-K)");
    if (n <= 0) return set_error(SMB_ERR_CUDA, "no 2-CTA cluster of the bf16 stream-K kernel fits on this device");
    max_clusters = n;
    configured_device = dev;
  }
  if (!L.tma_store || L.swiglu || L.peers.count > 0 || L.peers.route_rows > 0 || L.mtile_group != nullptr ||
      L.tile_row0 != nullptr || L.streamk_partial == nullptr || L.streamk_flags == nullptr)
    return set_error(SMB_ERR_UNSUPPORTED, "bf16: the stream-K walk has only the plain aligned store and needs its workspace");
  bf16s::Params p;
  p.M = L.M;
  p.N = L.N;
  p.K = L.K;
  p.tiles_m = (L.M + 255) / 256;
  p.tiles_n = (L.N + bf16s::kTileN - 1) / bf16s::kTileN;
  p.group_m = L.group_m > 0 ? L.group_m
                            : raster_group_rows(p.tiles_m, static_cast<long long>(L.K) * 2,
                                                static_cast<long long>(L.N) * L.K * 2);
  p.ldd = L.ldd;
  p.d_ptr = static_cast<uint16_t*>(L.d);
  p.status = L.status;
  p.prof = L.prof;
  p.peers.count = 0;
  p.peers.route_rows = 0;
  p.peers.first_block = 0;
  p.partial = L.streamk_partial;
  p.flags = L.streamk_flags;
  p.epoch = L.streamk_epoch;
  p.operands_static = L.operands_static ? 1 : 0;
  p.l2_a = L.l2_a;
  p.l2_b = L.l2_b;
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  int clusters = max_clusters;
  if (L.max_clusters > 0 && clusters > L.max_clusters) clusters = L.max_clusters;
  if (clusters > L.streamk_clusters) clusters = L.streamk_clusters;   // what the workspace has slots for
  bf16_streamk_plan(tiles, (L.K + 63) / 64, clusters, &p.walk);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(bf16s::kThreads, 1, 1);
  cfg.dynamicSmemBytes = bf16s::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute pdl;
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L.tmap_a, L.tmap_b, L.tmap_d, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "bf16 stream-K GEMM launch");
  return SMB_OK;
}

}  // namespace smb
