// Block-scaled FP4 GEMM for short K (K <= 2048) on sm_100a: the A panel stays in shared memory.
//
// Same arithmetic as gemm_nvfp4.cu (E2M1 codes, one UE8M0 scale per 32 K, kind::mxf4nvf4
// scale_vec::2X, FP32 accumulate, BF16 out).  What differs is the schedule, the counterpart of
// the reference's static same-row runs (src/kernels/gemm/sm100a/nvfp4/dense_gemm_nvfp4.cu:372-434):
//
//   * A cluster (2 CTAs, 256 rows) works through a RUN of consecutive 192-column tiles of one
//     tile row.  The row's A panel (128 rows x K/2 bytes per CTA, at most 8 K blocks = 128 KiB)
//     and its scales are loaded once per run into fixed slots and read again for every tile of
//     the run; only B and its scales stream through a 4-stage ring.  With short K the general
//     kernel spends its time waiting for operands (every tile pulls A and B through L2 again);
//     here a K block costs a CTA 14 KiB of L2 traffic instead of 44.
//   * Tiles are 256 x 192 so that TWO accumulator sets fit into tensor memory (2 x 192 columns
//     + 4 scale slots of 24): the epilogue of one tile overlaps the instructions of the next.
//     With 8 K blocks per tile the read-out would otherwise idle the tensor pipe a quarter of
//     the time.
//   * 192 columns are one and a half 128-row bands of B scales: every tile loads the two bands
//     it touches and odd tiles start two tensor-memory columns (64 rows) into the first.
//
// Shared memory (per CTA, after 1024-byte alignment):
//   [A slot 0..7: 128 rows x 128 B, 128-byte swizzle][SFA slot 0..7: 2 cells x 512 B]
//   [ring 0..3: B 96 rows x 128 B | SFB 2 bands x 2 cells x 512 B][8 store boxes x 4 KiB][barriers]
#include "epilogue.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace smb {

namespace fp4r {

constexpr int kBlockM = 128;
constexpr int kBlockKBytes = 128;     // bytes of K per row and K block (256 E2M1 values)
constexpr int kBlockK = 256;
constexpr int kThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kTileN = 192;
constexpr int kMaxKb = 8;             // K <= 2048
constexpr int kStages = 4;
constexpr int kCells = 2;             // 4-byte scale cells (K = 128) per row and K block
constexpr int kSfCellBytes = 512;     // 128 rows x 4 scale bytes
constexpr int kABytes = kBlockM * kBlockKBytes;             // 16 KiB
constexpr int kSfaBytes = kCells * kSfCellBytes;            // 1 KiB
constexpr int kBBytes = (kTileN / 2) * kBlockKBytes;        // 12 KiB: this CTA's 96 rows of B
constexpr int kBands = 2;                                   // 128-row scale bands a tile touches
constexpr int kSfbBytes = kBands * kCells * kSfCellBytes;   // 2 KiB
constexpr int kStageBytes = kBBytes + kSfbBytes;            // 14 KiB
constexpr int kOffSfb = kBBytes;
constexpr int kOffSfa = kMaxKb * kABytes;
constexpr int kOffRing = kOffSfa + kMaxKb * kSfaBytes;
constexpr int kOffStore = kOffRing + kStages * kStageBytes;
constexpr int kOffBars = kOffStore + kEpiWarps * kStoreBufBytes;
constexpr int kTotal = 1024 + kOffBars + 1024;
// Tensor memory: two accumulator sets, then one scale slot per ring stage:
// [SFA cell 0 (4 columns) | SFA cell 1 | SFB cell 0: band 0, band 1 | SFB cell 1: band 0, band 1].
constexpr int kAccCols = 2 * kTileN;
constexpr int kSlotCols = kCells * 4 + kBands * kCells * 4;
static_assert(kStageBytes % 1024 == 0 && kOffRing % 1024 == 0, "ring stages must stay 1024-byte aligned");
static_assert(kAccCols + kStages * kSlotCols <= 512, "tensor memory budget");
static_assert(kTotal <= 232448, "shared memory budget");

struct Params {
  int M, N, K;
  int tiles_m, tiles_n;
  int chunks, run_len;   // a tile row is cut into `chunks` runs of `run_len` tiles (the last may be shorter)
  int ldd;
  uint16_t* d_ptr;
  int* status;
  long long* prof;       // optional role timers: 8 counters per CTA, as in gemm_nvfp4.cu
  PeerCopies peers;      // extra destinations of every stored box (count 0: none)
  int m_rotate;          // the walk over tile rows starts here (0 unless rows are routed)
  int operands_static;   // 0: wait for the previous kernel before loading; 1: only before storing; 2: never
};

enum { kProfLoadWait = 0, kProfLoadTotal, kProfMmaWaitFull, kProfMmaWaitAcc, kProfMmaTotal,
       kProfEpiWait, kProfEpiTotal, kProfTiles, kProfCount };

template <bool kTmaStore>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_nvfp4_arun_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                       const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring_base = smem_base + kOffRing;
  const uint32_t store_base = smem_base + kOffStore;
  const uint32_t bar_base = smem_base + kOffBars;
  auto a_slot = [&](int kb) { return smem_base + static_cast<uint32_t>(kb) * kABytes; };
  auto sfa_slot = [&](int kb) { return smem_base + kOffSfa + static_cast<uint32_t>(kb) * kSfaBytes; };
  auto b_full_bar = [&](int s) { return bar_base + 8u * s; };
  auto b_empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto sfb_full_bar = [&](int s) { return bar_base + 8u * (2 * kStages + s); };
  auto sf_ready_bar = [&](int s) { return bar_base + 8u * (3 * kStages + s); };
  auto a_full_bar = [&](int kb) { return bar_base + 8u * (4 * kStages + kb); };
  auto a_empty_bar = [&](int kb) { return bar_base + 8u * (4 * kStages + kMaxKb + kb); };
  auto sfa_full_bar = [&](int kb) { return bar_base + 8u * (4 * kStages + 2 * kMaxKb + kb); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (4 * kStages + 3 * kMaxKb + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (4 * kStages + 3 * kMaxKb + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (4 * kStages + 3 * kMaxKb + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = static_cast<int>(cluster_id_x());
  const int n_clusters = static_cast<int>(num_clusters_x());
  const int num_runs = p.tiles_m * p.chunks;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;

  griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(b_full_bar(s), 1);
      mbar_init(b_empty_bar(s), 1);
      mbar_init(sfb_full_bar(s), 1);
      mbar_init(sf_ready_bar(s), 1);
    }
    for (int kb = 0; kb < kMaxKb; ++kb) {
      mbar_init(a_full_bar(kb), 1);
      mbar_init(a_empty_bar(kb), 1);
      mbar_init(sfa_full_bar(kb), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 2 * kEpiWarps);   // all epilogue warps of both CTAs
    }
    fence_mbar_init_cluster();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
    if (kTmaStore) tma_prefetch_desc(&tmap_d);
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
    const uint32_t leader_b_full0 = mapa_u32(b_full_bar(0), 0);
    const uint32_t leader_sfb_full0 = mapa_u32(sfb_full_bar(0), 0);
    const uint32_t leader_a_full0 = mapa_u32(a_full_bar(0), 0);
    const uint32_t leader_sfa_full0 = mapa_u32(sfa_full_bar(0), 0);
    int s = 0;
    uint32_t ph = 0;
    uint32_t run_parity = 0;
    bool ok = true;
    const bool prof = p.prof != nullptr;
    long long waited = 0;
    const long long t_begin = prof ? clock64() : 0;
    if (!p.operands_static) griddep_wait();
    for (int r = cluster; r < num_runs && ok; r += n_clusters, run_parity ^= 1u) {
      const int tm = (r % p.tiles_m + p.m_rotate) % p.tiles_m;   // routed stores: ranks start at different row blocks
      const int tn0 = (r / p.tiles_m) * p.run_len;
      const int tn1 = tn0 + p.run_len < p.tiles_n ? tn0 + p.run_len : p.tiles_n;
      const int row_a = tm * 256 + static_cast<int>(rank) * kBlockM;
      for (int tn = tn0; tn < tn1 && ok; ++tn) {
        const int col0 = tn * kTileN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (tn == tn0) {
            // The run's A panel, K block by K block, each as soon as the previous run's last
            // tile is through with the slot; interleaved with the B loads so that neither waits
            // for the other.
            if (!mbar_wait(a_empty_bar(kb), run_parity ^ 1u)) {
              report_status(p.status, kDevTimeoutProducer);
              ok = false;
              break;
            }
            if (elect_one()) {
              if (rank == 0) {
                mbar_arrive_expect_tx(sfa_full_bar(kb), 2 * kSfaBytes);
                mbar_arrive_expect_tx(a_full_bar(kb), 2 * kABytes);
              }
              tma_load_2d_pair(sfa_slot(kb), &tmap_sfa, leader_sfa_full0 + 8u * kb, kb * (kCells * 64), row_a / 128);
              tma_load_2d_pair(a_slot(kb), &tmap_a, leader_a_full0 + 8u * kb, kb * kBlockKBytes, row_a);
            }
            __syncwarp();
          }
          const long long w0 = prof ? clock64() : 0;
          if (!mbar_wait(b_empty_bar(s), ph ^ 1u)) {
            report_status(p.status, kDevTimeoutProducer);
            ok = false;
            break;
          }
          if (prof) waited += clock64() - w0;
          if (elect_one()) {
            const uint32_t dst = ring_base + s * kStageBytes;
            if (rank == 0) {
              mbar_arrive_expect_tx(sfb_full_bar(s), 2 * kSfbBytes);
              mbar_arrive_expect_tx(b_full_bar(s), 2 * kBBytes);
            }
            tma_load_2d_pair(dst + kOffSfb, &tmap_sfb, leader_sfb_full0 + 8u * s, kb * (kCells * 64), col0 / 128);
            tma_load_2d_pair(dst, &tmap_b, leader_b_full0 + 8u * s, kb * kBlockKBytes,
                             col0 + static_cast<int>(rank) * (kTileN / 2));
          }
          __syncwarp();
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
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
      int s = 0;
      uint32_t ph = 0;
      uint32_t run_parity = 0;
      int local = 0;
      bool ok = true;
      const bool prof = p.prof != nullptr;
      long long wait_full = 0, wait_acc = 0;
      const long long t_begin = prof ? clock64() : 0;
      for (int r = cluster; r < num_runs && ok; r += n_clusters, run_parity ^= 1u) {
        const int tn0 = (r / p.tiles_m) * p.run_len;
        const int tn1 = tn0 + p.run_len < p.tiles_n ? tn0 + p.run_len : p.tiles_n;
        for (int tn = tn0; tn < tn1 && ok; ++tn, ++local) {
          const int bank = local & 1;
          const long long a0 = prof ? clock64() : 0;
          if (!mbar_wait(acc_empty_bar(bank), (static_cast<uint32_t>(local >> 1) & 1u) ^ 1u)) {
            report_status(p.status, kDevTimeoutMmaAcc);
            ok = false;
            break;
          }
          if (prof) wait_acc += clock64() - a0;
          tc_fence_after_sync();
          const uint32_t acc = tmem_base + static_cast<uint32_t>(bank * kTileN);
          // Odd tiles start 64 rows into their first scale band: two columns further.
          const uint32_t band_shift = (tn & 1) ? 2u : 0u;
          for (int kb = 0; kb < num_kb && ok; ++kb) {
            const long long w0 = prof ? clock64() : 0;
            if (tn == tn0 && !mbar_wait(a_full_bar(kb), run_parity)) {
              report_status(p.status, kDevTimeoutMmaFull);
              ok = false;
              break;
            }
            if (!mbar_wait(b_full_bar(s), ph) || !mbar_wait(sf_ready_bar(s), ph)) {
              report_status(p.status, kDevTimeoutMmaFull);
              ok = false;
              break;
            }
            if (prof) wait_full += clock64() - w0;
            tc_fence_after_sync();
            if (elect_one()) {
              const uint32_t sf_t = tmem_base + static_cast<uint32_t>(kAccCols + s * kSlotCols);
              const uint64_t desc_a = make_smem_desc(a_slot(kb), 1024, 16, kSwizzle128B);
              const uint64_t desc_b = make_smem_desc(ring_base + s * kStageBytes, 1024, 16, kSwizzle128B);
#pragma unroll
              for (int ki = 0; ki < 4; ++ki) {
                // K = 64 per instruction = 32 bytes along the swizzled row; instructions 2c and
                // 2c + 1 share scale cell c (scale ids 0 and 2).
                const uint32_t sf_id = (ki & 1) ? 2u : 0u;
                const uint32_t cell = static_cast<uint32_t>(ki >> 1);
                const uint32_t idesc = make_idesc_mxf4(256, kTileN, sf_id, sf_id, true);
                mma_mxf4_ss<2>(acc, desc_a + 2u * ki, desc_b + 2u * ki, idesc, sf_t + 4u * cell,
                               sf_t + static_cast<uint32_t>(kCells * 4) + cell * (kBands * 4) + band_shift,
                               (kb > 0 || ki > 0) ? 1u : 0u);
              }
              mma_commit_pair(b_empty_bar(s), 0x3);
              if (tn == tn1 - 1) mma_commit_pair(a_empty_bar(kb), 0x3);   // the run is through with this slot
              if (kb == num_kb - 1) mma_commit_pair(acc_full_bar(bank), 0x3);
            }
            __syncwarp();
            if (++s == kStages) { s = 0; ph ^= 1u; }
          }
        }
      }
      if (prof && lane == 0) {
        p.prof[blockIdx.x * kProfCount + kProfMmaWaitFull] = wait_full;
        p.prof[blockIdx.x * kProfCount + kProfMmaWaitAcc] = wait_acc;
        p.prof[blockIdx.x * kProfCount + kProfMmaTotal] = clock64() - t_begin;
        p.prof[blockIdx.x * kProfCount + kProfTiles] = local;
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------- scale copies (leader CTA only)
    // Shared memory -> tensor memory with tcgen05.cp (32 lines of 16 bytes = 128 rows x 4 scale
    // bytes into 4 columns, replicated into all four lane quarters), issued for both CTAs.  A's
    // scales are copied again for every tile of the run (the tensor-memory slot belongs to the
    // ring stage), from the slot they were loaded into once.
    if (rank == 0) {
      int s = 0;
      uint32_t ph = 0;
      uint32_t run_parity = 0;
      bool ok = true;
      for (int r = cluster; r < num_runs && ok; r += n_clusters, run_parity ^= 1u) {
        const int tn0 = (r / p.tiles_m) * p.run_len;
        const int tn1 = tn0 + p.run_len < p.tiles_n ? tn0 + p.run_len : p.tiles_n;
        for (int tn = tn0; tn < tn1 && ok; ++tn) {
          for (int kb = 0; kb < num_kb; ++kb) {
            if ((tn == tn0 && !mbar_wait(sfa_full_bar(kb), run_parity)) || !mbar_wait(sfb_full_bar(s), ph)) {
              report_status(p.status, kDevTimeoutSched);
              ok = false;
              break;
            }
            tc_fence_after_sync();
            if (elect_one()) {
              const uint32_t sf_t = tmem_base + static_cast<uint32_t>(kAccCols + s * kSlotCols);
              const uint64_t sfa_desc = make_smem_desc(sfa_slot(kb), 128, 16, kSwizzleNone);
              const uint64_t sfb_desc = make_smem_desc(ring_base + s * kStageBytes + kOffSfb, 128, 16, kSwizzleNone);
#pragma unroll
              for (int cell = 0; cell < kCells; ++cell)
                tmem_cp_32x128b_warpx4<2>(sf_t + 4u * cell, sfa_desc + cell * (kSfCellBytes / 16));
              // Shared memory holds [band][cell], tensor memory [cell][band]: an instruction reads
              // the 6 adjacent columns of its 192 rows.
#pragma unroll
              for (int cell = 0; cell < kCells; ++cell) {
#pragma unroll
                for (int b = 0; b < kBands; ++b) {
                  tmem_cp_32x128b_warpx4<2>(sf_t + static_cast<uint32_t>(kCells * 4 + (cell * kBands + b) * 4),
                                            sfb_desc + (b * kCells + cell) * (kSfCellBytes / 16));
                }
              }
              mma_commit_pair(sf_ready_bar(s), 0x1);
            }
            __syncwarp();
            if (++s == kStages) { s = 0; ph ^= 1u; }
          }
        }
      }
    }
  } else if (warp >= 2 && warp < 2 + kEpiWarps) {
    // ------------------------------------------------------------- epilogue (8 warps, both CTAs)
    // Warp group 0 takes columns 0-127 of the tile, group 1 columns 128-191; each warp its lane
    // quarter's 32 rows.
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const uint32_t leader_acc_empty0 = mapa_u32(acc_empty_bar(0), 0);
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
    if (p.operands_static == 1) griddep_wait();
    const bool prof = p.prof != nullptr && warp == 2 && lane == 0;
    long long waited = 0;
    const long long t_begin = prof ? clock64() : 0;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    for (int r = cluster; r < num_runs && ok; r += n_clusters) {
      const int tm = (r % p.tiles_m + p.m_rotate) % p.tiles_m;   // routed stores: ranks start at different row blocks
      const int tn0 = (r / p.tiles_m) * p.run_len;
      const int tn1 = tn0 + p.run_len < p.tiles_n ? tn0 + p.run_len : p.tiles_n;
      const int row0 = tm * 256 + static_cast<int>(rank) * kBlockM + quarter * 32;
      for (int tn = tn0; tn < tn1; ++tn, ++local) {
        const int bank = local & 1;
        const long long w0 = prof ? clock64() : 0;
        if (!mbar_wait(acc_full_bar(bank), static_cast<uint32_t>(local >> 1) & 1u)) {
          if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
          ok = false;
          break;
        }
        if (prof) waited += clock64() - w0;
        tc_fence_after_sync();
        const uint32_t taddr = lane_base + static_cast<uint32_t>(bank * kTileN + group * 128);
        const int col0 = tn * kTileN + group * 128;
        if (group == 0)
          drain_and_store<128, kTmaStore>(taddr, sbuf, out, row0, col0, leader_acc_empty0 + 8u * bank, lane);
        else
          drain_and_store<64, kTmaStore>(taddr, sbuf, out, row0, col0, leader_acc_empty0 + 8u * bank, lane);
      }
    }
    drain_store_groups<kTmaStore>(lane);
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

}  // namespace fp4r

// -----------------------------------------------------------------------------------
// Host side
// -----------------------------------------------------------------------------------
namespace {

// Cycles a 256 x 192 tile of `kb` K blocks keeps a cluster busy, and what a run costs on top (its
// first K blocks wait for A).  Measured, all 74 clusters running: 880-950 cycles per K block
// (the tensor pipe alone would need 384): a B load takes 2100 cycles from issue to arrival on an
// otherwise idle GPU and 2600-2900 under load, whether or not the line is already in L2, and
// the ring holds four of them.
constexpr double kArunCyclesPerKBlock = 900.0;
// A run costs about 0.45 tiles on top of its tiles (splits chosen with that ratio measured 10-25 %
// faster on 4096^2 x 2048 and 14080 x 5120 x 2048 than splits chosen with a fifth of a tile).
constexpr double kArunTileOverhead = 150.0, kArunRunOverheadTiles = 0.45;

}  // namespace

bool fp4_arun_supports(int M, int N, int K) {
  return K <= fp4r::kMaxKb * fp4r::kBlockK && N >= 2 * fp4r::kTileN && M >= 1;
}

double fp4_arun_split(int M, int N, int K, int clusters, int* chunks, int* run_len) {
  const int tiles_m = (M + 255) / 256;
  const int tiles_n = (N + fp4r::kTileN - 1) / fp4r::kTileN;
  const double kb = (K + fp4r::kBlockK - 1) / fp4r::kBlockK;
  const double tile = kb * kArunCyclesPerKBlock + kArunTileOverhead;
  if (clusters < 1) clusters = 1;
  double best = -1.0;
  for (int c = 1; c <= tiles_n; ++c) {
    const int len = (tiles_n + c - 1) / c;
    if ((c - 1) * len >= tiles_n) continue;   // the last run would be empty
    const long long runs = static_cast<long long>(tiles_m) * c;
    const long long waves = (runs + clusters - 1) / clusters;
    const double cost = static_cast<double>(waves) * (len * tile + kArunRunOverheadTiles * tile);
    if (best < 0.0 || cost < best * 0.999) {
      best = cost;
      *chunks = c;
      *run_len = len;
    }
  }
  return best;
}

}  // namespace smb

// Host-side view of the run split, for known-answer tests (no device needed).
extern "C" int smb_debug_fp4_arun_split(int M, int N, int K, int clusters, int* chunks, int* run_len) {
  if (!smb::fp4_arun_supports(M, N, K)) return 0;
  smb::fp4_arun_split(M, N, K, clusters, chunks, run_len);
  return 1;
}

namespace smb {

namespace {

template <bool kTmaStore>
int launch_arun(const Fp4Launch& L, cudaStream_t stream) {
  auto kernel = fp4r::gemm_nvfp4_arun_kernel<kTmaStore>;
  static thread_local int configured_device = -1;
  static thread_local int max_clusters = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_error(SMB_ERR_CUDA, "cudaGetDevice failed");
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, fp4r::kTotal);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaFuncSetAttribute(nvfp4 A-resident smem)");
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2, 1, 1);
    probe.blockDim = dim3(fp4r::kThreads, 1, 1);
    probe.dynamicSmemBytes = fp4r::kTotal;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    probe.attrs = &attr;
    probe.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kernel, &probe);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaOccupancyMaxActiveClusters(nvfp4 A-resident)");
    if (n <= 0) return set_error(SMB_ERR_CUDA, "no 2-CTA cluster of the A-resident nvfp4 kernel fits on this device");
    max_clusters = n;
    configured_device = dev;
  }
  int clusters = max_clusters;
  if (L.max_clusters > 0 && clusters > L.max_clusters) clusters = L.max_clusters;
  fp4r::Params p;
  p.M = L.M;
  p.N = L.N;
  p.K = L.K;
  p.tiles_m = (L.M + 255) / 256;
  p.tiles_n = (L.N + fp4r::kTileN - 1) / fp4r::kTileN;
  p.chunks = 1;
  p.run_len = p.tiles_n;
  fp4_arun_split(L.M, L.N, L.K, clusters, &p.chunks, &p.run_len);
  p.ldd = L.ldd;
  p.d_ptr = static_cast<uint16_t*>(L.d);
  p.status = L.status;
  p.prof = L.prof;
  p.peers = L.peers;
  p.m_rotate = L.peers.route_rows > 0 ? (L.peers.first_block * (L.peers.route_rows / 256)) % p.tiles_m : 0;
  p.operands_static = L.operands_static ? (L.output_independent ? 2 : 1) : 0;
  const long long runs = static_cast<long long>(p.tiles_m) * p.chunks;
  if (runs < clusters) clusters = static_cast<int>(runs);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(fp4r::kThreads, 1, 1);
  cfg.dynamicSmemBytes = fp4r::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute pdl;
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L.tmap_a, L.tmap_b0, L.tmap_sfa, L.tmap_sfb, L.tmap_d, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "nvfp4 A-resident GEMM launch");
  return SMB_OK;
}

}  // namespace

int fp4_arun_launch(const Fp4Launch& L, cudaStream_t stream) {
  if (!fp4_arun_supports(L.M, L.N, L.K))
    return set_error(SMB_ERR_UNSUPPORTED, "nvfp4: the A-resident kernel needs K <= 2048 and N >= 384");
  if (L.block16 || L.swiglu || L.mtile_group != nullptr || L.tile_row0 != nullptr || L.dynamic)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "nvfp4: the A-resident kernel has no block-16, gated, grouped or queued form");
  return L.tma_store ? launch_arun<true>(L, stream) : launch_arun<false>(L, stream);
}

}  // namespace smb
