// Dense BF16 GEMM for sm_100a:  D[M,N] = bf16( A[M,K] . BT[N,K]^T ), FP32 accumulate.
//
// From-scratch counterpart of the reference kernel dense_gemm_bf16_k0_impl
// (src/kernels/gemm/sm100a/dense_gemm_bf16.cu:86-234) and of the warp-role bodies it
// composes (blocks/88 load, blocks/90 MMA, blocks/93 epilogue, blocks/97 scheduler).
// Differences by design: M, N and K are run-time values with edge predication (the
// reference takes K as a template value and rejects ragged shapes); the epilogue stages
// through 128-byte-swizzled shared memory with one TMA store chain per warp (no CTA-wide
// barrier); every wait is bounded; tiles are walked in a grouped raster so that the
// clusters of one wave share A and B panels in L2; and for long K a 256 x 512 tile is
// used, because on B200 the L2 sector rate, not the tensor pipe, limits a 256 x 256 tile
// fed without multicast loads.
//
// One cluster = 2 CTAs = one output tile of 256 x (NB * TN), TN in {256, 128, 64}, NB in {1, 2}:
//   CTA r loads A rows [m0 + 128 r, +128) and, per N sub-block h, BT rows
//   [n0 + h TN + TN/2 r, +TN/2) for each 64-wide K block; the leader CTA (rank 0) issues
//   tcgen05.mma.cta_group::2 with M = 256, N = TN, K = 16; CTA r ends up with rows
//   [m0 + 128 r, +128) of the tile as fp32 in its tensor memory.
// Tensor memory (512 columns) holds two accumulator slots of up to 256 columns:
//   NB = 1: the slots are two banks, the epilogue of tile i overlaps the main loop of i + 1;
//   NB = 2: the slots are the two N halves of one tile; the MMA role restarts half h of the
//           next tile as soon as the epilogue has drained half h.
// Warp roles per CTA (352 threads): warp 0 TMA producer, warp 1 MMA issue + TMEM owner, warp 10
// tile scheduler (sched.cuh), warps 2-9 epilogue (warp w reads TMEM lanes 32 (w % 4) .. +31; warps 2-5 take the first
// half of a slot's columns / slot 0, warps 6-9 the second half / slot 1).
#include "epilogue.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"
#include "sched.cuh"

namespace smb {

namespace bf16k {

constexpr int kBlockM = 128;          // rows of A per CTA
constexpr int kBlockK = 64;           // K elements per stage (= 128 bytes per row)
constexpr int kThreads = 352;
constexpr int kEpiWarps = 8;
constexpr int kABytes = kBlockM * kBlockK * 2;        // 16 KiB
enum { kStorePlain = 0, kStoreTma = 1, kStoreSwiglu = 2 };   // epilogue variants

// R = CTAs of this kernel that fit on one SM.  Narrow tiles (N <= 128 problems) move 1.5 to 2.5
// times the operand bytes per flop of a 256-wide tile and are bound by the L2 -> SM path, not by
// the tensor pipe.  With R = 2 their CTAs take half the shared memory (a 3 or 4 stage ring), half
// the tensor memory and at most 88 registers, so that prologue, first load, accumulator drain and
// exit of one cluster overlap the main loop of a neighbour on the same SM pair.  That pays when
// launches overlap (operands not produced by the previous kernel: measured 6.2 against 9.7 us per
// launch of 14080 x 128 x 2048).  A launch that runs alone is better off with R = 1: two clusters
// that start together on one SM pair while other pairs idle take twice as long as one.
template <int TN, int NB, int R = 1>
struct Cfg {
  static_assert(TN == 64 || TN == 128 || TN == 256, "tile width");
  static_assert(NB == 1 || (NB == 2 && TN == 256), "two sub-blocks only at full width");
  static_assert(R == 1 || (R == 2 && TN <= 128), "two resident CTAs only for narrow tiles");
  static constexpr int kResident = R;
  static constexpr int kRingBudget = (kResident == 2) ? (TN == 64 ? 92 : 76) * 1024 : 192 * 1024;
  static constexpr int kTmemCols = (kResident == 2) ? 2 * TN : 512;   // two accumulator slots
  static constexpr int kBBytes = (TN / 2) * kBlockK * 2;         // one sub-block, one CTA
  static constexpr int kStageBytes = kABytes + NB * kBBytes;
  static constexpr int kStages = kRingBudget / kStageBytes;      // R = 1: 9, 8, 6 or 4; R = 2: 4 or 3
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kTileN = TN * NB;
  // Columns of one accumulator slot are split between the two epilogue warp groups when
  // there are at least 128 of them (each group then stores whole 64-column boxes).
  static constexpr int kGroupsPerSlot = (NB == 2) ? 1 : (TN >= 128 ? 2 : 1);
  static constexpr int kEpiWarpsActive = (NB == 2) ? kEpiWarps : 4 * kGroupsPerSlot;
  static constexpr int kStoreBytes = kEpiWarpsActive * kStoreBufBytes;   // working warps come first
  static constexpr int kBarrierBytes = 1024;
  // + 1024 so that the kernel can round the dynamic base up to a 1024-byte boundary.
  static constexpr int kTotal = 1024 + kRingBytes + kStoreBytes + kBarrierBytes;
  static constexpr int kColsPerWarp = TN / kGroupsPerSlot;
  static constexpr int kSlotReaders = 2 * 4 * kGroupsPerSlot;    // arrivals per drained slot
  static_assert(kTotal <= (kResident == 2 ? 115712 : 232448), "shared memory budget");
  static_assert(kStages >= 2 && kStages <= 16, "ring depth");
};

struct Params {
  int M, N, K;
  int tiles_m, tiles_n;
  int group_m;        // raster group height in tiles
  int ldd;            // elements between rows of D (used by the plain-store epilogue)
  uint16_t* d_ptr;    // D base (used by the plain-store epilogue)
  int* status;
  long long* prof;    // optional: 8 cycle counters per CTA (see kProf* below), or null
  int dynamic;        // 1: tiles come from the hardware work queue (one cluster launched per tile)
  PeerCopies peers;     // extra destinations of every stored box (count 0: none)
  int m_rotate;         // the tile walk starts at this 256-row tile (0 unless rows are routed)
  const int* mtile_group;  // grouped GEMM: group of every 256-row tile of A (device), or null
  const int* tile_row0;    // ragged groups: first row of every row tile (device), or null: tile t starts at 256 t
  const int* tile_row_end; // ... and the row where the tile's group ends
  int operands_static;  // 1: A and BT are not written by the previous kernel on the stream
  int l2_a, l2_b;       // L2 eviction hint of the A / BT loads: 0 none, 1 evict-last, 2 evict-first
};

// Per-CTA role timers (cycles), written when Params::prof is set.
enum { kProfLoadWait = 0, kProfLoadTotal, kProfMmaWaitFull, kProfMmaWaitAcc, kProfMmaTotal,
       kProfEpiWait, kProfEpiTotal, kProfTiles, kProfCount };

template <int TN, int NB, int kStore, int R>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, R)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ Params p) {
  using C = Cfg<TN, NB, R>;
  constexpr bool kTmaStore = (kStore != kStorePlain);
  constexpr bool kSwiglu = (kStore == kStoreSwiglu);   // D is [M, N/2]: silu(gate) * up
  static_assert(!kSwiglu || C::kColsPerWarp % 128 == 0, "gated epilogue: 64 output columns per box");
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring_base = smem_base;
  const uint32_t store_base = ring_base + C::kRingBytes;
  const uint32_t bar_base = store_base + C::kStoreBytes;
  // Barrier block: full[kStages], empty[kStages], acc_full[2], acc_empty[2], tmem slot.
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
  SchedSmem sched;
  sched.response = bar_base + 512u;
  sched.slot_full = bar_base + 528u;
  sched.slot_empty = bar_base + 536u;
  // Consumers of a scheduler response: both load threads, the MMA thread, every working epilogue warp.
  constexpr int kEpiWarpsActive = C::kEpiWarpsActive;
  constexpr int kSchedConsumers = 2 + 1 + 2 * kEpiWarpsActive;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = static_cast<int>(cluster_id_x());
  const int n_clusters = static_cast<int>(num_clusters_x());
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;

  // Programmatic dependent launch: the next kernel on the stream may begin its prologue while
  // this grid is still running (it waits, below, before it loads or stores anything).
  griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);    // the leader's arrive.expect_tx covers both CTAs' bytes
      mbar_init(empty_bar(s), 1);   // one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);                 // one tcgen05.commit
      mbar_init(acc_empty_bar(b), C::kSlotReaders);  // every epilogue warp that reads the slot
    }
    mbar_init(sched.slot_full, 1);
    mbar_init(sched.slot_empty, kSchedConsumers);
    fence_mbar_init_cluster();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (kTmaStore) tma_prefetch_desc(&tmap_d);
  }
  if (warp == 1) {
    tmem_alloc<2>(tmem_slot, C::kTmemCols);
    tmem_relinquish<2>();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  uint32_t tmem_base;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot) : "memory");

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    // The whole warp walks the loop and waits; one elected lane issues.  Keeping the control
    // flow warp-uniform lets the compiler hold addresses and descriptors in uniform registers,
    // which is what the TMA and tcgen05 instructions take (measured on the FP4 kernel: the same
    // loop run by lane 0 alone issued each instruction about 50 cycles slower).
    {
      const uint32_t leader_full0 = mapa_u32(full_bar(0), 0);
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      const bool prof = p.prof != nullptr;
      long long waited = 0;
      const long long t_begin = prof ? clock64() : 0;
      TileCursor cursor;
      cursor.init(p.dynamic != 0, n_clusters, num_tiles, sched);
      const uint64_t pol_a = p.l2_a == 2 ? l2_policy_evict_first() : l2_policy_evict_last();
      const uint64_t pol_b = p.l2_b == 2 ? l2_policy_evict_first() : l2_policy_evict_last();
      // Everything before this point overlapped the tail of the previous kernel on the stream;
      // its results (possibly this kernel's operands, certainly the old contents of D) are
      // complete and visible once this returns.  Unless the caller vouches that the operands are
      // not that kernel's output, all data flow of this kernel starts here; if it does, only the
      // epilogue waits (before it overwrites D) and loads and MMAs overlap the previous tail.
      if (!p.operands_static) griddep_wait();
      for (int t = cluster; t >= 0 && ok; t = cursor.next(t, lane == 0, true)) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
        tm = (tm + p.m_rotate) % p.tiles_m;   // routed stores: ranks start at different row blocks
        const int row_a = (p.tile_row0 != nullptr ? __ldg(p.tile_row0 + tm) : tm * 256) + static_cast<int>(rank) * kBlockM;
        // Grouped GEMM: BT is [groups * N, K]; the rows of this row tile of A belong to one group
        // (rows it reads beyond the end of its group are never stored) and meet that group's N rows.
        const int group_row = p.mtile_group != nullptr ? __ldg(p.mtile_group + tm) * p.N : 0;
        const int row_b = group_row + tn * C::kTileN + static_cast<int>(rank) * (TN / 2);
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long w0 = prof ? clock64() : 0;
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
            report_status(p.status, kDevTimeoutProducer);
            ok = false;
            break;
          }
          if (prof) waited += clock64() - w0;
          const uint32_t bar = leader_full0 + 8u * s;
          const uint32_t dst_a = ring_base + s * C::kStageBytes;
          // Only the leader arms its barrier (for both CTAs' bytes); the peer's copies credit the
          // same barrier and may land before or after the arming, which mbarrier tolerates.
          if (elect_one()) {
            if (rank == 0) mbar_arrive_expect_tx(full_bar(s), 2 * C::kStageBytes);
            if (p.l2_a != 0) tma_load_2d_pair_hint(dst_a, &tmap_a, bar, kb * kBlockK, row_a, pol_a);
            else tma_load_2d_pair(dst_a, &tmap_a, bar, kb * kBlockK, row_a);
#pragma unroll
            for (int h = 0; h < NB; ++h) {
              if (p.l2_b != 0)
                tma_load_2d_pair_hint(dst_a + kABytes + h * C::kBBytes, &tmap_b, bar, kb * kBlockK,
                                      row_b + h * TN, pol_b);
              else
                tma_load_2d_pair(dst_a + kABytes + h * C::kBBytes, &tmap_b, bar, kb * kBlockK,
                                 row_b + h * TN);
            }
          }
          __syncwarp();
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {
        // Give copies already in flight time to land before this CTA's shared memory goes away.
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
      if (prof && lane == 0) {
        p.prof[blockIdx.x * kProfCount + kProfLoadWait] = waited;
        p.prof[blockIdx.x * kProfCount + kProfLoadTotal] = clock64() - t_begin;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issue (leader CTA only)
    if (rank == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, TN);
      int s = 0;
      uint32_t ph = 0;
      int local = 0;
      bool ok = true;
      const bool prof = p.prof != nullptr;
      long long wait_full = 0, wait_acc = 0;
      const long long t_begin = prof ? clock64() : 0;
      TileCursor cursor;
      cursor.init(p.dynamic != 0, n_clusters, num_tiles, sched);
      for (int t = cluster; t >= 0 && ok; t = cursor.next(t, lane == 0, true), ++local) {
        // NB = 1: slot = bank (local & 1), used every second tile.  NB = 2: slots 0 and 1 are the
        // two halves of every tile.
        const int bank = (NB == 1) ? (local & 1) : 0;
        const uint32_t use_parity =
            static_cast<uint32_t>((NB == 1) ? (local >> 1) : local) & 1u;
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          const long long w0 = prof ? clock64() : 0;
          if (!mbar_wait(full_bar(s), ph)) {
            report_status(p.status, kDevTimeoutMmaFull);
            ok = false;
            break;
          }
          if (prof) wait_full += clock64() - w0;
          tc_fence_after_sync();
          const uint32_t a_addr = ring_base + s * C::kStageBytes;
          const uint64_t desc_a = make_smem_desc(a_addr, 1024, 16, kSwizzle128B);
#pragma unroll
          for (int h = 0; h < NB; ++h) {
            const int slot = (NB == 1) ? bank : h;
            if (kb == 0) {
              // The epilogue must have drained this slot (previous user) before it is overwritten.
              const long long a0 = prof ? clock64() : 0;
              if (!mbar_wait(acc_empty_bar(slot), use_parity ^ 1u)) {
                report_status(p.status, kDevTimeoutMmaAcc);
                ok = false;
                break;
              }
              if (prof) wait_acc += clock64() - a0;
              tc_fence_after_sync();
            }
            const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(slot * TN);
            const uint64_t desc_b =
                make_smem_desc(a_addr + kABytes + h * C::kBBytes, 1024, 16, kSwizzle128B);
            if (elect_one()) {
#pragma unroll
              for (int k = 0; k < kBlockK / 16; ++k) {
                // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row.
                mma_bf16_ss<2>(tmem_d, desc_a + 2u * k, desc_b + 2u * k, idesc,
                               (kb > 0 || k > 0) ? 1u : 0u);
              }
            }
            __syncwarp();
          }
          if (!ok) break;
          if (elect_one()) mma_commit_pair(empty_bar(s), 0x3);
          __syncwarp();
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        if (ok && elect_one()) mma_commit_pair(acc_full_bar(bank), 0x3);
        __syncwarp();
      }
      if (prof && lane == 0) {
        p.prof[blockIdx.x * kProfCount + kProfMmaWaitFull] = wait_full;
        p.prof[blockIdx.x * kProfCount + kProfMmaWaitAcc] = wait_acc;
        p.prof[blockIdx.x * kProfCount + kProfMmaTotal] = clock64() - t_begin;
        p.prof[blockIdx.x * kProfCount + kProfTiles] = local;
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------- tile scheduler (leader CTA)
    if (p.dynamic != 0 && rank == 0 && lane == 0) clc_scheduler_loop(sched, p.status);
  } else {
    // ------------------------------------------------------------- epilogue (8 warps)
    const int quarter = warp & 3;           // TMEM lane quarter this warp may read
    const int group = (warp - 2) >> 2;      // 0: warps 2-5, 1: warps 6-9
    const bool active = (NB == 2) || (group < C::kGroupsPerSlot);
    if (active) {
      const uint32_t leader_acc_empty0 = mapa_u32(acc_empty_bar(0), 0);
      const uint32_t sbuf = store_base + (warp - 2) * kStoreBufBytes;
      StoreTarget out;
      out.tmap_d = &tmap_d;
      out.d_ptr = p.d_ptr;
      out.ldd = p.ldd;
      out.M = p.M;
      out.N = kSwiglu ? p.N / 2 : p.N;
      out.peers = &p.peers;
      out.alpha = 1.0f;
      out.row_end = p.M;
      int local = 0;
      bool ok = true;
      if (p.operands_static == 1) griddep_wait();   // 2: D is independent too, no wait at all
      const bool prof = p.prof != nullptr && warp == 2 && lane == 0;
      long long waited = 0;
      const long long t_begin = prof ? clock64() : 0;
      TileCursor cursor;
      cursor.init(p.dynamic != 0, n_clusters, num_tiles, sched);
      for (int t = cluster; t >= 0 && ok; t = cursor.next(t, lane == 0, true), ++local) {
        int tm, tn;
        tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, tm, tn);
        tm = (tm + p.m_rotate) % p.tiles_m;   // routed stores: ranks start at different row blocks
        const int bank = (NB == 1) ? (local & 1) : 0;
        const int slot = (NB == 1) ? bank : group;
        const uint32_t use_parity =
            static_cast<uint32_t>((NB == 1) ? (local >> 1) : local) & 1u;
        const long long w0 = prof ? clock64() : 0;
        if (!mbar_wait(acc_full_bar(bank), use_parity)) {
          if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
          ok = false;
          break;
        }
        if (prof) waited += clock64() - w0;
        tc_fence_after_sync();
        const int row0 = (p.tile_row0 != nullptr ? __ldg(p.tile_row0 + tm) : tm * 256) +
                         static_cast<int>(rank) * kBlockM + quarter * 32;
        out.row_end = p.tile_row_end != nullptr ? __ldg(p.tile_row_end + tm) : p.M;
        // First column (in the tile and in tensor memory) this warp is responsible for.
        const int tile_col = (NB == 1) ? group * C::kColsPerWarp : group * TN;
        const int col0 = tn * C::kTileN + tile_col;
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               static_cast<uint32_t>((NB == 1) ? bank * TN + tile_col : tile_col);
        // Pull this warp's share of the slot out of tensor memory, hand the slot back to the MMA
        // role, then store.  With 256 x 512 tiles the main loop of the next tile cannot start
        // until the slot is handed back, so no store sits in front of that.
        drain_and_store<C::kColsPerWarp, kTmaStore, kSwiglu>(taddr, sbuf, out, row0, col0,
                                                              leader_acc_empty0 + 8u * slot, lane);
      }
      drain_store_groups<kTmaStore>(lane);
      if (prof) {
        p.prof[blockIdx.x * kProfCount + kProfEpiWait] = waited;
        p.prof[blockIdx.x * kProfCount + kProfEpiTotal] = clock64() - t_begin;
      }
    }
  }
  __syncwarp();

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc<2>(tmem_base, C::kTmemCols);
  }
}

}  // namespace bf16k

// -----------------------------------------------------------------------------------
// Host side
// -----------------------------------------------------------------------------------
namespace {

template <int TN, int NB, int kStore, int R = 1>
int launch_bf16(const Bf16Launch& L, cudaStream_t stream) {
  using C = bf16k::Cfg<TN, NB, R>;
  auto kernel = bf16k::gemm_bf16_kernel<TN, NB, kStore, R>;
  static thread_local int configured_device = -1;
  static thread_local int max_clusters = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_error(SMB_ERR_CUDA, "cudaGetDevice failed");
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kTotal);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaFuncSetAttribute(bf16 smem)");
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2, 1, 1);
    probe.blockDim = dim3(bf16k::kThreads, 1, 1);
    probe.dynamicSmemBytes = C::kTotal;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    probe.attrs = &attr;
    probe.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kernel, &probe);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaOccupancyMaxActiveClusters(bf16)");
    if (n <= 0) return set_error(SMB_ERR_CUDA, "no 2-CTA cluster of the bf16 kernel fits on this device");
    max_clusters = n;
    configured_device = dev;
  }
  bf16k::Params p;
  p.M = L.M;
  p.N = L.N;
  p.K = L.K;
  p.tiles_m = L.tile_row0 != nullptr ? L.tile_rows : (L.M + 255) / 256;
  p.tiles_n = (L.N + C::kTileN - 1) / C::kTileN;
  p.tile_row0 = L.tile_row0;
  p.tile_row_end = L.tile_row_end;
  p.group_m = L.group_m > 0 ? L.group_m
                            : raster_group_rows(p.tiles_m, static_cast<long long>(L.K) * 2,
                                                static_cast<long long>(L.N) * L.K * 2);
  p.ldd = L.ldd;
  p.d_ptr = static_cast<uint16_t*>(L.d);
  p.status = L.status;
  p.prof = L.prof;
  p.operands_static = L.operands_static ? (L.output_independent ? 2 : 1) : 0;
  p.peers = L.peers;
  p.m_rotate = L.peers.route_rows > 0 ? (L.peers.first_block * (L.peers.route_rows / 256)) % p.tiles_m : 0;
  p.mtile_group = L.mtile_group;
  p.l2_a = L.l2_a;
  p.l2_b = L.l2_b;
  const long long tiles = static_cast<long long>(p.tiles_m) * p.tiles_n;
  int clusters = static_cast<int>(tiles < max_clusters ? tiles : max_clusters);
  if (L.max_clusters > 0 && clusters > L.max_clusters) clusters = L.max_clusters;
  // Hardware work queue: one cluster per tile is launched; those that get to run take over the
  // tiles of those that have not started.  Pointless when every tile has a cluster anyway.
  p.dynamic = (L.dynamic && tiles > clusters && L.max_clusters == 0) ? 1 : 0;
  if (p.dynamic) {
    if (tiles > (1LL << 30)) return set_error(SMB_ERR_UNSUPPORTED, "bf16: too many tiles for one grid");
    clusters = static_cast<int>(tiles);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(bf16k::kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute pdl;
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L.tmap_a, L.tmap_b, L.tmap_d, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "bf16 GEMM launch");
  return SMB_OK;
}

template <int TN, int NB>
int launch_bf16_store(const Bf16Launch& L, cudaStream_t stream) {
  if (L.swiglu) {
    if constexpr (TN == 256) {
      return launch_bf16<TN, NB, bf16k::kStoreSwiglu>(L, stream);
    } else {
      return set_error(SMB_ERR_UNSUPPORTED, "bf16: the gated epilogue needs 256-wide tiles");
    }
  }
  if constexpr (TN <= 128) {
    // Narrow tiles: two CTAs per SM when consecutive launches may overlap (see Cfg).
    if (L.operands_static) {
      return L.tma_store ? launch_bf16<TN, NB, bf16k::kStoreTma, 2>(L, stream)
                         : launch_bf16<TN, NB, bf16k::kStorePlain, 2>(L, stream);
    }
  }
  return L.tma_store ? launch_bf16<TN, NB, bf16k::kStoreTma>(L, stream)
                     : launch_bf16<TN, NB, bf16k::kStorePlain>(L, stream);
}

}  // namespace

void bf16_pick_tile(int M, int N, int K, int clusters, int* tile_n, int* sub_blocks) {
  *sub_blocks = 1;
  if (N <= 64) {
    *tile_n = 64;
    return;
  }
  if (N <= 128) {
    *tile_n = 128;
    return;
  }
  *tile_n = 256;
  if (N <= 256) return;
  // 256 x 512 tiles against 256 x 256 tiles.  Both keep the tensor pipe busy ~99 % of the
  // cycles; the wide tile moves a quarter less data per flop through L2 and shared memory, which
  // under the power cap is worth ~6 % of clock, but it has half as many tiles to spread over
  // the clusters and exposes ~2500 cycles of accumulator drain per tile.  Estimated cycles:
  if (clusters < 1) clusters = 74;
  const long long tiles_m = (M + 255) / 256;
  const long long kb = (K + 63) / 64;
  const long long waves1 = (tiles_m * ((N + 255) / 256) + clusters - 1) / clusters;
  const long long waves2 = (tiles_m * ((N + 511) / 512) + clusters - 1) / clusters;
  const double cost1 = static_cast<double>(waves1) * (kb * 512.0);
  const double cost2 = static_cast<double>(waves2) * (kb * 1024.0 + 2500.0) / 1.06;
  if (cost2 < cost1) *sub_blocks = 2;
}

int bf16_launch(const Bf16Launch& L, cudaStream_t stream) {
  if (L.sub_blocks == 2 && L.tile_n == 256) return launch_bf16_store<256, 2>(L, stream);
  if (L.sub_blocks != 1) return set_error(SMB_ERR_INVALID, "bf16: two sub-blocks need 256-wide tiles");
  switch (L.tile_n) {
    case 256: return launch_bf16_store<256, 1>(L, stream);
    case 128: return launch_bf16_store<128, 1>(L, stream);
    case 64: return launch_bf16_store<64, 1>(L, stream);
    default: return set_error(SMB_ERR_INVALID, "bf16 tile width must be 64, 128 or 256");
  }
}

}  // namespace smb
