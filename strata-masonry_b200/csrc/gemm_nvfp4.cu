// Dense block-scaled FP4 GEMM for sm_100a:
//   D[M,N] = bf16( sum_k (A[m,k] * SFA[m,k/32]) * (B[n,k] * SFB[n,k/32]) ),  FP32 accumulate,
// A and B are E2M1 codes, two per byte (even k in the low nibble), SFA/SFB are UE8M0 bytes in
// the packed layout of smb_sf_packed_bytes().
//
// From-scratch counterpart of the reference kernel dense_gemm_nvfp4_k1_impl
// (src/kernels/gemm/sm100a/nvfp4/dense_gemm_nvfp4.cu:1705-2250) and of its local load / MMA /
// epilogue bodies (:448-852, :970-1333, :1343-1674).  Same numerics (kind::mxf4nvf4,
// scale_vec::2X, UE8M0) and the same scale path (TMA -> shared memory -> tcgen05.cp -> tensor
// memory, two K=64 instructions sharing one 4-byte scale cell through the scale-id field).
// Differences by design: run-time M, N, K with edge predication; no multicast loads (each CTA
// fetches its own copy of the B scales); tile widths up to 384 columns with a single
// accumulator set, because at FP4 rates the L2 sector rate bounds narrower tiles; bounded waits.
//
// One cluster = 2 CTAs = one 256 x (W0 + W1) output tile, built from one or two N sub-blocks of
// width 128 or 256.  Per 256-wide K block (= 128 bytes per row) CTA r loads
//   A rows [m0 + 128 r, +128)                             16 KiB
//   for sub-block h: B rows [n_h + W_h/2 r, +W_h/2)       W_h/2 x 128 B
//   SFA for its own 128 rows                              1 KiB  (two 512-byte cells, K 0-127 / 128-255)
//   SFB for ALL columns of the tile                       (W0 + W1)/128 KiB  (every CTA multiplies
//                                                         its 128 rows with every column)
// Tensor memory: accumulators first (two banks of 128 columns when the tile is 128 wide, else one
// set of W0 + W1 columns), then a ring of scale slots, one per pipeline stage:
//   [SFA cell 0 (4 cols) | SFA cell 1 | SFB sub-block 0: cell 0 (W0/32 cols) | cell 1 | SFB sub-block 1 ...]
#include "epilogue.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"
#include "sched.cuh"

namespace smb {

namespace fp4k {

constexpr int kBlockM = 128;          // rows of A per CTA
constexpr int kBlockKBytes = 128;     // bytes of K per row per stage (= 256 E2M1 values)
constexpr int kBlockK = 256;
constexpr int kThreads = 384;
constexpr int kEpiWarps = 8;
constexpr int kABytes = kBlockM * kBlockKBytes;   // 16 KiB
constexpr int kSfCellBytes = 512;     // 128 rows x 4 scale bytes (K = 128)
enum { kStorePlain = 0, kStoreTma = 1, kStoreSwiglu = 2 };   // epilogue variants

// V4: NVFP4 proper, one UE4M3 scale per 16 K (scale_vec::4X): a 4-byte scale cell per K=64
// instruction, four cells per stage instead of two (the layout the reference sketches but does
// not build, nvfp4/dense_gemm_nvfp4.cu:109-129).
// R = CTAs of the kernel that fit on one SM.  R = 2 exists for the 128-wide tile (N <= 128
// problems, bound by the L2 -> SM path): half the shared memory (3 stages), 256 tensor-memory
// columns with a single accumulator bank, at most 80 registers, so that two clusters share an SM
// pair and one's prologue, drain and exit overlap the other's main loop.  Used when consecutive
// launches may overlap (as for the BF16 kernel's narrow tiles); a launch that runs alone keeps
// R = 1 and its two accumulator banks.
template <int W0, int W1, bool V4 = false, int R = 1>
struct Cfg {
  static_assert(W0 == 128 || W0 == 256, "first sub-block width");
  static_assert(W1 == 0 || W1 == 128 || W1 == 256, "second sub-block width");
  static_assert(R == 1 || (R == 2 && W0 == 128 && W1 == 0 && !V4), "two resident CTAs: 128-wide tile only");
  static constexpr int kResident = R;
  static constexpr int kTmemCols = (R == 2) ? 256 : 512;
  static constexpr int kRingBudget = (R == 2) ? 78 * 1024 : 192 * 1024;
  static constexpr int kSubs = (W1 == 0) ? 1 : 2;
  static constexpr int kTileN = W0 + W1;
  static constexpr bool kTwoBanks = (kTileN == 128) && R == 1;    // epilogue overlaps next main loop
  static constexpr int kB0Bytes = (W0 / 2) * kBlockKBytes;
  static constexpr int kB1Bytes = (W1 / 2) * kBlockKBytes;
  static constexpr int kCells = V4 ? 4 : 2;                       // 4-byte scale cells per row and stage
  static constexpr int kSfaBytes = kCells * kSfCellBytes;         // this CTA's 128 rows, K = 256
  static constexpr int kSfbBytes = (kTileN / 128) * kCells * kSfCellBytes;
  static constexpr int kStageBytes = kABytes + kB0Bytes + kB1Bytes + kSfaBytes + kSfbBytes;
  static constexpr int kOffB0 = kABytes;
  static constexpr int kOffB1 = kOffB0 + kB0Bytes;
  static constexpr int kOffSfa = kOffB1 + kB1Bytes;
  static constexpr int kOffSfb = kOffSfa + kSfaBytes;
  // Tensor memory map.
  static constexpr int kAccCols = kTwoBanks ? 256 : kTileN;
  static constexpr int kSfaCols = kCells * 4;                      // cells x 4 columns
  static constexpr int kSfbCols = (kTileN / 128) * kCells * 4;
  static constexpr int kSlotCols = kSfaCols + kSfbCols;
  static constexpr int kMaxSlots = (kTmemCols - kAccCols) / kSlotCols;
  static constexpr int kStagesBySmem = kRingBudget / kStageBytes;
  static constexpr int kStages = kStagesBySmem < kMaxSlots ? kStagesBySmem : kMaxSlots;
  static constexpr int kRingBytes = kStages * kStageBytes;
  static constexpr int kStoreBytes = kEpiWarps * kStoreBufBytes;
  static constexpr int kTotal = 1024 + kRingBytes + kStoreBytes + 1024;
  static constexpr int kColsPerWarp = kTileN / 2;                  // two epilogue warp groups
  static_assert(kStageBytes % 1024 == 0, "stage bases must stay 1024-byte aligned");
  static_assert(kColsPerWarp % kStoreCols == 0, "epilogue split");
  static_assert(kAccCols + kStages * kSlotCols <= kTmemCols, "tensor memory budget");
  static_assert(kTotal <= (R == 2 ? 115712 : 232448), "shared memory budget");
  static_assert(kStages >= 2, "ring depth");
};

struct Params {
  int M, N, K;
  int tiles_m, tiles_n;
  // Tiles are handed out in two phases: first `tiles_n` full-width tiles per tile row over the
  // columns [0, tiles_n * kTileN), then `narrow_tiles_n` tiles of the first sub-block's width (W0)
  // over [narrow_col0, N).  With equal tiles the last wave leaves clusters idle (8192^3 with
  // 256 x 384 tiles: 10 tile times per cluster where 9.5 would be balanced); a few narrower tiles
  // at the end of the list even the clusters out.  narrow_tiles_n = 0: one phase, as before.
  int narrow_tiles_n, narrow_col0;
  int group_m;
  int ldd;
  uint16_t* d_ptr;
  int* status;
  long long* prof;
  int prefetch;   // L2 prefetch distance in K blocks (0 = off)
  int dynamic;    // 1: tiles come from the hardware work queue (one cluster launched per tile)
  PeerCopies peers;     // extra destinations of every stored box (count 0: none)
  int m_rotate;         // the tile walk starts at this 256-row tile (0 unless rows are routed)
  const int* mtile_group;  // grouped GEMM: group of every 256-row tile of A (device), or null
  const int* tile_row0;    // ragged groups (multiples of 128 rows): first row of every row tile (device), or null
  const int* tile_row_end; // ... and the row where the tile's group ends
  float alpha;          // factor on every accumulator (block-16 variant: 1 / (global scale A x B))
  int operands_static;  // 1: operands and scales are not written by the previous kernel on the stream
  int l2_a, l2_b;       // L2 eviction hint of the A / B loads: 0 none, 1 evict-last, 2 evict-first
};

enum { kProfLoadWait = 0, kProfLoadTotal, kProfMmaWaitFull, kProfMmaWaitAcc, kProfMmaTotal,
       kProfEpiWait, kProfEpiTotal, kProfTiles, kProfCount };

// Tile index -> tile row, first column, and whether the tile has its second sub-block.  Tiles
// are walked in groups of `group_m` tile rows (as in tile_coords); inside a group first the
// full-width tiles, M fastest, then the group's narrow tiles: the rows of A a narrow tile needs
// are the ones its group has just used, still in L2.  (Narrow tiles of ALL rows at the very end of
// the list measured 2 % slower on 30720 x 2048 x 4096: every one of them fetched its A panel from
// DRAM again.)
template <int kTileN, int W0>
__host__ __device__ inline void fp4_tile(int t, int tiles_m, int tiles_n, int narrow_tiles_n, int narrow_col0,
                                         int group_m, int& tm, int& col0, bool& full_width) {
  const int per_row = tiles_n + narrow_tiles_n;
  const int per_group = group_m * per_row;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int rows = (tiles_m - first_m) < group_m ? (tiles_m - first_m) : group_m;
  int r = t - g * per_group;
  const int wide = rows * tiles_n;
  if (r < wide) {
    tm = first_m + r % rows;
    col0 = (r / rows) * kTileN;
    full_width = true;
  } else {
    r -= wide;
    tm = first_m + r % rows;
    col0 = narrow_col0 + (r / rows) * W0;
    full_width = false;
  }
}

template <int W0, int W1, int kStore, bool V4 = false, int R = 1>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, R)
gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap tmap_a,
                  const __grid_constant__ CUtensorMap tmap_b0,
                  const __grid_constant__ CUtensorMap tmap_b1,
                  const __grid_constant__ CUtensorMap tmap_sfa,
                  const __grid_constant__ CUtensorMap tmap_sfb,
                  const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ Params p) {
  using C = Cfg<W0, W1, V4, R>;
  constexpr int kCells = C::kCells;
  constexpr bool kTmaStore = (kStore != kStorePlain);
  constexpr bool kSwiglu = (kStore == kStoreSwiglu);   // D is [M, N/2]: silu(gate) * up
  static_assert(!kSwiglu || C::kSubs == 2 || C::kColsPerWarp % 128 == 0, "gated epilogue: 64 output columns per box");
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t ring_base = smem_base;
  const uint32_t store_base = ring_base + C::kRingBytes;
  const uint32_t bar_base = store_base + C::kStoreBytes;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (2 * kStages + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (2 * kStages + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * kStages + 4);
  auto sf_ready_bar = [&](int s) { return bar_base + 8u * (2 * kStages + 6 + s); };
  auto sf_full_bar = [&](int s) { return bar_base + 8u * (3 * kStages + 6 + s); };
  SchedSmem sched;
  sched.response = bar_base + 768u;
  sched.slot_full = bar_base + 784u;
  sched.slot_empty = bar_base + 792u;
  // Consumers of a scheduler response: both load threads, MMA thread, scale thread, 16 epilogue warps.
  constexpr int kSchedConsumers = 2 + 1 + 1 + 2 * kEpiWarps;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster = static_cast<int>(cluster_id_x());
  const int n_clusters = static_cast<int>(num_clusters_x());
  const int num_tiles = p.tiles_m * (p.tiles_n + p.narrow_tiles_n);
  const int num_kb = (p.K + kBlockK - 1) / kBlockK;

  // Programmatic dependent launch: the next kernel on the stream may begin its prologue while
  // this grid is still running (it waits, below, before it loads or stores anything).
  griddep_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(sf_ready_bar(s), 1);
      mbar_init(sf_full_bar(s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 2 * kEpiWarps);   // all epilogue warps of both CTAs
    }
    mbar_init(sched.slot_full, 1);
    mbar_init(sched.slot_empty, kSchedConsumers);
    fence_mbar_init_cluster();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b0);
    if (C::kSubs == 2) tma_prefetch_desc(&tmap_b1);
    tma_prefetch_desc(&tmap_sfa);
    tma_prefetch_desc(&tmap_sfb);
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
    // which is what the TMA and tcgen05 instructions take.
    {
      const uint32_t leader_full0 = mapa_u32(full_bar(0), 0);
      const uint32_t leader_sf_full0 = mapa_u32(sf_full_bar(0), 0);
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
        int tm, col0;
        bool full_width;
        fp4_tile<C::kTileN, W0>(t, p.tiles_m, p.tiles_n, p.narrow_tiles_n, p.narrow_col0, p.group_m, tm, col0,
                                full_width);
        tm = (tm + p.m_rotate) % p.tiles_m;   // routed stores: ranks start at different row blocks
        const int row_a = (p.tile_row0 != nullptr ? __ldg(p.tile_row0 + tm) : tm * 256) + static_cast<int>(rank) * kBlockM;
        const int band_a = row_a / 128;                         // 128-row band of SFA
        // Grouped GEMM: B and its scales are stacked [groups * N, ...] (N % 128 == 0); this tile of
        // A belongs to one group and meets that group's N rows.
        const int group_row = p.mtile_group != nullptr ? __ldg(p.mtile_group + tm) * p.N : 0;
        const int band_b = (group_row + col0) / 128;            // first 128-row band of SFB
        // No second sub-block in a narrow tile, nor where it would lie beyond the right edge of D.
        const bool has_sub1 = (C::kSubs == 2) && full_width && (col0 + W0 < p.N);
        for (int kb = 0; kb < num_kb; ++kb) {
          const long long w0 = prof ? clock64() : 0;
          if (!mbar_wait(empty_bar(s), ph ^ 1u)) {
            report_status(p.status, kDevTimeoutProducer);
            ok = false;
            break;
          }
          if (prof) waited += clock64() - w0;
          const uint32_t bar = leader_full0 + 8u * s;
          const uint32_t sf_bar = leader_sf_full0 + 8u * s;
          const uint32_t dst = ring_base + s * C::kStageBytes;
          constexpr int kSfBytes = C::kSfaBytes + C::kSfbBytes;
          if (elect_one()) {
          if (rank == 0) {
            mbar_arrive_expect_tx(sf_full_bar(s), 2 * kSfBytes);
            mbar_arrive_expect_tx(full_bar(s),
                                  2 * (C::kStageBytes - kSfBytes - (has_sub1 ? 0 : C::kB1Bytes)));
          }
          // Scales first and on their own barrier: the scale warp can move them into tensor
          // memory while the (ten times larger) operand boxes are still in flight.  The packed
          // scale buffer is viewed as [bands, K/128 * 64] 64-bit words; one stage covers 128
          // words (two 512-byte cells) of each band.
          tma_load_2d_pair(dst + C::kOffSfa, &tmap_sfa, sf_bar, kb * (kCells * 64), band_a);
          tma_load_2d_pair(dst + C::kOffSfb, &tmap_sfb, sf_bar, kb * (kCells * 64), band_b);
          if (p.l2_a != 0) tma_load_2d_pair_hint(dst, &tmap_a, bar, kb * kBlockKBytes, row_a, pol_a);
          else tma_load_2d_pair(dst, &tmap_a, bar, kb * kBlockKBytes, row_a);
          const int row_b0 = group_row + col0 + static_cast<int>(rank) * (W0 / 2);
          if (p.l2_b != 0) tma_load_2d_pair_hint(dst + C::kOffB0, &tmap_b0, bar, kb * kBlockKBytes, row_b0, pol_b);
          else tma_load_2d_pair(dst + C::kOffB0, &tmap_b0, bar, kb * kBlockKBytes, row_b0);
          if (C::kSubs == 2 && has_sub1) {
            const int row_b1 = group_row + col0 + W0 + static_cast<int>(rank) * (W1 / 2);
            if (p.l2_b != 0) tma_load_2d_pair_hint(dst + C::kOffB1, &tmap_b1, bar, kb * kBlockKBytes, row_b1, pol_b);
            else tma_load_2d_pair(dst + C::kOffB1, &tmap_b1, bar, kb * kBlockKBytes, row_b1);
          }
          if (p.prefetch > 0 && kb + p.prefetch < num_kb) {
            const int kp = (kb + p.prefetch) * kBlockKBytes;
            tma_prefetch_l2_2d(&tmap_a, kp, row_a);
            tma_prefetch_l2_2d(&tmap_b0, kp, group_row + col0 + static_cast<int>(rank) * (W0 / 2));
            if (C::kSubs == 2 && has_sub1)
              tma_prefetch_l2_2d(&tmap_b1, kp, group_row + col0 + W0 + static_cast<int>(rank) * (W1 / 2));
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
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issue (leader CTA only)
    if (rank == 0) {
      int s = 0;
      uint32_t ph = 0;
      int local = 0;
      int sub1_tiles = 0;   // tiles so far that had a second sub-block (its barriers' phase count)
      bool ok = true;
      const bool prof = p.prof != nullptr;
      long long wait_full = 0, wait_acc = 0;
      const long long t_begin = prof ? clock64() : 0;
      TileCursor cursor;
      cursor.init(p.dynamic != 0, n_clusters, num_tiles, sched);
      for (int t = cluster; t >= 0 && ok; t = cursor.next(t, lane == 0, true), ++local) {
        int tm, col0;
        bool full_width;
        fp4_tile<C::kTileN, W0>(t, p.tiles_m, p.tiles_n, p.narrow_tiles_n, p.narrow_col0, p.group_m, tm, col0,
                                full_width);
        const bool has_sub1 = (C::kSubs == 2) && full_width && (col0 + W0 < p.N);
        const int bank = C::kTwoBanks ? (local & 1) : 0;
        const uint32_t use_parity =
            static_cast<uint32_t>(C::kTwoBanks ? (local >> 1) : local) & 1u;
        if constexpr (C::kSubs == 1) {
          const long long a0 = prof ? clock64() : 0;
          if (!mbar_wait(acc_empty_bar(bank), use_parity ^ 1u)) {
            report_status(p.status, kDevTimeoutMmaAcc);
            ok = false;
            break;
          }
          if (prof) wait_acc += clock64() - a0;
          tc_fence_after_sync();
        }
        const uint32_t acc_base = tmem_base + static_cast<uint32_t>(bank * 128);
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          // Operands in shared memory (full) and scales in tensor memory (sf_ready, committed by
          // the scale warp).
          const long long w0 = prof ? clock64() : 0;
          if (!mbar_wait(full_bar(s), ph) || !mbar_wait(sf_ready_bar(s), ph)) {
            report_status(p.status, kDevTimeoutMmaFull);
            ok = false;
            break;
          }
          if (prof) wait_full += clock64() - w0;
          tc_fence_after_sync();
          const uint32_t stage = ring_base + s * C::kStageBytes;
          const uint32_t sf_t = tmem_base + static_cast<uint32_t>(C::kAccCols + s * C::kSlotCols);
          const uint64_t desc_a = make_smem_desc(stage, 1024, 16, kSwizzle128B);
          // One K = 64 instruction of sub-block h.  K = 64 per instruction = 32 bytes along the
          // swizzled row.  Atoms 2c and 2c + 1 share scale cell c: the first reads bytes 0-1 of
          // each cell (scale id 0), the second bytes 2-3 (scale id 2).
          auto issue = [&](int h, int ki) {
            const uint32_t sf_id = V4 ? 0u : ((ki & 1) ? 2u : 0u);
            const uint32_t cell = static_cast<uint32_t>(V4 ? ki : (ki >> 1));
            const int width = (h == 0) ? W0 : W1;
            const int bands = width / 128;
            const uint32_t sfb_col = C::kSfaCols + (h == 0 ? 0u : static_cast<uint32_t>((W0 / 128) * kCells * 4));
            const uint32_t acc_col = (h == 0) ? 0u : static_cast<uint32_t>(W0);
            const uint64_t desc_b = make_smem_desc(stage + (h == 0 ? C::kOffB0 : C::kOffB1), 1024, 16, kSwizzle128B);
            const uint32_t idesc = make_idesc_mxf4(256, width, sf_id, sf_id, !V4);
            const uint32_t sfa_t = sf_t + 4u * cell;
            const uint32_t sfb_t = sf_t + sfb_col + cell * static_cast<uint32_t>(bands * 4);
            const uint32_t accum = (kb > 0 || ki > 0) ? 1u : 0u;
            if (V4) mma_nvf4_ss<2>(acc_base + acc_col, desc_a + 2u * ki, desc_b + 2u * ki, idesc, sfa_t, sfb_t, accum);
            else mma_mxf4_ss<2>(acc_base + acc_col, desc_a + 2u * ki, desc_b + 2u * ki, idesc, sfa_t, sfb_t, accum);
          };
          if (C::kSubs == 2 && (kb == 0 || kb == num_kb - 1)) {
            // Two sub-blocks have a barrier pair each (a narrow tile uses only the first).  In the
            // tile's first and last K block the instructions go sub-block by sub-block: the first
            // K block multiplies into sub-block 0 as soon as the epilogue has read it out, while
            // sub-block 1 is still being read; the last hands sub-block 0 to the epilogue while
            // sub-block 1 still multiplies.
            const bool first = kb == 0, last = kb == num_kb - 1;
            for (int h = 0; h < 2 && ok; ++h) {
              if (h == 1 && !has_sub1) break;
              if (first) {
                const long long a0 = prof ? clock64() : 0;
                const uint32_t use = static_cast<uint32_t>(h == 0 ? local : sub1_tiles) & 1u;
                if (!mbar_wait(acc_empty_bar(h), use ^ 1u)) {
                  report_status(p.status, kDevTimeoutMmaAcc);
                  ok = false;
                  break;
                }
                if (prof) wait_acc += clock64() - a0;
                tc_fence_after_sync();
              }
              if (elect_one()) {
#pragma unroll
                for (int ki = 0; ki < 4; ++ki) issue(h, ki);
                if (last) mma_commit_pair(acc_full_bar(h), 0x3);
              }
              __syncwarp();
            }
            if (!ok) break;
            if (elect_one()) mma_commit_pair(empty_bar(s), 0x3);
          } else if (elect_one()) {
#pragma unroll
            for (int ki = 0; ki < 4; ++ki) {
#pragma unroll
              for (int h = 0; h < C::kSubs; ++h) {
                if (h == 0 || has_sub1) issue(h, ki);
              }
            }
            mma_commit_pair(empty_bar(s), 0x3);
          }
          __syncwarp();
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
        if (C::kSubs == 1) {
          if (ok && elect_one()) mma_commit_pair(acc_full_bar(bank), 0x3);
          __syncwarp();
        }
        if (has_sub1) ++sub1_tiles;
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
    // Scale cells go shared memory -> tensor memory with tcgen05.cp: one copy moves 32 lines of 16
    // bytes (= 128 rows x 4 scale bytes) into 4 columns, replicated into all four lane quarters.
    // SFB in shared memory is [band][cell][512 B]; in tensor memory, per sub-block,
    // [cell][band][4 columns], so that one instruction of width W reads W/32 adjacent columns.
    // The copies are issued from this warp, not from the MMA thread: issued in line with the MMAs
    // they cost the tensor pipe about 50 cycles each (measured: 256 x 256 tiles went from 3.6 to
    // 5.1 PFLOP/s when they moved here), from a second warp they overlap the MMAs.
    if (rank == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      TileCursor cursor;
      cursor.init(p.dynamic != 0, n_clusters, num_tiles, sched);
      for (int t = cluster; t >= 0 && ok; t = cursor.next(t, lane == 0, true)) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(sf_full_bar(s), ph)) {
            report_status(p.status, kDevTimeoutSched);
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t stage = ring_base + s * C::kStageBytes;
          const uint32_t sf_t = tmem_base + static_cast<uint32_t>(C::kAccCols + s * C::kSlotCols);
          const uint64_t sfa_desc = make_smem_desc(stage + C::kOffSfa, 128, 16, kSwizzleNone);
          const uint64_t sfb_desc = make_smem_desc(stage + C::kOffSfb, 128, 16, kSwizzleNone);
          if (elect_one()) {
#pragma unroll
          for (int cell = 0; cell < kCells; ++cell) {
            tmem_cp_32x128b_warpx4<2>(sf_t + 4u * cell, sfa_desc + cell * (kSfCellBytes / 16));
          }
          int band0 = 0;
          uint32_t col = C::kSfaCols;
#pragma unroll
          for (int h = 0; h < C::kSubs; ++h) {
            const int bands = (h == 0 ? W0 : W1) / 128;
#pragma unroll
            for (int cell = 0; cell < kCells; ++cell) {
#pragma unroll
              for (int b = 0; b < bands; ++b) {
                tmem_cp_32x128b_warpx4<2>(sf_t + col + static_cast<uint32_t>((cell * bands + b) * 4),
                                          sfb_desc + ((band0 + b) * kCells + cell) * (kSfCellBytes / 16));
              }
            }
            band0 += bands;
            col += static_cast<uint32_t>(bands * kCells * 4);
          }
          mma_commit_pair(sf_ready_bar(s), 0x1);
          }
          __syncwarp();
          if (++s == kStages) { s = 0; ph ^= 1u; }
        }
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------- tile scheduler (leader CTA)
    if (p.dynamic != 0 && rank == 0 && lane == 0) clc_scheduler_loop(sched, p.status);
  } else {
    // ------------------------------------------------------------- epilogue (8 warps)
    const int quarter = warp & 3;
    const int group = (warp - 2) >> 2;
    const uint32_t leader_acc_empty0 = mapa_u32(acc_empty_bar(0), 0);
    const uint32_t sbuf = store_base + (warp - 2) * kStoreBufBytes;
    StoreTarget out;
    out.tmap_d = &tmap_d;
    out.d_ptr = p.d_ptr;
    out.ldd = p.ldd;
    out.M = p.M;
    const int n_out = kSwiglu ? p.N / 2 : p.N;
    out.N = n_out;
    out.peers = &p.peers;
    out.alpha = p.alpha;
    out.row_end = p.M;
    int local = 0;
    int sub1_tiles = 0;   // tiles so far that had a second sub-block
    bool ok = true;
    if (p.operands_static == 1) griddep_wait();   // 2: D is independent too, no wait at all
    const bool prof = p.prof != nullptr && warp == 2 && lane == 0;
    long long waited = 0;
    const long long t_begin = prof ? clock64() : 0;
    TileCursor cursor;
    cursor.init(p.dynamic != 0, n_clusters, num_tiles, sched);
    for (int t = cluster; t >= 0 && ok; t = cursor.next(t, lane == 0, true), ++local) {
      int tm, tile_col0;
      bool full_width;
      fp4_tile<C::kTileN, W0>(t, p.tiles_m, p.tiles_n, p.narrow_tiles_n, p.narrow_col0, p.group_m, tm, tile_col0,
                              full_width);
      tm = (tm + p.m_rotate) % p.tiles_m;   // routed stores: ranks start at different row blocks
      // A narrow tile has no second sub-block: its accumulator columns beyond W0 hold nothing and
      // the columns of D there belong to the next tile.
      if (C::kSubs == 2) {
        const int limit = (tile_col0 + (full_width ? C::kTileN : W0)) / (kSwiglu ? 2 : 1);
        out.N = limit < n_out ? limit : n_out;
      }
      const int bank = C::kTwoBanks ? (local & 1) : 0;
      const uint32_t use_parity = static_cast<uint32_t>(C::kTwoBanks ? (local >> 1) : local) & 1u;
      const int row0 = (p.tile_row0 != nullptr ? __ldg(p.tile_row0 + tm) : tm * 256) +
                       static_cast<int>(rank) * kBlockM + quarter * 32;
      out.row_end = p.tile_row_end != nullptr ? __ldg(p.tile_row_end + tm) : p.M;
      const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      if constexpr (C::kSubs == 2) {
        // Both warp groups read their half of sub-block 0 and hand it back, then their share of
        // sub-block 1 (if the tile has one), and only then store.
        static_assert(W0 == 256 && W1 == 128, "two sub-blocks: the 256 + 128 tile");
        const bool has_sub1 = full_width && (tile_col0 + W0 < p.N);
        // Plain: group g takes 128 columns of sub-block 0 and 64 of sub-block 1.  Gated: four
        // accumulator columns make two outputs, so 128 columns fill one 64-column store box: group g
        // takes 128 columns of sub-block 0, group 0 all 128 of sub-block 1.
        constexpr int kOut0 = kSwiglu ? 64 : 128;
        constexpr int kCols1 = kSwiglu ? 128 : 64;
        constexpr int kOut1 = 64;
        uint32_t packed0[kOut0 / 2], packed1[kOut1 / 2];
        const bool reads_sub1 = !kSwiglu || group == 0;
        const long long w0 = prof ? clock64() : 0;
        if (!mbar_wait(acc_full_bar(0), static_cast<uint32_t>(local) & 1u)) {
          if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
          ok = false;
          break;
        }
        if (prof) waited += clock64() - w0;
        tc_fence_after_sync();
        drain_columns<128, kSwiglu, V4>(lane_base + static_cast<uint32_t>(group * 128), out.alpha, packed0);
        release_columns(leader_acc_empty0, lane);
        if (has_sub1) {
          const long long w1 = prof ? clock64() : 0;
          if (!mbar_wait(acc_full_bar(1), static_cast<uint32_t>(sub1_tiles) & 1u)) {
            if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
            ok = false;
            break;
          }
          if (prof) waited += clock64() - w1;
          tc_fence_after_sync();
          if (reads_sub1)
            drain_columns<kCols1, kSwiglu, V4>(lane_base + static_cast<uint32_t>(W0 + (kSwiglu ? 0 : group * 64)),
                                               out.alpha, packed1);
          release_columns(leader_acc_empty0 + 8u, lane);
          ++sub1_tiles;
        }
        const int out_col0 = (tile_col0 + group * 128) / (kSwiglu ? 2 : 1);
        const int out_col1 = kSwiglu ? (tile_col0 + W0) / 2 : tile_col0 + W0 + group * 64;
        store_columns<kOut0, kTmaStore>(packed0, sbuf, out, row0, out_col0, lane);
        if (has_sub1 && reads_sub1) store_columns<kOut1, kTmaStore>(packed1, sbuf, out, row0, out_col1, lane);
      } else {
        const long long w0 = prof ? clock64() : 0;
        if (!mbar_wait(acc_full_bar(bank), use_parity)) {
          if (lane == 0) report_status(p.status, kDevTimeoutEpilogue);
          ok = false;
          break;
        }
        if (prof) waited += clock64() - w0;
        tc_fence_after_sync();
        const int tile_col = group * C::kColsPerWarp;
        const int col0 = tile_col0 + tile_col;
        const uint32_t taddr = lane_base + static_cast<uint32_t>(bank * 128 + tile_col);
        drain_and_store<C::kColsPerWarp, kTmaStore, kSwiglu, V4>(taddr, sbuf, out, row0, col0,
                                                                  leader_acc_empty0 + 8u * bank, lane);
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
    tmem_dealloc<2>(tmem_base, C::kTmemCols);
  }
}

}  // namespace fp4k

// -----------------------------------------------------------------------------------
// Host side
// -----------------------------------------------------------------------------------
namespace {

template <int W0, int W1, int kStore, bool V4 = false, int R = 1>
int launch_fp4(const Fp4Launch& L, cudaStream_t stream) {
  using C = fp4k::Cfg<W0, W1, V4, R>;
  auto kernel = fp4k::gemm_nvfp4_kernel<W0, W1, kStore, V4, R>;
  static thread_local int configured_device = -1;
  static thread_local int max_clusters = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return set_error(SMB_ERR_CUDA, "cudaGetDevice failed");
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::kTotal);
    if (e != cudaSuccess) return set_cuda_error(e, "cudaFuncSetAttribute(nvfp4 smem)");
    cudaLaunchConfig_t probe = {};
    probe.gridDim = dim3(2, 1, 1);
    probe.blockDim = dim3(fp4k::kThreads, 1, 1);
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
    if (e != cudaSuccess) return set_cuda_error(e, "cudaOccupancyMaxActiveClusters(nvfp4)");
    if (n <= 0) return set_error(SMB_ERR_CUDA, "no 2-CTA cluster of the nvfp4 kernel fits on this device");
    max_clusters = n;
    configured_device = dev;
  }
  fp4k::Params p;
  p.M = L.M;
  p.N = L.N;
  p.K = L.K;
  p.tiles_m = L.tile_row0 != nullptr ? L.tile_rows : (L.M + 255) / 256;
  p.tiles_n = (L.N + C::kTileN - 1) / C::kTileN;
  p.tile_row0 = L.tile_row0;
  p.tile_row_end = L.tile_row_end;
  p.narrow_tiles_n = 0;
  p.narrow_col0 = 0;
  if (C::kSubs == 2 && !L.uniform_tiles) {
    int clusters_now = max_clusters;
    if (L.max_clusters > 0 && clusters_now > L.max_clusters) clusters_now = L.max_clusters;
    fp4_split_phases(L.M, L.N, L.K, W0, W1, clusters_now, &p.tiles_n, &p.narrow_tiles_n);
    p.narrow_col0 = p.tiles_n * C::kTileN;
  }
  p.group_m = L.group_m > 0 ? L.group_m : raster_group_rows_fp4(p.tiles_m, static_cast<long long>(L.K) / 2);
  p.ldd = L.ldd;
  p.d_ptr = static_cast<uint16_t*>(L.d);
  p.status = L.status;
  p.prof = L.prof;
  p.operands_static = L.operands_static ? (L.output_independent ? 2 : 1) : 0;
  p.peers = L.peers;
  p.m_rotate = L.peers.route_rows > 0 ? (L.peers.first_block * (L.peers.route_rows / 256)) % p.tiles_m : 0;
  p.mtile_group = L.mtile_group;
  p.alpha = L.alpha;
  p.prefetch = L.prefetch;
  p.l2_a = L.l2_a;
  p.l2_b = L.l2_b;
  const long long tiles = static_cast<long long>(p.tiles_m) * (p.tiles_n + p.narrow_tiles_n);
  int clusters = static_cast<int>(tiles < max_clusters ? tiles : max_clusters);
  if (L.max_clusters > 0 && clusters > L.max_clusters) clusters = L.max_clusters;
  p.dynamic = (L.dynamic && tiles > clusters && L.max_clusters == 0) ? 1 : 0;
  if (p.dynamic) {
    if (tiles > (1LL << 30)) return set_error(SMB_ERR_UNSUPPORTED, "nvfp4: too many tiles for one grid");
    clusters = static_cast<int>(tiles);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters, 1, 1);
  cfg.blockDim = dim3(fp4k::kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute pdl;
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &pdl;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, L.tmap_a, L.tmap_b0, L.tmap_b1, L.tmap_sfa,
                                     L.tmap_sfb, L.tmap_d, p);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "nvfp4 GEMM launch");
  return SMB_OK;
}

template <int W0, int W1>
int launch_fp4_store(const Fp4Launch& L, cudaStream_t stream) {
  if (L.block16) {
    if constexpr (W0 == 256 && W1 == 0) {
      if (L.swiglu) return set_error(SMB_ERR_UNSUPPORTED, "nvfp4: no gated epilogue for block-16 scales");
      return L.tma_store ? launch_fp4<W0, W1, fp4k::kStoreTma, true>(L, stream)
                         : launch_fp4<W0, W1, fp4k::kStorePlain, true>(L, stream);
    } else {
      return set_error(SMB_ERR_UNSUPPORTED, "nvfp4: block-16 scales need 256-wide tiles");
    }
  }
  if (L.swiglu) {
    if constexpr (W0 == 256) {
      return launch_fp4<W0, W1, fp4k::kStoreSwiglu>(L, stream);
    } else {
      return set_error(SMB_ERR_UNSUPPORTED, "nvfp4: the gated epilogue needs tiles of 256 or 384 columns");
    }
  }
  if constexpr (W0 == 128 && W1 == 0) {
    // Narrow tile: two CTAs per SM when consecutive launches may overlap (see Cfg).
    if (L.operands_static) {
      return L.tma_store ? launch_fp4<W0, W1, fp4k::kStoreTma, false, 2>(L, stream)
                         : launch_fp4<W0, W1, fp4k::kStorePlain, false, 2>(L, stream);
    }
  }
  return L.tma_store ? launch_fp4<W0, W1, fp4k::kStoreTma>(L, stream)
                     : launch_fp4<W0, W1, fp4k::kStorePlain>(L, stream);
}

}  // namespace

// How many full-width (w0 + w1) tiles per tile row, and how many w0-wide tiles after them, make
// the round-robin walk of `clusters` clusters over the tile list end soonest.  Cost of a tile in
// SM cycles, fitted to measurements (8192^3, 14080 x 5120 x 2048, 14080 x 2048 x 4096 at the
// ~1.57 GHz the kernels run at): a 256-wide K block costs 811 cycles on a 384-wide tile and 556
// on a 256-wide one (768 and 512 would be the tensor pipe's own time).  Between a tile's last
// instruction and the first of the next the 384-wide kernel (one accumulator set) idles for the
// tail of the tensor pipe, the accumulator drain and the barrier round trips: 1450 cycles after a
// full tile (two sub-blocks to read out), 1950 after a 256-wide one (fitted before and after the
// accumulator hand-over lost its cluster-scope release, which had cost 1750 and 1150 of the
// former 3200 and 3100).  The 256-wide kernel (two accumulator sets) fits 3100 per tile.
constexpr double kFp4CyclesPerColumnAndKBlock384 = 811.0 / 384.0;
constexpr double kFp4CyclesPerColumnAndKBlock256 = 556.0 / 256.0;
constexpr double kFp4TileOverhead384 = 1450.0, kFp4TileOverheadNarrowIn384 = 1950.0, kFp4TileOverhead256 = 3100.0;
namespace {
thread_local double g_last_phase_cost = 0.0;   // written by fp4_split_phases for fp4_pick_tile (same thread, same call)
}

void fp4_split_phases(int M, int N, int K, int w0, int w1, int clusters, int* wide_tiles_n, int* narrow_tiles_n) {
  const int tile_n = w0 + w1;
  const int tiles_m = (M + 255) / 256;
  const int max_wide = (N + tile_n - 1) / tile_n;
  *wide_tiles_n = max_wide;
  *narrow_tiles_n = 0;
  if (w1 == 0 || clusters < 1) return;
  const double kb = (K + 255) / 256;
  const double cost_wide = kb * kFp4CyclesPerColumnAndKBlock384 * tile_n + kFp4TileOverhead384;
  const double cost_narrow = kb * kFp4CyclesPerColumnAndKBlock256 * w0 + kFp4TileOverheadNarrowIn384;
  double best = -1.0;
  // Only the last few wide tiles of a row are worth trading: beyond that the narrow tiles'
  // extra drains and operand traffic outweigh any balance gained.
  const int lowest = max_wide - 8 > 0 ? max_wide - 8 : 0;
  for (int a = max_wide; a >= lowest; --a) {
    const long long rest = static_cast<long long>(N) - static_cast<long long>(a) * tile_n;
    const int b = rest > 0 ? static_cast<int>((rest + w0 - 1) / w0) : 0;
    // A last full-width tile that reaches beyond N by its whole second sub-block costs what a
    // narrow tile costs (that sub-block is neither loaded nor multiplied).
    const bool last_is_short = a > 0 && static_cast<long long>(a) * tile_n - N >= w1;
    const long long wide = static_cast<long long>(tiles_m) * (last_is_short ? a - 1 : a);
    const long long narrow = static_cast<long long>(tiles_m) * (last_is_short ? b + 1 : b);
    // The tiles are dealt to the clusters in turn; with the cheap tiles spread through the list
    // every cluster ends up with about its share of the work and at most one tile more.
    const double work = wide * cost_wide + narrow * cost_narrow;
    const double quantum = narrow > 0 ? cost_narrow : cost_wide;
    const double worst = work / clusters + 0.5 * quantum;
    if (best < 0.0 || worst < best * 0.998) {   // a change of plan must buy at least a fifth of a percent
      best = worst;
      *wide_tiles_n = a;
      *narrow_tiles_n = b;
    }
  }
  g_last_phase_cost = best;
}

}  // namespace smb

// Host-side views of the tile list, for known-answer tests (no device needed).
extern "C" void smb_debug_fp4_phases(int M, int N, int K, int clusters, int* wide_tiles_n, int* narrow_tiles_n) {
  smb::fp4_split_phases(M, N, K, 256, 128, clusters, wide_tiles_n, narrow_tiles_n);
}
extern "C" void smb_debug_fp4_tile(int t, int tiles_m, int wide_tiles_n, int narrow_tiles_n, int group_m, int* tm,
                                   int* col0, int* full_width) {
  bool full = false;
  smb::fp4k::fp4_tile<384, 256>(t, tiles_m, wide_tiles_n, narrow_tiles_n, wide_tiles_n * 384, group_m, *tm, *col0,
                                full);
  *full_width = full ? 1 : 0;
}

namespace smb {

void fp4_pick_tile(int M, int N, int K, int clusters, int* w0, int* w1) {
  *w1 = 0;
  if (N <= 128) {
    *w0 = 128;
    return;
  }
  *w0 = 256;
  if (N <= 256) return;
  // 256 x 384 against 256 x 256 tiles (one accumulator set each): the wider tile moves less data
  // per flop and pays the per-tile overhead less often, the narrower one spreads better over the
  // clusters.  Estimated cycles with the fitted costs above:
  if (clusters < 1) clusters = 74;
  const long long tiles_m = (M + 255) / 256;
  const long long kb = (K + 255) / 256;
  // One or two K blocks per tile are all read-out: the A-resident schedule (two accumulator sets,
  // 192-column tiles) hides it behind the next tile.  8192 x 8192 x 512: 2590-2600 TFLOP/s against
  // 2410 (256-wide) and 2226 (384-wide); K = 256: 1402-1410 against 1280-1297 and 1223-1231.
  if (kb <= 2 && fp4_arun_supports(M, N, K)) {
    *w0 = 192;
    return;
  }
  if (kb <= 1) return;   // ... and where that schedule has no form, the 256-wide tile (26.5 against 28.3 us)
  const long long waves256 = (tiles_m * ((N + 255) / 256) + clusters - 1) / clusters;
  const long long waves384 = (tiles_m * ((N + 383) / 384) + clusters - 1) / clusters;
  const double cost256 = static_cast<double>(waves256) * (kb * 556.0 + kFp4TileOverhead256);
  double cost384 = static_cast<double>(waves384) * (kb * 811.0 + kFp4TileOverhead384);
  // The 384-wide kernel ends its tile list with 256-wide tiles where that evens the clusters out.
  int wide = 0, narrow = 0;
  fp4_split_phases(M, N, K, 256, 128, clusters, &wide, &narrow);
  if (g_last_phase_cost > 0.0 && g_last_phase_cost < cost384) cost384 = g_last_phase_cost;
  if (cost384 <= cost256) *w1 = 128;
}

int fp4_launch(const Fp4Launch& L, cudaStream_t stream) {
  if (L.w0 == 192 && L.w1 == 0) return fp4_arun_launch(L, stream);
  if (L.w0 == 128 && L.w1 == 0) return launch_fp4_store<128, 0>(L, stream);
  if (L.w0 == 256 && L.w1 == 0) return launch_fp4_store<256, 0>(L, stream);
  if (L.w0 == 256 && L.w1 == 128) return launch_fp4_store<256, 128>(L, stream);
  return set_error(SMB_ERR_INVALID, "nvfp4: unsupported tile %d + %d", L.w0, L.w1);
}

}  // namespace smb
