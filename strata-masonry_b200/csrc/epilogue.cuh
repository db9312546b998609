// Accumulator read-back shared by the GEMM kernels: tensor memory -> registers (rounded to
// bf16) -> 128-byte-swizzled shared memory -> TMA store, one independent chain per warp.
// Counterpart of the reference's epilogue blocks (blocks/93_epi_warp_blackwell.cuh:192-321 and
// the per-warp store chains of nvfp4/dense_gemm_nvfp4.cu:1343-1424), without CTA-wide barriers.
#pragma once

#include "gemm_common.cuh"
#include "ptx.cuh"

namespace smb {

constexpr int kStoreCols = 64;                        // columns per store box (128 bytes of bf16)
constexpr int kStoreBufBytes = 32 * kStoreCols * 2;   // one warp's 32 x 64 bf16 staging box

// Extra destinations of every stored box: the same [M, N] block written into other buffers,
// normally the full D of the other GPUs of the box (the all-gather of a column-sharded GEMM done
// by the epilogue itself, over peer-mapped memory).  Plain 16-byte stores: peer memory takes
// ordinary stores, and nothing here waits on another GPU; the data is visible to the peer once
// this kernel has completed.  No counterpart in the reference (it is single-GPU).
// (struct PeerCopies: gemm_common.cuh)

struct StoreTarget {
  const CUtensorMap* tmap_d;   // D as [M, N] bf16, box 32 x 64, 128-byte swizzle (TMA path)
  uint16_t* d_ptr;             // D base and pitch (plain-store path)
  int ldd;
  int M, N;
  const PeerCopies* peers;     // kernel parameter, TMA path only (N % 8 == 0 there)
  float alpha;                 // factor on every accumulator (kScaled instantiations only)
  int row_end;                 // rows >= row_end are not written (a tile's share of a ragged group;
                               // M where tiles own whole boxes)
};

// One warp drains kCols fp32 columns of its 32 TMEM lanes starting at `taddr`, then writes them
// to D rows [row0, row0 + 32), columns [col0, col0 + kCols).
//   Phase 1: everything is pulled into registers (two bf16 per register) and `release_bar` (a
//   cluster-mapped mbarrier address) gets one arrival: the accumulator columns are free again
//   before any store is issued.
//   Phase 2: 64-column boxes go through the warp's staging buffer `sbuf` (1024-byte aligned).
// kTmaStore = false is the path for a D whose rows are not 16-byte aligned.
//
// kSwiglu: gated-activation epilogue (the reference's epi_warp_blackwell_*_bf16_swiglu,
// blocks/93_epi_warp_blackwell.cuh:439-596, with composites/130_swiglu_act.cuh): B rows are
// interleaved, even = up, odd = gate, so accumulator column 2n is up_n and 2n + 1 is gate_n;
// the output is D[m, n] = bf16(silu(gate_n) * up_n), half as wide as the accumulator.  col0 is
// then the accumulator column; out.N and the tensor map describe the [M, N/2] output.
// kScaled: every accumulator is multiplied by out.alpha first (the per-tensor scales of NVFP4).
// Phase 1 alone: kCols fp32 columns of this warp's 32 lanes, starting at `taddr`, into
// `packed` (two bf16 per register; kSwiglu: one output pair per four accumulator columns).
template <int kCols, bool kSwiglu = false, bool kScaled = false>
__device__ __forceinline__ void drain_columns(uint32_t taddr, float alpha,
                                              uint32_t (&packed)[(kSwiglu ? kCols / 2 : kCols) / 2]) {
#pragma unroll
  for (int g = 0; g < kCols / 32; ++g) {
    uint32_t v[32];
    tmem_ld_32x32b_x32(taddr + g * 32, v);
    tmem_ld_wait();
    if (kScaled) {
#pragma unroll
      for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
    }
    if (kSwiglu) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float o0 = swiglu_f32(__uint_as_float(v[4 * i + 1]), __uint_as_float(v[4 * i]));
        const float o1 = swiglu_f32(__uint_as_float(v[4 * i + 3]), __uint_as_float(v[4 * i + 2]));
        packed[g * 8 + i] = pack_bf16x2(__float_as_uint(o0), __float_as_uint(o1));
      }
    } else {
#pragma unroll
      for (int i = 0; i < 16; ++i) packed[g * 16 + i] = pack_bf16x2(v[2 * i], v[2 * i + 1]);
    }
  }
}

// Hand the drained accumulator columns back to the MMA role: one arrival on `release_bar` (a
// cluster-mapped mbarrier address) per warp.  Every lane's tcgen05.ld has completed
// (tcgen05.wait::ld in drain_columns) and is fenced before the warp-level sync; the arrival itself
// publishes no memory, so it carries no cluster-scope release (which cost the MMA role 1700 idle
// cycles per 256 x 384 tile when it did).
__device__ __forceinline__ void release_columns(uint32_t release_bar, int lane) {
  tc_fence_before_sync();
  __syncwarp();
  if (lane == 0) mbar_arrive_cluster_no_release(release_bar);
}

// Phase 2 alone: kOutCols packed columns to D rows [row0, row0 + 32), columns [col0, col0 + kOutCols),
// in 64-column boxes through the warp's staging buffer.
template <int kOutCols, bool kTmaStore>
__device__ __forceinline__ void store_columns(const uint32_t (&packed)[kOutCols / 2], uint32_t sbuf,
                                              const StoreTarget& out, int row0, int col0, int lane) {
  static_assert(kOutCols % kStoreCols == 0, "whole store boxes only");
#pragma unroll
  for (int c = 0; c < kOutCols / kStoreCols; ++c) {
    // The TMA store that last read the staging buffer must have finished reading it.
    if (kTmaStore) {
      if (lane == 0) bulk_wait_group_read<0>();
    }
    __syncwarp();
    // Row `lane` of the box; 16-byte chunk j goes to chunk (j ^ (lane & 7)): the 128-byte
    // swizzle the store tensor map expects.
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t dst = sbuf + lane * 128 + ((j ^ (lane & 7)) << 4);
      st_shared_v4(dst, packed[c * 32 + 4 * j], packed[c * 32 + 4 * j + 1],
                   packed[c * 32 + 4 * j + 2], packed[c * 32 + 4 * j + 3]);
    }
    const int gcol0 = col0 + c * kStoreCols;
    if (kTmaStore) {
      fence_proxy_async_smem();
      __syncwarp();
      const int n_peers = out.peers->count;
      const int route_rows = out.peers->route_rows;   // > 0: rows are routed, D itself is not written
      const bool whole_box = row0 + 32 <= out.row_end || out.row_end >= out.M;
      if (lane == 0) {
        if (whole_box && route_rows == 0 && row0 < out.M && gcol0 < out.N) tma_store_2d(out.tmap_d, sbuf, gcol0, row0);
        bulk_commit_group();
      }
      if (!whole_box && route_rows == 0 && row0 < out.row_end) {
        // The tile's rows end inside this box (last tile of a group whose row count is not a
        // multiple of 32): the rows that belong to it go out with 16-byte stores, lane l chunk
        // l % 8 of rows l / 8 + 4 i, read back from the swizzled staging box.
        const int chunk = lane & 7;
        const int gcol = gcol0 + chunk * 8;
#pragma unroll 1
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          uint32_t x0, x1, x2, x3;
          ld_shared_v4(sbuf + r * 128 + ((chunk ^ (r & 7)) << 4), x0, x1, x2, x3);
          const int grow = row0 + r;
          if (grow < out.row_end && gcol < out.N)
            st_global_v4(out.d_ptr + static_cast<long long>(grow) * out.ldd + gcol, x0, x1, x2, x3);
        }
      }
      if (n_peers > 0) {
        // Lane l copies 16-byte chunk (l % 8) of rows (l / 8) + 4 i: a warp instruction covers
        // four whole 128-byte row segments, read back from the swizzled staging box.
        const int chunk = lane & 7;
        const int gcol = gcol0 + chunk * 8;
#pragma unroll 1
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          uint32_t x0, x1, x2, x3;
          ld_shared_v4(sbuf + r * 128 + ((chunk ^ (r & 7)) << 4), x0, x1, x2, x3);
          const int grow = row0 + r;
          if (grow < out.M && grow < out.row_end && gcol < out.N) {
            if (route_rows > 0) {
              // Row block b (route_rows rows, a multiple of the tile height, so a warp's 32 rows
              // share it) goes to destination b, at its row inside the block.
              const int b = row0 / route_rows;
              const long long off = static_cast<long long>(grow - b * route_rows) * out.peers->ld + gcol;
              st_global_v4(out.peers->base[b] + off, x0, x1, x2, x3);
            } else {
              const long long off = static_cast<long long>(grow) * out.peers->ld + gcol;
#pragma unroll 1
              for (int q = 0; q < n_peers; ++q) st_global_v4(out.peers->base[q] + off, x0, x1, x2, x3);
            }
          }
        }
      }
    } else {
      // Read the staged box back so that consecutive lanes write consecutive columns of a row.
      __syncwarp();
      for (int r = 0; r < 32; ++r) {
        const int grow = row0 + r;
        if (grow >= out.M || grow >= out.row_end) break;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int cc = h * 32 + lane;
          const int gcol = gcol0 + cc;
          const uint32_t src = sbuf + r * 128 + ((((cc >> 3) ^ (r & 7)) << 4) | ((cc & 7) << 1));
          uint16_t val;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(val) : "r"(src) : "memory");
          if (gcol < out.N) out.d_ptr[static_cast<size_t>(grow) * out.ldd + gcol] = val;
        }
      }
      __syncwarp();
    }
  }
}

template <int kCols, bool kTmaStore, bool kSwiglu = false, bool kScaled = false>
__device__ __forceinline__ void drain_and_store(uint32_t taddr, uint32_t sbuf, const StoreTarget& out,
                                                int row0, int col0, uint32_t release_bar, int lane) {
  constexpr int kOutCols = kSwiglu ? kCols / 2 : kCols;
  static_assert(kOutCols % kStoreCols == 0, "whole store boxes only");
  static_assert(!kSwiglu || kTmaStore, "the gated epilogue uses the aligned store path");
  if (kSwiglu) col0 /= 2;
  uint32_t packed[kOutCols / 2];
  drain_columns<kCols, kSwiglu, kScaled>(taddr, out.alpha, packed);
  release_columns(release_bar, lane);
  store_columns<kOutCols, kTmaStore>(packed, sbuf, out, row0, col0, lane);
}

// Call once per warp after its last tile: the CTA's shared memory must outlive the reads of its
// outstanding TMA stores.  Waiting for the reads is enough: the global writes themselves are
// ordinary memory traffic in flight, which completes before the grid is reported complete (and
// before a dependent grid's griddepcontrol.wait returns).
template <bool kTmaStore>
__device__ __forceinline__ void drain_store_groups(int lane) {
  if (kTmaStore) {
    if (lane == 0) bulk_wait_group_read<0>();
  }
  __syncwarp();
}

}  // namespace smb
