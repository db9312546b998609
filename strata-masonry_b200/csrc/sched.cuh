// Tile hand-out for the persistent GEMM kernels: a static stride walk, or the hardware work
// queue of Blackwell ("cluster launch control", CLC): the grid is launched with one cluster per
// tile, the clusters that get to run keep running and cancel clusters that have not started yet,
// taking over their tile.  Counterpart of the reference's scheduler pieces
// (blocks/97_sched_warp_clc.cuh:108-211, composites/106_clc_fetch_next_tile.cuh:129-258,
// primitives/61, 62), reduced to one response slot: a cluster holds at most one tile beyond the
// one it is working on, so the tail of the kernel is at most one tile long.
//
// Protocol (per 2-CTA cluster, one slot):
//   scheduler thread (leader CTA):  wait slot_empty -> arm slot_full in both CTAs (16 bytes) ->
//       clusterlaunchcontrol.try_cancel ... multicast::cluster::all (response lands at the same
//       shared-memory offset in both CTAs and completes both slot_full barriers) ->
//       read its own copy; stop after the first request that cancelled nothing.
//   every consumer (load, MMA, scale, epilogue roles of both CTAs):  wait slot_full -> read the
//       response -> fence.proxy.async (the next response is written by the async proxy) ->
//       arrive on the leader's slot_empty.
#pragma once

#include "ptx.cuh"

namespace smb {

__device__ __forceinline__ void clc_try_cancel_all(uint32_t response, uint32_t bar) {
  asm volatile(
      "clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes"
      ".multicast::cluster::all.b128 [%0], [%1];"
      ::"r"(response), "r"(bar)
      : "memory");
}

// Decode a 16-byte response: returns the x index of the first CTA of the cancelled cluster, or
// -1 when nothing was cancelled.
__device__ __forceinline__ int clc_decode(uint32_t response) {
  uint32_t r0, r1, r2, r3;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(response)
               : "memory");
  uint32_t ok, x;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b128 h;\n\t"
      "mov.b128 h, {%2, %3, %4, %5};\n\t"
      "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, h;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "mov.b32 %1, 0;\n\t"
      "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %1, h;\n\t"
      "}"
      : "=r"(ok), "=r"(x)
      : "r"(r0), "r"(r1), "r"(r2), "r"(r3));
  return ok ? static_cast<int>(x) : -1;
}

// Shared-memory words the scheduler needs (inside the kernel's barrier block, 16-byte aligned
// response first).
struct SchedSmem {
  uint32_t response;     // 16 bytes
  uint32_t slot_full;    // mbarrier, count 1 + 16 transaction bytes, one per CTA
  uint32_t slot_empty;   // mbarrier in the leader CTA, count = consumers of both CTAs
};

// Per-consumer cursor over the tiles of this cluster.
struct TileCursor {
  bool dynamic;
  int stride, num_tiles;
  uint32_t full_bar, response, leader_empty, parity;

  __device__ __forceinline__ void init(bool dyn, int n_clusters, int tiles, const SchedSmem& s) {
    dynamic = dyn;
    stride = n_clusters;
    num_tiles = tiles;
    full_bar = s.slot_full;
    response = s.response;
    leader_empty = mapa_u32(s.slot_empty, 0);
    parity = 0;
  }

  // Tile after `t`; -1 when there is none; -2 when the scheduler did not answer in time.
  // `release`: this thread performs the consumer's arrival (one thread per consuming warp).
  // `whole_warp`: all 32 lanes of the warp call this together (epilogue warps); single-thread
  // roles pass false.
  __device__ __forceinline__ int next(int t, bool release, bool whole_warp) {
    if (!dynamic) {
      const int n = t + stride;
      return n < num_tiles ? n : -1;
    }
    if (!mbar_wait(full_bar, parity)) return -2;
    parity ^= 1u;
    const int cta_x = clc_decode(response);
    fence_proxy_async_smem();
    if (whole_warp) __syncwarp();
    if (release) mbar_arrive_cluster(leader_empty);
    return cta_x < 0 ? -1 : (cta_x >> 1);
  }
};

// Body of the scheduler thread (leader CTA, one thread).  Returns when the queue is drained.
__device__ __forceinline__ void clc_scheduler_loop(const SchedSmem& s, int* status) {
  const uint32_t peer_full = mapa_u32(s.slot_full, 1);
  uint32_t empty_parity = 1, full_parity = 0;
  while (true) {
    if (!mbar_wait(s.slot_empty, empty_parity)) {
      report_status(status, kDevTimeoutSched);
      return;
    }
    empty_parity ^= 1u;
    mbar_arrive_expect_tx(s.slot_full, 16);
    mbar_arrive_expect_tx_cluster(peer_full, 16);
    clc_try_cancel_all(s.response, s.slot_full);
    if (!mbar_wait(s.slot_full, full_parity)) {
      report_status(status, kDevTimeoutSched);
      return;
    }
    full_parity ^= 1u;
    const int got = clc_decode(s.response);
    fence_proxy_async_smem();
    if (got < 0) return;   // nothing left to take over: never ask again
  }
}

}  // namespace smb
