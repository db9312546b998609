// Thin inline-PTX layer for sm_100a: mbarrier, TMA, tcgen05 (TMEM + 5th-gen tensor
// cores), cluster helpers.  Every wait in here is bounded: a wait that runs out of
// budget returns false, the caller records a status word and leaves its loop, so a
// protocol slip shows up as an error code instead of a hung GPU.
//
// Replaces, for the dense GEMM path, the reference's one-instruction wrappers under
// src/primitives/ (0,1,2 tcgen05 alloc/dealloc/relinquish; 3,5 tcgen05.mma; 8 idesc;
// 9,12 tcgen05.ld/wait; 11 commit; 13 tcgen05.cp; 19 TMA load (2-SM form); 22,25 TMA
// store + bulk groups; 29-35 mbarrier + fences; 38 cluster barrier; 42 smem
// descriptor; 63 cvt; 67 mapa; 68 L2 policies).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

namespace smb {

// ---------------------------------------------------------------------------------
// Status words written by kernels (first writer wins).
// ---------------------------------------------------------------------------------
enum DeviceStatus : int {
  kDevOk = 0,
  kDevTimeoutProducer = 101,   // load role gave up waiting for a free ring slot
  kDevTimeoutMmaFull = 102,    // MMA role gave up waiting for a filled ring slot
  kDevTimeoutMmaAcc = 103,     // MMA role gave up waiting for a drained accumulator
  kDevTimeoutEpilogue = 104,   // epilogue role gave up waiting for an accumulator
  kDevTimeoutSched = 105,      // a role gave up waiting for the tile scheduler
  kDevTimeoutFixup = 106,      // split-K fix-up wait gave up
  kDevTimeoutProbe = 107,      // the bounded-wait self test (expected outcome)
  kDevTimeoutActivations = 108,  // decode kernel gave up waiting for the grid's activation quantiser
};

// Wait budget in SM clock cycles (~2 s at 2 GHz).  The longest legitimate wait on this
// path is one full K loop of a tile (tens of microseconds).
#ifndef SMB_WAIT_BUDGET_CYCLES
#define SMB_WAIT_BUDGET_CYCLES (4000000000LL)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

__device__ __forceinline__ uint32_t cluster_id_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r));
  return r;
}

__device__ __forceinline__ uint32_t num_clusters_x() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r));
  return r;
}

// Address of the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local_addr, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(local_addr), "r"(rank));
  return out;
}

__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  cluster_arrive();
  cluster_wait();
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init_cluster() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Local arrive (count 1).
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier that may live in another CTA of the cluster (address from mapa), ordering
// this thread's earlier memory accesses before it at cluster scope.  The cluster-scope release is
// expensive when the thread has memory operations in flight: 600 to 1300 cycles per arrival were
// measured in an epilogue warp that had just issued its TMA stores.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}

// The same arrival without the cluster-scope release (about 50 cycles).  For hand-overs that
// publish no memory: tensor-memory columns a warp has finished reading, where
// tcgen05.wait::ld + tcgen05.fence::before_thread_sync already order the reads before the arrival.
__device__ __forceinline__ void mbar_arrive_cluster_no_release(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}

// Local arrive + expect-tx.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

// Arrive + expect-tx on a barrier that may live in another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_expect_tx_cluster(uint32_t cluster_bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(
                   cluster_bar),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the cycle budget ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          long long budget = SMB_WAIT_BUDGET_CYCLES) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (clock64() - t0 > budget) return false;
    }
  }
  return true;
}

// ---------------------------------------------------------------------------------
// TMA
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}

// 2-D tiled load into this CTA's shared memory with an L2 eviction hint (kernels launched
// without clusters: the CTA is its own cluster of one).
__device__ __forceinline__ void tma_load_2d_cta_hint(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                                     int x, int y, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(m), "r"(bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

// Same, issued from one CTA of a cta_group::2 pair: data lands in this CTA's shared memory,
// completion bytes are credited to `cluster_bar`, which may be the leader CTA's barrier.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m,
                                                 uint32_t cluster_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile"
      ".mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(m), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t dst, const CUtensorMap* m,
                                                      uint32_t cluster_bar, int x, int y,
                                                      uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile"
      ".mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(m), "r"(cluster_bar), "r"(x), "r"(y), "l"(policy)
      : "memory");
}

// Pull one box into L2 only (no shared-memory destination, no completion signal).
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* m, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(m), "r"(x),
               "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(m), "r"(src), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---------------------------------------------------------------------------------
// tcgen05: tensor memory management
// ---------------------------------------------------------------------------------
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
                 "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
                 "r"(ncols)
                 : "memory");
  }
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (CTA_GROUP == 1) {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  }
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------------------------
// tcgen05: descriptors
// ---------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes
// with the 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B produces).
// Bit layout: [0,14) start address >> 4; [16,30) leading byte offset >> 4; [32,46) stride
// byte offset >> 4 (distance between 8-row groups = 1024 B); [46,48) constant 0b01;
// [49,52) base offset; [61,64) swizzle mode (2 = 128 B, 0 = none).
__host__ __device__ constexpr uint64_t make_smem_desc(uint32_t smem_addr, uint32_t sbo_bytes,
                                                      uint32_t lbo_bytes, uint32_t swizzle_mode) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) |
         (static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         (static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) |
         (static_cast<uint64_t>(swizzle_mode & 7u) << 61);
}
constexpr uint32_t kSwizzleNone = 0;
constexpr uint32_t kSwizzle128B = 2;

// Instruction descriptor, kind::f16 with BF16 operands, FP32 accumulate, both operands
// K-major.  [4,6) D format (1 = F32); [7,10) A format (1 = BF16); [10,13) B format;
// [15] A major; [16] B major (0 = K); [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int mma_m, int mma_n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((static_cast<uint32_t>(mma_n) >> 3) << 17) |
         ((static_cast<uint32_t>(mma_m) >> 4) << 24);
}

// Instruction descriptor, kind::mxf4nvf4 with E2M1 operands, block scales.
// [4,6) B scale-factor id; [7,10) A format (1 = E2M1); [10,13) B format (1 = E2M1);
// [17,23) N >> 3; [23] scale type (1 = UE8M0); [27,29) M >> 7; [29,31) A scale-factor id.
__host__ __device__ constexpr uint32_t make_idesc_mxf4(int mma_m, int mma_n, uint32_t sf_id_a,
                                                       uint32_t sf_id_b, bool ue8m0) {
  return ((sf_id_b & 3u) << 4) | (1u << 7) | (1u << 10) |
         ((static_cast<uint32_t>(mma_n) >> 3) << 17) | ((ue8m0 ? 1u : 0u) << 23) |
         (((static_cast<uint32_t>(mma_m) >> 7) & 3u) << 27) | ((sf_id_a & 3u) << 29);
}

// ---------------------------------------------------------------------------------
// tcgen05: MMA issue, commit, scale copy
// ---------------------------------------------------------------------------------
template <int CTA_GROUP>
__device__ __forceinline__ void mma_bf16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Block-scaled E2M1 x E2M1, one UE4M3 scale per 16 K (four scales = one 4-byte cell per K=64
// instruction; scale ids are 0).
template <int CTA_GROUP>
__device__ __forceinline__ void mma_nvf4_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                            uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X"
        " [%0], %1, %2, %3, [%4], [%5], p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X"
        " [%0], %1, %2, %3, [%4], [%5], p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(accumulate)
        : "memory");
  }
}

// Block-scaled E2M1 x E2M1, one scale per 32 K (two scales per K=64 instruction).
template <int CTA_GROUP>
__device__ __forceinline__ void mma_mxf4_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                            uint32_t idesc, uint32_t tmem_sfa, uint32_t tmem_sfb,
                                            uint32_t accumulate) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::2X"
        " [%0], %1, %2, %3, [%4], [%5], p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::2X"
        " [%0], %1, %2, %3, [%4], [%5], p;\n\t"
        "}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(tmem_sfa), "r"(tmem_sfb),
        "r"(accumulate)
        : "memory");
  }
}

// Copy 32 rows x 16 bytes of shared memory into 4 TMEM columns, replicated into all four
// 32-lane quarters (the layout block-scaled MMA reads its scale factors from).
template <int CTA_GROUP>
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint64_t smem_desc) {
  if constexpr (CTA_GROUP == 1) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc)
                 : "memory");
  } else {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc)
                 : "memory");
  }
}

// Make `bar` (this CTA) complete one arrival once all tensor-core work issued so far by this
// thread has finished.
__device__ __forceinline__ void mma_commit_1cta(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// Pair form: the barrier at the same offset in every CTA named by `cta_mask` gets one arrival.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;"
      ::"r"(bar), "h"(cta_mask)
      : "memory");
}

// ---------------------------------------------------------------------------------
// tcgen05: accumulator read-back
// ---------------------------------------------------------------------------------
// 32 lanes x 32 consecutive fp32 columns: thread i of the warp receives lane (base+i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Two fp32 -> packed bf16x2 (round to nearest even); `lo` lands in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(uint32_t lo_f32_bits, uint32_t hi_f32_bits) {
  uint32_t out;
  asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;"
               : "=r"(out)
               : "f"(__uint_as_float(hi_f32_bits)), "f"(__uint_as_float(lo_f32_bits)));
  return out;
}

// silu(gate) * up with silu(z) = 0.5 z (1 + tanh(z / 2)) on the hardware tanh approximation: the
// form of the reference's gated epilogue (composites/130_swiglu_act.cuh:33-50); finite for all
// finite inputs.
__device__ __forceinline__ float swiglu_f32(float gate, float up) {
  const float half_z = 0.5f * gate;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(half_z));
  return __fmaf_rn(half_z, t, half_z) * up;
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

__device__ __forceinline__ void ld_shared_v4(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c,
                                             uint32_t& d) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "r"(addr)
               : "memory");
}

// 16-byte store to (possibly another GPU's) global memory; `ptr` must be 16-byte aligned.
__device__ __forceinline__ void st_global_v4(void* ptr, uint32_t a, uint32_t b, uint32_t c,
                                             uint32_t d) {
  asm volatile("st.global.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(ptr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}

// Programmatic dependent launch: let the next grid on the stream start early / wait for the
// previous grid to finish and its writes to become visible.
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// First writer wins.
__device__ __forceinline__ void report_status(int* status, int code) {
  if (status != nullptr) atomicCAS(status, 0, code);
}

}  // namespace smb
