// C-ABI of the block-scaled FP4 GEMM: plans, launch, status check, host-buffer path.
// Host-side counterpart of run_one_k1 in the reference
// (src/kernels/gemm/sm100a/nvfp4/dense_gemm_nvfp4.cu:2353-2700).
#include <cstdio>
#include <cstdlib>
#include <new>
#include <vector>

#include "formats.cuh"
#include "gemm_common.cuh"

namespace smb {
const char* device_status_name(int code);
int build_group_tiles(const int* offsets, int groups, int align, int** table_dev, int* tiles_out, int* m_total);
}

using namespace smb;

struct smb_fp4_plan {
  Fp4Launch launch;
  int* status_dev;
  bool owns_status;   // false: the word belongs to a host context that several plans report into
  int device;   // the device that was current at creation
  // Skinny shapes (M <= 128) run the decode kernel.  Its scratch (partial-sum slots and tile
  // counters) is only touched when the CTA count is capped and tiles are split along K.
  bool decode;
  Fp4DecodeLaunch dlaunch;
  void* scratch_dev;      // fp32 slabs followed by the per-tile counters
  size_t scratch_bytes;
  // Plans created from BF16 activations quantise them into plan-owned buffers before every run.
  const void* act_src;
  int64_t act_ld;
  void* act_codes;
  void* act_sf;
  void* act_counter;   // 8 bytes: CTAs counted in by the in-kernel quantiser
  int* tile_table_dev; // ragged grouped plans: [3][tiles] = first row, end of group, group id
};

namespace {

int fp4_plan_create_impl(smb_fp4_plan** out, const void* a, const void* sfa, const void* b, const void* sfb,
                         void* d, int M, int N, int K, int64_t lda_bytes, int64_t ldb_bytes, int64_t ldd,
                         unsigned flags, int groups, const int* mtile_group, int* shared_status = nullptr) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null output handle");
  *out = nullptr;
  if (a == nullptr || b == nullptr || sfa == nullptr || sfb == nullptr || d == nullptr)
    return set_error(SMB_ERR_INVALID, "fp4 plan: null operand pointer");
  if (M <= 0 || N <= 0 || K <= 0)
    return set_error(SMB_ERR_INVALID, "fp4 plan: dimensions must be positive (M=%d N=%d K=%d)", M, N, K);
  if (K % 32 != 0)
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: K=%d must be a multiple of 32 (one scale per 32 K)", K);
  const bool block16 = (flags & SMB_FLAG_SCALE_BLOCK16) != 0;
  if (block16 && K % 64 != 0)
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: block-16 scales need K %% 64 == 0 (K=%d)", K);
  if (block16 && (flags & SMB_FLAG_EPILOGUE_SWIGLU))
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: no gated epilogue for block-16 scales");
  const bool swiglu = (flags & SMB_FLAG_EPILOGUE_SWIGLU) != 0;
  if (swiglu && N % 2 != 0)
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: the gated epilogue needs an even N (up/gate row pairs of B)");
  if (swiglu && M <= 128 && !(flags & SMB_FLAG_NO_DECODE) && (flags & SMB_FLAG_DECODE_SINGLE))
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: the decode kernel's single-tile form has no gated epilogue");
  const int n_out = swiglu ? N / 2 : N;
  if (lda_bytes < K / 2 || ldb_bytes < K / 2 || ldd < n_out)
    return set_error(SMB_ERR_INVALID, "fp4 plan: leading dimension smaller than the row length");
  if (lda_bytes % 16 != 0 || ldb_bytes % 16 != 0)
    return set_error(SMB_ERR_INVALID, "fp4 plan: operand row pitches must be multiples of 16 bytes");
  if (ldd > 0x7FFFFFFFLL)
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: ldd above 2^31 - 1 elements");
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess)
    return set_error(SMB_ERR_CUDA, "fp4 plan: no current CUDA device");

  smb_fp4_plan* p = new (std::nothrow) smb_fp4_plan();
  if (p == nullptr) return set_error(SMB_ERR_NOMEM, "fp4 plan: out of host memory");
  p->device = device;
  Fp4Launch& L = p->launch;
  L.M = M;
  L.N = N;
  L.K = K;
  fp4_pick_tile(M, N, K, device_cluster_slots(), &L.w0, &L.w1);
  if (flags & SMB_FLAG_TILE_N_128) { L.w0 = 128; L.w1 = 0; }
  if (flags & SMB_FLAG_TILE_N_256) { L.w0 = 256; L.w1 = 0; }
  if (flags & SMB_FLAG_TILE_N_384) { L.w0 = 256; L.w1 = 128; }
  if (flags & SMB_FLAG_TILE_N_192) {
    if (!fp4_arun_supports(M, N, K) || block16 || swiglu || mtile_group != nullptr || (flags & SMB_FLAG_DYNAMIC_TILES)) {
      delete p;
      return set_error(SMB_ERR_UNSUPPORTED,
                       "fp4 plan: the A-resident schedule needs K <= 2048, N >= 384 and the plain UE8M0 GEMM");
    }
    L.w0 = 192;
    L.w1 = 0;
  }
  L.group_m = 0;
  L.max_clusters = 0;
  L.prof = nullptr;
  L.prefetch = 0;
  L.uniform_tiles = false;
  L.l2_a = L.l2_b = 0;
  if (const char* env = getenv("SMB_TUNE_FP4_L2")) {   // tuning sweeps: "<a><b>", digits 0..2
    if (env[0] >= '0' && env[0] <= '2' && env[1] >= '0' && env[1] <= '2') {
      L.l2_a = env[0] - '0';
      L.l2_b = env[1] - '0';
    }
  }
  if (getenv("SMB_TUNE_FP4_UNIFORM")) L.uniform_tiles = true;
  L.dynamic = (flags & SMB_FLAG_DYNAMIC_TILES) != 0;
  L.operands_static = (flags & (SMB_FLAG_OPERANDS_STATIC | SMB_FLAG_LAUNCH_INDEPENDENT)) != 0;
  L.output_independent = (flags & SMB_FLAG_LAUNCH_INDEPENDENT) != 0;
  L.peers.count = 0;
  L.peers.route_rows = 0;
  L.peers.first_block = 0;
  L.mtile_group = mtile_group;
  L.tile_row0 = L.tile_row_end = nullptr;
  L.tile_rows = 0;
  p->tile_table_dev = nullptr;
  L.d = d;
  L.ldd = static_cast<int>(ldd);
  L.tma_store = (ldd % 8 == 0) && (reinterpret_cast<uintptr_t>(d) % 16 == 0) &&
                !(flags & SMB_FLAG_FORCE_PLAIN_STORE);
  L.block16 = block16;
  L.alpha = 1.0f;
  if (block16) {
    L.w0 = 256;
    L.w1 = 0;
  }
  // The A-resident schedule has no grouped or queued form (and no block-16 or gated one: those
  // choose their tile above and below).
  if (L.w0 == 192 && !(flags & SMB_FLAG_TILE_N_192) && (mtile_group != nullptr || L.dynamic)) {
    L.w0 = 256;
    L.w1 = 0;
  }
  L.swiglu = swiglu;
  if (swiglu) {
    if (!L.tma_store) {
      delete p;
      return set_error(SMB_ERR_UNSUPPORTED,
                       "fp4 plan: the gated epilogue needs a 16-byte-aligned D with ldd %% 8 == 0");
    }
    if (L.w0 < 256) {   // four accumulator columns make two outputs: at least 128 columns per warp
      L.w0 = 256;
      L.w1 = 0;
    }
  }
  p->status_dev = nullptr;
  p->decode = (M <= 128) && !(flags & SMB_FLAG_NO_DECODE) && mtile_group == nullptr;
  p->scratch_dev = nullptr;
  p->scratch_bytes = 0;
  p->act_src = nullptr;
  p->act_ld = 0;
  p->act_codes = p->act_sf = p->act_counter = nullptr;

  // Packed scales: chunks of 4 scale bytes per row, i.e. K = 128 (one scale per 32) or K = 64
  // (one per 16); a stage (K = 256) reads 2 or 4 chunks of 64 words.
  const uint64_t kchunks = block16 ? static_cast<uint64_t>(K) / 64 : (static_cast<uint64_t>(K) / 32 + 3) / 4;
  const uint32_t sf_box = block16 ? 256 : 128;
  const uint64_t bands_a = (static_cast<uint64_t>(M) + 127) / 128;
  const uint64_t rows_b = static_cast<uint64_t>(groups) * N;   // B (and its scales) of all groups stacked
  const uint64_t bands_b = (rows_b + 127) / 128;
  const int tile_n = L.w0 + L.w1;
  int rc = encode_tmap_2d(&L.tmap_a, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K / 2, lda_bytes, 128, 128, true);
  if (rc == SMB_OK)
    rc = encode_tmap_2d(&L.tmap_b0, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows_b, K / 2, ldb_bytes, L.w0 / 2, 128, true);
  if (rc == SMB_OK) {
    if (L.w1 > 0)
      rc = encode_tmap_2d(&L.tmap_b1, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, rows_b, K / 2, ldb_bytes, L.w1 / 2, 128, true);
    else
      L.tmap_b1 = L.tmap_b0;
  }
  if (rc == SMB_OK)
    rc = encode_tmap_2d(&L.tmap_sfa, sfa, CU_TENSOR_MAP_DATA_TYPE_UINT64, 8, bands_a, kchunks * 64,
                        kchunks * 512, 1, sf_box, false);
  if (rc == SMB_OK)
    rc = encode_tmap_2d(&L.tmap_sfb, sfb, CU_TENSOR_MAP_DATA_TYPE_UINT64, 8, bands_b, kchunks * 64,
                        kchunks * 512, (tile_n + 127) / 128, sf_box, false);
  if (rc == SMB_OK) {
    if (L.tma_store)
      rc = encode_tmap_2d(&L.tmap_d, d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, n_out, ldd * 2, 32, 64, true);
    else
      L.tmap_d = L.tmap_a;
  }
  p->owns_status = (shared_status == nullptr);
  if (rc == SMB_OK && p->owns_status) {
    cudaError_t e = cudaMalloc(&p->status_dev, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(p->status_dev, 0, sizeof(int));
    if (e != cudaSuccess) rc = set_cuda_error(e, "fp4 plan: status word allocation");
  } else if (rc == SMB_OK) {
    p->status_dev = shared_status;
  }
  if (rc == SMB_OK && p->decode) {
    // Operands swap roles: the weights (B, N rows) fill the 128 rows of the MMA, the
    // activations (A, M rows) its N dimension.
    Fp4DecodeLaunch& D = p->dlaunch;
    D.M = M;
    D.N = N;
    D.K = K;
    D.max_ctas = 0;
    D.max_stages = 0;
    D.no_overlap = (flags & SMB_FLAG_NO_LAUNCH_OVERLAP) != 0;
    D.activations_dynamic = false;
    D.block16 = block16;
    D.alpha = 1.0f;
    D.swiglu = swiglu;
    D.dual = swiglu ? true : fp4_decode_prefers_dual(M);
    if (flags & SMB_FLAG_DECODE_DUAL) D.dual = true;
    // Asked for by name, the dual form keeps its operands swapped for every M (no wide form).
    D.narrow = (flags & SMB_FLAG_DECODE_DUAL) != 0;
    D.act_src = nullptr;
    D.act_ld = 0;
    D.act_mode = 0;
    D.act_codes = D.act_sf = nullptr;
    D.act_counter = nullptr;
    if (flags & SMB_FLAG_DECODE_SINGLE) D.dual = false;
    const int m_pad = (M + 15) / 16 * 16;
    rc = encode_tmap_2d(&D.tmap_w, b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, N, K / 2, ldb_bytes, 128, 128, true);
    if (rc == SMB_OK)
      rc = encode_tmap_2d(&D.tmap_x, a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, M, K / 2, lda_bytes, m_pad, 128, true);
    if (rc == SMB_OK)
      rc = encode_tmap_2d(&D.tmap_sfw, sfb, CU_TENSOR_MAP_DATA_TYPE_UINT64, 8, bands_b, kchunks * 64,
                          kchunks * 512, 1, sf_box, false);
    if (rc == SMB_OK)
      rc = encode_tmap_2d(&D.tmap_sfx, sfa, CU_TENSOR_MAP_DATA_TYPE_UINT64, 8, bands_a, kchunks * 64,
                          kchunks * 512, 1, sf_box, false);
    if (rc == SMB_OK) rc = fp4_decode_bind_output(&D, d, M, N, ldd, !(flags & SMB_FLAG_FORCE_PLAIN_STORE));
    if (rc == SMB_OK) {
      // Two partial-sum slots per CTA (one CTA per SM of this device) and one counter per tile.
      int sms = 2 * device_cluster_slots();
      if (sms <= 0) sms = 148;
      const size_t slot_bytes = 2 * static_cast<size_t>(sms) * fp4_decode_slot_bytes(M);
      p->scratch_bytes = fp4_decode_scratch_bytes(M, N, sms);
      cudaError_t e = cudaMalloc(&p->scratch_dev, p->scratch_bytes);
      if (e == cudaSuccess) e = cudaMemset(p->scratch_dev, 0, p->scratch_bytes);
      if (e != cudaSuccess) rc = set_cuda_error(e, "fp4 plan: decode scratch allocation");
      D.scratch = static_cast<float*>(p->scratch_dev);
      D.scratch_ctas = sms;
      D.counters = reinterpret_cast<int*>(static_cast<char*>(p->scratch_dev) + slot_bytes);
    }
  }
  if (rc != SMB_OK) {
    if (p->status_dev && p->owns_status) cudaFree(p->status_dev);
    if (p->scratch_dev) cudaFree(p->scratch_dev);
    delete p;
    return rc;
  }
  L.status = p->status_dev;
  p->dlaunch.status = p->status_dev;
  *out = p;
  return SMB_OK;
}

}  // namespace

extern "C" int smb_fp4_plan_create(smb_fp4_plan** out, const void* a, const void* sfa, const void* b,
                                   const void* sfb, void* d, int M, int N, int K, int64_t lda_bytes,
                                   int64_t ldb_bytes, int64_t ldd, unsigned flags) {
  return fp4_plan_create_impl(out, a, sfa, b, sfb, d, M, N, K, lda_bytes, ldb_bytes, ldd, flags, 1, nullptr);
}

extern "C" int smb_fp4_grouped_plan_create(smb_fp4_plan** out, const void* a, const void* sfa,
                                           const void* b_stacked, const void* sfb_stacked, void* d,
                                           int M_total, int N, int K, int groups, const int* mtile_group_dev,
                                           unsigned flags) {
  if (groups < 1) return set_error(SMB_ERR_INVALID, "grouped fp4 plan: at least one group");
  if (mtile_group_dev == nullptr)
    return set_error(SMB_ERR_INVALID, "grouped fp4 plan: null tile-to-group map");
  if (M_total <= 0 || M_total % 256 != 0)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "grouped fp4 plan: every group's rows must be padded to a multiple of 256 (M_total=%d)",
                     M_total);
  if (N % 128 != 0)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "grouped fp4 plan: N=%d must be a multiple of 128 (scale bands of the stacked B)", N);
  if (static_cast<long long>(groups) * N > 0x7FFFFFFFLL)
    return set_error(SMB_ERR_UNSUPPORTED, "grouped fp4 plan: groups * N too large");
  return fp4_plan_create_impl(out, a, sfa, b_stacked, sfb_stacked, d, M_total, N, K, K / 2, K / 2, N, flags,
                              groups, mtile_group_dev);
}

extern "C" int smb_fp4_grouped_plan_create_offsets(smb_fp4_plan** out, const void* a, const void* sfa,
                                                   const void* b_stacked, const void* sfb_stacked, void* d, int N,
                                                   int K, int groups, const int* group_offsets, unsigned flags) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "grouped fp4 plan: null output handle");
  *out = nullptr;
  if (N % 128 != 0)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "grouped fp4 plan: N=%d must be a multiple of 128 (scale bands of the stacked B)", N);
  if (static_cast<long long>(groups) * N > 0x7FFFFFFFLL)
    return set_error(SMB_ERR_UNSUPPORTED, "grouped fp4 plan: groups * N too large");
  int* table = nullptr;
  int tiles = 0, m_total = 0;
  // The packed scales of A come in bands of 128 rows: a group has to start on a band.
  int rc = build_group_tiles(group_offsets, groups, 128, &table, &tiles, &m_total);
  if (rc != SMB_OK) return rc;
  rc = fp4_plan_create_impl(out, a, sfa, b_stacked, sfb_stacked, d, m_total, N, K, K / 2, K / 2,
                            (flags & SMB_FLAG_EPILOGUE_SWIGLU) ? N / 2 : N, flags | SMB_FLAG_NO_DECODE, groups,
                            table + 2 * tiles);
  if (rc != SMB_OK) {
    cudaFree(table);
    return rc;
  }
  (*out)->tile_table_dev = table;
  (*out)->launch.tile_row0 = table;
  (*out)->launch.tile_row_end = table + tiles;
  (*out)->launch.tile_rows = tiles;
  return SMB_OK;
}

extern "C" int smb_fp4_plan_tune(smb_fp4_plan* plan, int group_m, int max_clusters, int prefetch) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null handle");
  if (group_m < 0 || max_clusters < 0) return set_error(SMB_ERR_INVALID, "fp4 plan: negative tuning value");
  plan->launch.group_m = group_m;
  plan->launch.max_clusters = max_clusters;
  if (prefetch >= 0) plan->launch.prefetch = prefetch;
  // For the decode kernel the same two knobs cap the ring depth and the CTA count.
  plan->dlaunch.max_stages = group_m;
  plan->dlaunch.max_ctas = max_clusters;
  return SMB_OK;
}

extern "C" int smb_fp4_plan_set_peer_copies(smb_fp4_plan* plan, int count, void* const* dst,
                                            int64_t ld) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null handle");
  if (plan->decode && count != 0)
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: the decode kernel (M <= 128) has no peer copies");
  return set_peer_copies(&plan->launch.peers, plan->launch.tma_store, count, dst, ld,
                         plan->launch.swiglu ? plan->launch.N / 2 : plan->launch.N);
}

extern "C" int smb_fp4_plan_set_row_route(smb_fp4_plan* plan, int blocks, void* const* dst,
                                          int rows_per_block, int64_t ld, int first_block) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null handle");
  if (plan->decode && blocks != 0)
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: the decode kernel (M <= 128) has no row route");
  return set_row_route(&plan->launch.peers, plan->launch.tma_store, blocks, dst, rows_per_block, ld, first_block,
                       plan->launch.M, plan->launch.swiglu ? plan->launch.N / 2 : plan->launch.N);
}

extern "C" int smb_fp4_plan_set_alpha(smb_fp4_plan* plan, float alpha) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null handle");
  if (!plan->launch.block16)
    return set_error(SMB_ERR_UNSUPPORTED, "fp4 plan: the output factor belongs to block-16 plans");
  plan->launch.alpha = alpha;
  plan->dlaunch.alpha = alpha;
  return SMB_OK;
}

extern "C" int smb_fp4_plan_set_profile(smb_fp4_plan* plan, long long* counters) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null handle");
  plan->launch.prof = counters;
  return SMB_OK;
}

extern "C" int smb_fp4_plan_create_bf16_activations(smb_fp4_plan** out, const void* x_bf16, int64_t ldx,
                                                    const void* b, const void* sfb, void* d, int M, int N,
                                                    int K, int64_t ldb_bytes, int64_t ldd, unsigned flags) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null output handle");
  *out = nullptr;
  if (x_bf16 == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null activation pointer");
  if (flags & SMB_FLAG_SCALE_BLOCK16)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "fp4 plan: the chained activation quantiser produces UE8M0 scales per 32 K only");
  if (M <= 0 || K <= 0 || K % 32 != 0)
    return set_error(SMB_ERR_INVALID, "fp4 plan: bad activation shape (K must be a multiple of 32)");
  if (ldx < K || ldx % 8 != 0 || reinterpret_cast<uintptr_t>(x_bf16) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "fp4 plan: activation rows must be 16-byte aligned, pitch >= K");
  void *codes = nullptr, *sf = nullptr, *counter = nullptr;
  const size_t sf_bytes = smb_sf_packed_bytes(M, K / 32);
  cudaError_t e = cudaMalloc(&codes, static_cast<size_t>(M) * K / 2);
  if (e == cudaSuccess) e = cudaMalloc(&sf, sf_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&counter, 8);
  if (e == cudaSuccess) e = cudaMemset(counter, 0, 8);
  // Rows of the last 128-row band that no activation row fills keep the neutral scale byte.
  if (e == cudaSuccess) e = cudaMemset(sf, 127, sf_bytes);
  int rc = e == cudaSuccess ? SMB_OK : set_cuda_error(e, "fp4 plan: activation buffers");
  smb_fp4_plan* p = nullptr;
  // The quantised activations are written on the stream right before every GEMM: never static.
  if (rc == SMB_OK)
    rc = smb_fp4_plan_create(&p, codes, sf, b, sfb, d, M, N, K, K / 2, ldb_bytes, ldd,
                             flags & ~SMB_FLAG_OPERANDS_STATIC);
  if (rc != SMB_OK) {
    if (codes) cudaFree(codes);
    if (sf) cudaFree(sf);
    if (counter) cudaFree(counter);
    return rc;
  }
  p->act_src = x_bf16;
  p->act_ld = ldx;
  p->act_codes = codes;
  p->act_sf = sf;
  p->act_counter = counter;
  p->dlaunch.activations_dynamic = true;
  p->dlaunch.act_src = x_bf16;
  p->dlaunch.act_ld = ldx;
  p->dlaunch.act_codes = codes;
  p->dlaunch.act_sf = sf;
  p->dlaunch.act_counter = static_cast<unsigned long long*>(counter);
  // Default by measurement (N = 28672, K = 8192, us per step: shared by the grid / per CTA / chained):
  // M = 1 22.4 / 20.9 / 23.0, 16 22.7 / 22.3 / 23.7, 32 23.1 / 25.3 / 25.3, 64 24.1 / 27.9 / 27.9,
  // 128 26.6 / 28.7 / 29.1.
  p->dlaunch.act_mode = (flags & SMB_FLAG_ACT_QUANT_PER_CTA) ? 1 : ((flags & SMB_FLAG_ACT_QUANT_CHAINED) ? 2 : 0);
  if (!(flags & (SMB_FLAG_ACT_QUANT_PER_CTA | SMB_FLAG_ACT_QUANT_CHAINED | SMB_FLAG_ACT_QUANT_SHARED)) && M <= 16)
    p->dlaunch.act_mode = 1;
  *out = p;
  return SMB_OK;
}

extern "C" int smb_fp4_plan_run(smb_fp4_plan* plan, void* stream) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null handle");
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device != plan->device)
    return set_error(SMB_ERR_INVALID, "fp4 plan: created on device %d, run with device %d current",
                     plan->device, device);
  // Where the decode kernel quantises the BF16 activations itself there is nothing to launch first.
  if (plan->act_src != nullptr &&
      !(plan->decode && (fp4_decode_fuses_activations(plan->dlaunch) || fp4_decode_spreads_activations(plan->dlaunch)))) {
    const bool chained = !(plan->decode && plan->dlaunch.no_overlap);
    int rc = quantize_bf16_launch(plan->act_src, plan->act_ld, plan->act_codes, plan->launch.K / 2,
                                  plan->act_sf, nullptr, plan->launch.M, plan->launch.K, chained,
                                  static_cast<cudaStream_t>(stream));
    if (rc != SMB_OK) return rc;
  }
  if (plan->decode) return fp4_decode_launch(plan->dlaunch, static_cast<cudaStream_t>(stream));
  return fp4_launch(plan->launch, static_cast<cudaStream_t>(stream));
}

extern "C" int smb_fp4_plan_check(smb_fp4_plan* plan, void* stream) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null handle");
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return set_cuda_error(e, "fp4 plan check: stream synchronize");
  int status = 0;
  e = cudaMemcpy(&status, plan->status_dev, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return set_cuda_error(e, "fp4 plan check: status read");
  if (status != 0) {
    cudaMemset(plan->status_dev, 0, sizeof(int));
    // A decode launch that gave up may have left partial sums behind.
    if (plan->scratch_dev) cudaMemset(plan->scratch_dev, 0, plan->scratch_bytes);
    if (plan->act_counter) cudaMemset(plan->act_counter, 0, 8);
    return set_error(SMB_ERR_DEVICE, "nvfp4 GEMM kernel reported status %d: %s", status,
                     device_status_name(status));
  }
  return SMB_OK;
}

extern "C" int smb_fp4_plan_describe(smb_fp4_plan* plan, char* out, size_t capacity) {
  if (plan == nullptr || out == nullptr || capacity == 0)
    return set_error(SMB_ERR_INVALID, "fp4 plan describe: null argument");
  if (plan->decode) {
    const Fp4DecodeLaunch& D = plan->dlaunch;
    snprintf(out, capacity, "fp4 decode m_pad=%d %s%s%s", (D.M + 15) / 16 * 16,
             D.max_ctas > 0 ? "stream-k" : (D.dual ? "tile-pairs" : "single-tiles"), D.block16 ? " block16" : "",
             D.act_src != nullptr ? " bf16-activations" : "");
  } else {
    const Fp4Launch& L = plan->launch;
    snprintf(out, capacity, "fp4 tile 256x%d store=%s%s%s", L.w0 + L.w1,
             L.swiglu ? "swiglu" : (L.tma_store ? "tma" : "plain"), L.block16 ? " block16" : "",
             L.w0 == 192 ? " a-resident" : "");
  }
  return SMB_OK;
}

extern "C" int smb_fp4_plan_wait_probe(smb_fp4_plan* plan, long long budget_cycles, void* stream) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "fp4 plan: null handle");
  return wait_probe_launch(plan->status_dev, budget_cycles, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int smb_fp4_plan_destroy(smb_fp4_plan* plan) {
  if (plan == nullptr) return SMB_OK;
  if (plan->status_dev && plan->owns_status) cudaFree(plan->status_dev);
  if (plan->scratch_dev) cudaFree(plan->scratch_dev);
  if (plan->act_codes) cudaFree(plan->act_codes);
  if (plan->act_sf) cudaFree(plan->act_sf);
  if (plan->act_counter) cudaFree(plan->act_counter);
  if (plan->tile_table_dev) cudaFree(plan->tile_table_dev);
  delete plan;
  return SMB_OK;
}

extern "C" int smb_dense_gemm_nvfp4(const void* a, const void* sfa, const void* b, const void* sfb,
                                    void* d, int M, int N, int K, void* stream) {
  smb_fp4_plan* plan = nullptr;
  int rc = smb_fp4_plan_create(&plan, a, sfa, b, sfb, d, M, N, K, K / 2, K / 2, N, SMB_FLAG_NONE);
  if (rc != SMB_OK) return rc;
  rc = smb_fp4_plan_run(plan, stream);
  if (rc == SMB_OK) rc = smb_fp4_plan_check(plan, stream);
  smb_fp4_plan_destroy(plan);
  return rc;
}

extern "C" int smb_dense_gemm_nvfp4_host(const uint8_t* a, const uint8_t* sfa_rowmajor,
                                         const uint8_t* b, const uint8_t* sfb_rowmajor, uint16_t* d,
                                         int M, int N, int K) {
  if (a == nullptr || b == nullptr || sfa_rowmajor == nullptr || sfb_rowmajor == nullptr || d == nullptr)
    return set_error(SMB_ERR_INVALID, "host fp4 GEMM: null operand pointer");
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0)
    return set_error(SMB_ERR_INVALID, "host fp4 GEMM: bad dimensions (K must be a multiple of 32)");
  const int64_t kblocks = K / 32;
  std::vector<uint8_t> pa(smb_sf_packed_bytes(M, kblocks)), pb(smb_sf_packed_bytes(N, kblocks));
  int rc = smb_sf_pack_host(sfa_rowmajor, M, kblocks, pa.data());
  if (rc == SMB_OK) rc = smb_sf_pack_host(sfb_rowmajor, N, kblocks, pb.data());
  if (rc != SMB_OK) return rc;
  const size_t a_bytes = static_cast<size_t>(M) * K / 2;
  const size_t b_bytes = static_cast<size_t>(N) * K / 2;
  const int64_t ldd = (static_cast<int64_t>(N) + 7) / 8 * 8;
  const size_t d_bytes = static_cast<size_t>(M) * ldd * 2;
  void *da = nullptr, *db = nullptr, *dsa = nullptr, *dsb = nullptr, *dd = nullptr;
  cudaError_t e = cudaMalloc(&da, a_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&db, b_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&dsa, pa.size());
  if (e == cudaSuccess) e = cudaMalloc(&dsb, pb.size());
  if (e == cudaSuccess) e = cudaMalloc(&dd, d_bytes);
  if (e == cudaSuccess) e = cudaMemcpy(da, a, a_bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(db, b, b_bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(dsa, pa.data(), pa.size(), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaMemcpy(dsb, pb.data(), pb.size(), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) rc = set_cuda_error(e, "host fp4 GEMM: allocation or upload");
  smb_fp4_plan* plan = nullptr;
  if (rc == SMB_OK)
    rc = smb_fp4_plan_create(&plan, da, dsa, db, dsb, dd, M, N, K, K / 2, K / 2, ldd, SMB_FLAG_NONE);
  if (rc == SMB_OK) rc = smb_fp4_plan_run(plan, nullptr);
  if (rc == SMB_OK) rc = smb_fp4_plan_check(plan, nullptr);
  if (rc == SMB_OK) {
    e = cudaMemcpy2D(d, static_cast<size_t>(N) * 2, dd, static_cast<size_t>(ldd) * 2,
                     static_cast<size_t>(N) * 2, M, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) rc = set_cuda_error(e, "host fp4 GEMM: download");
  }
  smb_fp4_plan_destroy(plan);
  cudaFree(da);
  cudaFree(db);
  cudaFree(dsa);
  cudaFree(dsb);
  cudaFree(dd);
  return rc;
}

// ------------------------------------------------------------------------------------
// Host-buffer context, the FP4 twin of smb_bf16_host_ctx: device buffers, plans, streams and
// events are created once for a shape; a run uploads codes and row-major scales, packs the
// scales on the device, multiplies and downloads D.  The rows of A are cut into chunks (whole
// 128-row scale bands) so that the upload of chunk i + 1, the GEMM of chunk i and the download
// of chunk i - 1 overlap; the chunks shrink towards the end so that the last GEMM and download,
// which nothing overlaps, are short.  M <= 128 is one chunk (the decode kernel).  B and its
// scales go up first; a run given b == NULL keeps the weights of the previous run (a decode
// step: the weights stay resident, only the activations travel).
// ------------------------------------------------------------------------------------
namespace {

constexpr int kFp4HostChunkRows = 1024;
constexpr int kFp4HostChunkMinRows = 256;

int fp4_next_chunk_rows(int rows_left) {
  if (rows_left <= 128) return rows_left;
  if (rows_left >= 4 * kFp4HostChunkRows) return kFp4HostChunkRows;
  int rows = (rows_left / 4 + kFp4HostChunkMinRows - 1) / kFp4HostChunkMinRows * kFp4HostChunkMinRows;
  if (rows < kFp4HostChunkMinRows) rows = kFp4HostChunkMinRows;
  return rows < rows_left ? rows : rows_left;
}

// Row-major scale bytes [rows, kblocks] (rows row0 .. row0 + rows of the operand) into the packed
// layout of the whole operand.  Padding rows of the last band keep the neutral byte they were
// initialised with.
__global__ void sf_pack_kernel(const uint8_t* __restrict__ rowmajor, uint8_t* __restrict__ packed,
                               int64_t row0, int64_t rows, uint32_t kblocks) {
  const int64_t total = rows * kblocks;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / kblocks;
    const uint32_t j = static_cast<uint32_t>(i - r * kblocks);
    packed[fmt::sf_packed_offset(static_cast<uint32_t>(row0 + r), j, kblocks)] = rowmajor[(row0 + r) * kblocks + j];
  }
}

int sf_pack_launch(const void* rowmajor, void* packed, int64_t row0, int64_t rows, uint32_t kblocks,
                   cudaStream_t st) {
  const int64_t total = rows * kblocks;
  if (total <= 0) return SMB_OK;
  const int64_t want = (total + 255) / 256;
  const int blocks = static_cast<int>(want < 148 * 8 ? want : 148 * 8);
  sf_pack_kernel<<<blocks, 256, 0, st>>>(static_cast<const uint8_t*>(rowmajor), static_cast<uint8_t*>(packed), row0,
                                         rows, kblocks);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "scale pack launch");
  return SMB_OK;
}

}  // namespace

struct smb_fp4_host_ctx {
  int M, N, K;
  int64_t ldd;
  void *da, *db, *dsa_rm, *dsb_rm, *dsa, *dsb, *dd;
  int* status_dev;
  int* status_host;   // pinned
  bool weights_loaded;
  std::vector<smb_fp4_plan*> plans;   // one per row chunk
  std::vector<int> chunk_row0, chunk_rows;
  std::vector<cudaEvent_t> uploaded, computed;
  cudaStream_t up, compute, down;
  // Sharded form: this rank uploads only its M / world rows of A (codes and scales); the ranks
  // complete A over NVLink with all-gathers on the compute stream.
  smb_comm* comm;
  cudaEvent_t a_block_up, operands_up;
};

extern "C" int smb_fp4_host_ctx_destroy(smb_fp4_host_ctx* ctx) {
  if (ctx == nullptr) return SMB_OK;
  for (smb_fp4_plan* p : ctx->plans) smb_fp4_plan_destroy(p);
  for (cudaEvent_t e : ctx->uploaded) cudaEventDestroy(e);
  for (cudaEvent_t e : ctx->computed) cudaEventDestroy(e);
  if (ctx->a_block_up) cudaEventDestroy(ctx->a_block_up);
  if (ctx->operands_up) cudaEventDestroy(ctx->operands_up);
  void* bufs[] = {ctx->da, ctx->db, ctx->dsa_rm, ctx->dsb_rm, ctx->dsa, ctx->dsb, ctx->dd, ctx->status_dev};
  for (void* b : bufs)
    if (b) cudaFree(b);
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  if (ctx->up) cudaStreamDestroy(ctx->up);
  if (ctx->compute) cudaStreamDestroy(ctx->compute);
  if (ctx->down) cudaStreamDestroy(ctx->down);
  delete ctx;
  return SMB_OK;
}

namespace {
int fp4_host_ctx_create_impl(smb_fp4_host_ctx** out, int M, int N, int K, smb_comm* comm);
}

extern "C" int smb_fp4_host_ctx_create(smb_fp4_host_ctx** out, int M, int N, int K) {
  return fp4_host_ctx_create_impl(out, M, N, K, nullptr);
}

extern "C" int smb_fp4_host_ctx_create_sharded(smb_fp4_host_ctx** out, int M, int n_local, int K,
                                               smb_comm* comm) {
  if (comm == nullptr) return set_error(SMB_ERR_INVALID, "sharded fp4 host context: null communicator");
  if (M <= 0 || M % comm_world(comm) != 0)
    return set_error(SMB_ERR_INVALID, "sharded fp4 host context: M=%d is not divisible by %d ranks", M,
                     comm_world(comm));
  return fp4_host_ctx_create_impl(out, M, n_local, K, comm);
}

namespace {
int fp4_host_ctx_create_impl(smb_fp4_host_ctx** out, int M, int N, int K, smb_comm* comm) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "fp4 host context: null output handle");
  *out = nullptr;
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0)
    return set_error(SMB_ERR_INVALID, "fp4 host context: bad dimensions (K must be a multiple of 32)");
  smb_fp4_host_ctx* c = new (std::nothrow) smb_fp4_host_ctx();
  if (c == nullptr) return set_error(SMB_ERR_NOMEM, "fp4 host context: out of host memory");
  c->comm = comm;
  c->a_block_up = c->operands_up = nullptr;
  c->M = M;
  c->N = N;
  c->K = K;
  c->ldd = (static_cast<int64_t>(N) + 7) / 8 * 8;   // the aligned store path is always usable
  c->da = c->db = c->dsa_rm = c->dsb_rm = c->dsa = c->dsb = c->dd = nullptr;
  c->status_dev = c->status_host = nullptr;
  c->up = c->compute = c->down = nullptr;
  c->weights_loaded = false;
  const int64_t kblocks = K / 32;
  const size_t sfa_bytes = smb_sf_packed_bytes(M, kblocks), sfb_bytes = smb_sf_packed_bytes(N, kblocks);
  int rc = SMB_OK;
  cudaError_t e = cudaStreamCreateWithFlags(&c->up, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->compute, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->down, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(&c->da, static_cast<size_t>(M) * K / 2);
  if (e == cudaSuccess) e = cudaMalloc(&c->db, static_cast<size_t>(N) * K / 2);
  if (e == cudaSuccess) e = cudaMalloc(&c->dsa_rm, static_cast<size_t>(M) * kblocks);
  if (e == cudaSuccess) e = cudaMalloc(&c->dsb_rm, static_cast<size_t>(N) * kblocks);
  if (e == cudaSuccess) e = cudaMalloc(&c->dsa, sfa_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&c->dsb, sfb_bytes);
  if (e == cudaSuccess) e = cudaMemset(c->dsa, 127, sfa_bytes);
  if (e == cudaSuccess) e = cudaMemset(c->dsb, 127, sfb_bytes);
  if (e == cudaSuccess) e = cudaMalloc(&c->dd, static_cast<size_t>(M) * c->ldd * 2);
  if (e == cudaSuccess) e = cudaMalloc(&c->status_dev, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->status_dev, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost(&c->status_host, sizeof(int));
  if (e == cudaSuccess && comm != nullptr) e = cudaEventCreateWithFlags(&c->a_block_up, cudaEventDisableTiming);
  if (e == cudaSuccess && comm != nullptr) e = cudaEventCreateWithFlags(&c->operands_up, cudaEventDisableTiming);
  if (e != cudaSuccess) rc = set_cuda_error(e, "fp4 host context: allocation");
  const size_t band_bytes = static_cast<size_t>((kblocks + 3) / 4) * 512;
  for (int row0 = 0; rc == SMB_OK && row0 < M;) {
    const int rows = fp4_next_chunk_rows(M - row0);
    smb_fp4_plan* plan = nullptr;
    // A chunk's operands arrive by host copies ordered with events, never from the GEMM launched
    // before it on the stream, so consecutive chunk GEMMs may overlap.
    rc = fp4_plan_create_impl(&plan, static_cast<char*>(c->da) + static_cast<size_t>(row0) * K / 2,
                              static_cast<char*>(c->dsa) + static_cast<size_t>(row0 / 128) * band_bytes, c->db, c->dsb,
                              static_cast<char*>(c->dd) + static_cast<size_t>(row0) * c->ldd * 2, rows, N, K, K / 2,
                              K / 2, c->ldd, SMB_FLAG_OPERANDS_STATIC, 1, nullptr, c->status_dev);
    if (rc != SMB_OK) break;
    c->plans.push_back(plan);
    c->chunk_row0.push_back(row0);
    c->chunk_rows.push_back(rows);
    cudaEvent_t ev_up = nullptr, ev_done = nullptr;
    e = cudaEventCreateWithFlags(&ev_up, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ev_done, cudaEventDisableTiming);
    if (ev_up) c->uploaded.push_back(ev_up);
    if (ev_done) c->computed.push_back(ev_done);
    if (e != cudaSuccess) rc = set_cuda_error(e, "fp4 host context: event creation");
    row0 += rows;
  }
  if (rc != SMB_OK) {
    smb_fp4_host_ctx_destroy(c);
    return rc;
  }
  *out = c;
  return SMB_OK;
}
}  // namespace

namespace {
// An error in the middle of a run: nothing may still read or write the caller's buffers when the
// call returns.
int fp4_host_ctx_abort(smb_fp4_host_ctx* c, int rc) {
  cudaStreamSynchronize(c->up);
  cudaStreamSynchronize(c->compute);
  cudaStreamSynchronize(c->down);
  return rc;
}
}  // namespace

extern "C" int smb_fp4_host_ctx_run(smb_fp4_host_ctx* c, const uint8_t* a, const uint8_t* sfa_rowmajor,
                                    const uint8_t* b, const uint8_t* sfb_rowmajor, uint16_t* d) {
  if (c == nullptr) return set_error(SMB_ERR_INVALID, "fp4 host context: null handle");
  if (a == nullptr || sfa_rowmajor == nullptr || d == nullptr)
    return set_error(SMB_ERR_INVALID, "fp4 host context: null operand pointer");
  if ((b == nullptr) != (sfb_rowmajor == nullptr))
    return set_error(SMB_ERR_INVALID, "fp4 host context: B and its scales come together or not at all");
  if (b == nullptr && !c->weights_loaded)
    return set_error(SMB_ERR_INVALID, "fp4 host context: no weights from an earlier run to reuse");
  const int64_t kblocks = c->K / 32;
  const size_t row_bytes = static_cast<size_t>(c->K) / 2;
  cudaError_t e = cudaSuccess;
  int rc = SMB_OK;
  const bool sharded = c->comm != nullptr;
  if (sharded) {
    // `a` and `sfa_rowmajor` hold this rank's M / world rows.  They go up first so that the
    // all-gathers over NVLink run while B is still crossing PCIe; then all of SFA is packed.
    const size_t block_rows = static_cast<size_t>(c->M / comm_world(c->comm));
    const size_t r = static_cast<size_t>(comm_rank(c->comm));
    e = cudaMemcpyAsync(static_cast<char*>(c->da) + r * block_rows * row_bytes, a, block_rows * row_bytes,
                        cudaMemcpyHostToDevice, c->up);
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(static_cast<char*>(c->dsa_rm) + r * block_rows * kblocks, sfa_rowmajor,
                          block_rows * kblocks, cudaMemcpyHostToDevice, c->up);
    if (e == cudaSuccess) e = cudaEventRecord(c->a_block_up, c->up);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->compute, c->a_block_up, 0);
    if (e != cudaSuccess) return fp4_host_ctx_abort(c, set_cuda_error(e, "fp4 host context: upload of the A block"));
    rc = comm_allgather_inplace(c->comm, c->da, block_rows * row_bytes, c->compute);
    if (rc == SMB_OK) rc = comm_allgather_inplace(c->comm, c->dsa_rm, block_rows * kblocks, c->compute);
    if (rc == SMB_OK) rc = sf_pack_launch(c->dsa_rm, c->dsa, 0, c->M, static_cast<uint32_t>(kblocks), c->compute);
    if (rc != SMB_OK) return fp4_host_ctx_abort(c, rc);
  }
  if (b != nullptr) {
    e = cudaMemcpyAsync(c->db, b, static_cast<size_t>(c->N) * row_bytes, cudaMemcpyHostToDevice, c->up);
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(c->dsb_rm, sfb_rowmajor, static_cast<size_t>(c->N) * kblocks, cudaMemcpyHostToDevice, c->up);
    if (e != cudaSuccess) return fp4_host_ctx_abort(c, set_cuda_error(e, "fp4 host context: upload of B"));
    rc = sf_pack_launch(c->dsb_rm, c->dsb, 0, c->N, static_cast<uint32_t>(kblocks), c->up);
    if (rc != SMB_OK) return fp4_host_ctx_abort(c, rc);
    c->weights_loaded = true;
  }
  if (sharded) {
    e = cudaEventRecord(c->operands_up, c->up);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->compute, c->operands_up, 0);
    if (e != cudaSuccess) return fp4_host_ctx_abort(c, set_cuda_error(e, "fp4 host context: upload order"));
  }
  const size_t chunks = c->plans.size();
  for (size_t i = 0; i < chunks; ++i) {
    const size_t row0 = static_cast<size_t>(c->chunk_row0[i]);
    const size_t rows = static_cast<size_t>(c->chunk_rows[i]);
    if (!sharded) {
      e = cudaMemcpyAsync(static_cast<char*>(c->da) + row0 * row_bytes, a + row0 * row_bytes, rows * row_bytes,
                          cudaMemcpyHostToDevice, c->up);
      if (e == cudaSuccess)
        e = cudaMemcpyAsync(static_cast<char*>(c->dsa_rm) + row0 * kblocks, sfa_rowmajor + row0 * kblocks,
                            rows * kblocks, cudaMemcpyHostToDevice, c->up);
      if (e != cudaSuccess) return fp4_host_ctx_abort(c, set_cuda_error(e, "fp4 host context: upload of A"));
      rc = sf_pack_launch(c->dsa_rm, c->dsa, static_cast<int64_t>(row0), static_cast<int64_t>(rows),
                          static_cast<uint32_t>(kblocks), c->up);
      if (rc != SMB_OK) return fp4_host_ctx_abort(c, rc);
      e = cudaEventRecord(c->uploaded[i], c->up);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(c->compute, c->uploaded[i], 0);
      if (e != cudaSuccess) return fp4_host_ctx_abort(c, set_cuda_error(e, "fp4 host context: upload order"));
    }
    rc = smb_fp4_plan_run(c->plans[i], c->compute);
    if (rc != SMB_OK) return fp4_host_ctx_abort(c, rc);
    e = cudaEventRecord(c->computed[i], c->compute);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->down, c->computed[i], 0);
    if (e == cudaSuccess) {
      char* dst = reinterpret_cast<char*>(d) + row0 * static_cast<size_t>(c->N) * 2;
      const char* src = static_cast<char*>(c->dd) + row0 * static_cast<size_t>(c->ldd) * 2;
      if (c->ldd == c->N) {
        e = cudaMemcpyAsync(dst, src, rows * static_cast<size_t>(c->N) * 2, cudaMemcpyDeviceToHost, c->down);
      } else {
        e = cudaMemcpy2DAsync(dst, static_cast<size_t>(c->N) * 2, src, static_cast<size_t>(c->ldd) * 2,
                              static_cast<size_t>(c->N) * 2, rows, cudaMemcpyDeviceToHost, c->down);
      }
    }
    if (e != cudaSuccess) return fp4_host_ctx_abort(c, set_cuda_error(e, "fp4 host context: download of D"));
  }
  // The download stream has waited for every GEMM: the status word is final when it gets there,
  // and the next run may overwrite the operand buffers.
  e = cudaMemcpyAsync(c->status_host, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost, c->down);
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->down);
  if (e != cudaSuccess) return fp4_host_ctx_abort(c, set_cuda_error(e, "fp4 host context: synchronize"));
  const int status = *c->status_host;
  if (status != 0) {
    cudaMemset(c->status_dev, 0, sizeof(int));
    return set_error(SMB_ERR_DEVICE, "nvfp4 GEMM kernel reported status %d: %s", status, device_status_name(status));
  }
  return SMB_OK;
}
