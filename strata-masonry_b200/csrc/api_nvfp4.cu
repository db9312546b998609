// C-ABI of the block-scaled FP4 GEMM: plans, launch, status check, host-buffer path.
// Host-side counterpart of run_one_k1 in the reference
// (src/kernels/gemm/sm100a/nvfp4/dense_gemm_nvfp4.cu:2353-2700).
#include <new>
#include <vector>

#include "formats.cuh"
#include "gemm_common.cuh"

namespace smb {
const char* device_status_name(int code);
}

using namespace smb;

struct smb_fp4_plan {
  Fp4Launch launch;
  int* status_dev;
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
};

namespace {

int fp4_plan_create_impl(smb_fp4_plan** out, const void* a, const void* sfa, const void* b, const void* sfb,
                         void* d, int M, int N, int K, int64_t lda_bytes, int64_t ldb_bytes, int64_t ldd,
                         unsigned flags, int groups, const int* mtile_group) {
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
  if (swiglu && (N % 2 != 0 || (M <= 128 && !(flags & SMB_FLAG_NO_DECODE))))
    return set_error(SMB_ERR_UNSUPPORTED,
                     "fp4 plan: the gated epilogue needs an even N and the tiled kernel (M > 128)");
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
  L.group_m = 0;
  L.max_clusters = 0;
  L.prof = nullptr;
  L.prefetch = 0;
  L.dynamic = (flags & SMB_FLAG_DYNAMIC_TILES) != 0;
  L.operands_static = (flags & (SMB_FLAG_OPERANDS_STATIC | SMB_FLAG_LAUNCH_INDEPENDENT)) != 0;
  L.output_independent = (flags & SMB_FLAG_LAUNCH_INDEPENDENT) != 0;
  L.peers.count = 0;
  L.peers.route_rows = 0;
  L.peers.first_block = 0;
  L.mtile_group = mtile_group;
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
  L.swiglu = swiglu;
  if (swiglu) {
    if (!L.tma_store) {
      delete p;
      return set_error(SMB_ERR_UNSUPPORTED,
                       "fp4 plan: the gated epilogue needs a 16-byte-aligned D with ldd %% 8 == 0");
    }
    L.w0 = 256;
    L.w1 = 0;
  }
  p->status_dev = nullptr;
  p->decode = (M <= 128) && !(flags & SMB_FLAG_NO_DECODE) && mtile_group == nullptr;
  p->scratch_dev = nullptr;
  p->scratch_bytes = 0;
  p->act_src = nullptr;
  p->act_ld = 0;
  p->act_codes = p->act_sf = nullptr;

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
                        kchunks * 512, tile_n / 128, sf_box, false);
  if (rc == SMB_OK) {
    if (L.tma_store)
      rc = encode_tmap_2d(&L.tmap_d, d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, n_out, ldd * 2, 32, 64, true);
    else
      L.tmap_d = L.tmap_a;
  }
  if (rc == SMB_OK) {
    cudaError_t e = cudaMalloc(&p->status_dev, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(p->status_dev, 0, sizeof(int));
    if (e != cudaSuccess) rc = set_cuda_error(e, "fp4 plan: status word allocation");
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
    D.dual = fp4_decode_prefers_dual(M);
    if (flags & SMB_FLAG_DECODE_DUAL) D.dual = true;
    // Asked for by name, the dual form keeps its operands swapped for every M (no wide form).
    D.narrow = (flags & SMB_FLAG_DECODE_DUAL) != 0;
    D.act_src = nullptr;
    D.act_ld = 0;
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
    if (p->status_dev) cudaFree(p->status_dev);
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
  void *codes = nullptr, *sf = nullptr;
  const size_t sf_bytes = smb_sf_packed_bytes(M, K / 32);
  cudaError_t e = cudaMalloc(&codes, static_cast<size_t>(M) * K / 2);
  if (e == cudaSuccess) e = cudaMalloc(&sf, sf_bytes);
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
    return rc;
  }
  p->act_src = x_bf16;
  p->act_ld = ldx;
  p->act_codes = codes;
  p->act_sf = sf;
  p->dlaunch.activations_dynamic = true;
  p->dlaunch.act_src = x_bf16;
  p->dlaunch.act_ld = ldx;
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
  if (plan->act_src != nullptr && !(plan->decode && fp4_decode_fuses_activations(plan->dlaunch))) {
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
    return set_error(SMB_ERR_DEVICE, "nvfp4 GEMM kernel reported status %d: %s", status,
                     device_status_name(status));
  }
  return SMB_OK;
}

extern "C" int smb_fp4_plan_destroy(smb_fp4_plan* plan) {
  if (plan == nullptr) return SMB_OK;
  if (plan->status_dev) cudaFree(plan->status_dev);
  if (plan->scratch_dev) cudaFree(plan->scratch_dev);
  if (plan->act_codes) cudaFree(plan->act_codes);
  if (plan->act_sf) cudaFree(plan->act_sf);
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
