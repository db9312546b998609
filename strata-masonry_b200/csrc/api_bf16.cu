// C-ABI of the BF16 GEMM: plans (tensor maps + tile choice), launch, status check, and the
// host-buffer convenience path.  Host-side counterpart of run_one_impl in the reference
// (src/kernels/gemm/sm100a/dense_gemm_bf16.cu:281-445).
#include <cstdio>
#include <cstdlib>
#include <new>
#include <vector>

#include "gemm_common.cuh"

namespace smb {
const char* last_error_message();
void clear_error();
const char* device_status_name(int code);
}  // namespace smb

using namespace smb;

struct smb_bf16_plan {
  Bf16Launch launch;
  int* status_dev;
  bool owns_status;
  int* tile_table_dev;   // ragged grouped plans: [3][tiles] = first row, end of group, group id
  unsigned launches;     // stream-K plans: launches so far (the flags carry the launch number)
  int device;   // the device that was current at creation: pointers and status word live there
};

extern "C" int smb_version(void) { return 1000; }

extern "C" const char* smb_last_error(void) { return last_error_message(); }

namespace smb {
const char* device_status_name(int code) {
  switch (code) {
    case 0: return "ok";
    case 101: return "load role timed out waiting for a free ring slot";
    case 102: return "MMA role timed out waiting for a filled ring slot";
    case 103: return "MMA role timed out waiting for a drained accumulator";
    case 104: return "epilogue role timed out waiting for an accumulator";
    case 105: return "a role timed out waiting for the tile scheduler";
    case 106: return "split-K fix-up timed out";
    case 107: return "bounded-wait probe ran out of budget";
    case 108: return "decode kernel timed out waiting for the activation quantiser of its grid";
    default: return "unknown device status";
  }
}
}  // namespace smb

namespace {

// `shared_status`: device status word owned by the caller (several plans reporting into one
// word), or null for a word owned by the plan.
int bf16_plan_create_impl(smb_bf16_plan** out, const void* a, const void* bt, void* d, int M, int N,
                          int K, int64_t lda, int64_t ldb, int64_t ldd, unsigned flags,
                          int* shared_status, int groups = 1, const int* mtile_group = nullptr) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "plan: null output handle");
  *out = nullptr;
  if (a == nullptr || bt == nullptr || d == nullptr)
    return set_error(SMB_ERR_INVALID, "plan: null operand pointer");
  if (M <= 0 || N <= 0 || K <= 0)
    return set_error(SMB_ERR_INVALID, "plan: dimensions must be positive (M=%d N=%d K=%d)", M, N, K);
  if (K % 8 != 0)
    return set_error(SMB_ERR_UNSUPPORTED, "plan: K=%d must be a multiple of 8 (16-byte operand rows)", K);
  const bool swiglu = (flags & SMB_FLAG_EPILOGUE_SWIGLU) != 0;
  if (swiglu && N % 2 != 0)
    return set_error(SMB_ERR_INVALID, "plan: the gated epilogue needs an even N (up/gate row pairs of BT)");
  const int n_out = swiglu ? N / 2 : N;
  if (lda < K || ldb < K || ldd < n_out)
    return set_error(SMB_ERR_INVALID, "plan: leading dimension smaller than the row length");
  if (lda % 8 != 0 || ldb % 8 != 0)
    return set_error(SMB_ERR_INVALID, "plan: lda and ldb must be multiples of 8 elements");
  if (ldd > 0x7FFFFFFFLL || lda > 0x7FFFFFFFLL || ldb > 0x7FFFFFFFLL)
    return set_error(SMB_ERR_UNSUPPORTED, "plan: leading dimensions above 2^31 - 1 elements");
  if (reinterpret_cast<uintptr_t>(d) % 2 != 0)
    return set_error(SMB_ERR_INVALID, "plan: D is not 2-byte aligned");
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return set_error(SMB_ERR_CUDA, "plan: no current CUDA device");

  smb_bf16_plan* p = new (std::nothrow) smb_bf16_plan();
  if (p == nullptr) return set_error(SMB_ERR_NOMEM, "plan: out of host memory");
  p->device = device;
  Bf16Launch& L = p->launch;
  L.M = M;
  L.N = N;
  L.K = K;
  bf16_pick_tile(M, N, K, device_cluster_slots(), &L.tile_n, &L.sub_blocks);
  if (flags & SMB_FLAG_TILE_N_512) { L.tile_n = 256; L.sub_blocks = 2; }
  if (flags & SMB_FLAG_TILE_N_256) { L.tile_n = 256; L.sub_blocks = 1; }
  if (flags & SMB_FLAG_TILE_N_128) { L.tile_n = 128; L.sub_blocks = 1; }
  if (flags & SMB_FLAG_TILE_N_64) { L.tile_n = 64; L.sub_blocks = 1; }
  L.group_m = 0;
  L.max_clusters = 0;
  // Evict-last on both operands: +1-2 % sustained on 8192^3 over no hint.  A BT too large to stay
  // in L2 between raster groups (above 256 MB) gets no hint: marked evict-last it pushes the A
  // panel of the group out (32768 x 57344 x 8192: 1344 with, 1382-1417 without, TFLOP/s sustained).
  L.l2_a = 1;
  L.l2_b = (static_cast<long long>(groups) * N * K * 2 > (256ll << 20)) ? 0 : 1;
  if (const char* env = getenv("SMB_TUNE_BF16_L2")) {   // tuning sweeps: "<a><b>", digits 0..2
    if (env[0] >= '0' && env[0] <= '2' && env[1] >= '0' && env[1] <= '2') {
      L.l2_a = env[0] - '0';
      L.l2_b = env[1] - '0';
    }
  }
  L.prof = nullptr;
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
  L.swiglu = swiglu;
  if (swiglu) {
    if (!L.tma_store) {
      delete p;
      return set_error(SMB_ERR_UNSUPPORTED,
                       "plan: the gated epilogue needs a 16-byte-aligned D with ldd %% 8 == 0");
    }
    L.tile_n = 256;   // 64 output columns per store box = 128 accumulator columns per warp
  }
  p->status_dev = nullptr;
  p->launches = 0;
  L.streamk_partial = nullptr;
  L.streamk_flags = nullptr;
  L.streamk_clusters = 0;
  L.streamk_epoch = 0;
  // Whole tiles, or K loops cut where the clusters' shares end: the second where the tiles leave
  // much of the last wave idle (or on request), for the plain GEMM with 256 x 512 tiles.
  bool streamk = (flags & SMB_FLAG_STREAM_K) != 0;
  const bool streamk_possible = L.tile_n == 256 && L.tma_store && !swiglu && mtile_group == nullptr &&
                                !L.dynamic && N > 256;
  if (streamk && !streamk_possible) {
    delete p;
    return set_error(SMB_ERR_UNSUPPORTED,
                     "plan: the stream-K walk needs N > 256, an aligned D and the plain, ungrouped GEMM");
  }
  if (!streamk && streamk_possible && L.sub_blocks == 2 && !(flags & SMB_FLAG_TILE_N_512))
    streamk = bf16_streamk_pays(M, N, K, device_cluster_slots());
  if (const char* env = getenv("SMB_TUNE_BF16_STREAMK")) {   // tuning sweeps: 0 = never
    if (env[0] == '0' && !(flags & SMB_FLAG_STREAM_K)) streamk = false;
  }
  if (streamk) L.sub_blocks = 2;

  int rc = encode_tmap_2d(&L.tmap_a, a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, K, lda * 2, 128, 64, true);
  if (rc == SMB_OK)
    rc = encode_tmap_2d(&L.tmap_b, bt, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                        static_cast<uint64_t>(groups) * N, K, ldb * 2, L.tile_n / 2, 64, true);
  if (rc == SMB_OK) {
    if (L.tma_store) {
      rc = encode_tmap_2d(&L.tmap_d, d, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, M, n_out, ldd * 2, 32, 64, true);
    } else {
      L.tmap_d = L.tmap_a;  // never dereferenced by the plain-store kernel
    }
  }
  p->owns_status = (shared_status == nullptr);
  if (rc == SMB_OK && p->owns_status) {
    cudaError_t e = cudaMalloc(&p->status_dev, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(p->status_dev, 0, sizeof(int));
    if (e != cudaSuccess) rc = set_cuda_error(e, "plan: status word allocation");
  } else if (rc == SMB_OK) {
    p->status_dev = shared_status;
  }
  if (rc == SMB_OK && streamk) {
    const int slots = device_cluster_slots() > 0 ? device_cluster_slots() : 74;
    cudaError_t e = cudaMalloc(&L.streamk_partial, bf16_streamk_workspace_bytes(slots));
    if (e == cudaSuccess) e = cudaMalloc(&L.streamk_flags, bf16_streamk_flag_bytes(slots));
    if (e == cudaSuccess) e = cudaMemset(L.streamk_flags, 0, bf16_streamk_flag_bytes(slots));
    if (e != cudaSuccess) rc = set_cuda_error(e, "plan: stream-K workspace allocation");
    L.streamk_clusters = slots;
  }
  if (rc != SMB_OK) {
    if (p->status_dev && p->owns_status) cudaFree(p->status_dev);
    if (L.streamk_partial) cudaFree(L.streamk_partial);
    if (L.streamk_flags) cudaFree(L.streamk_flags);
    delete p;
    return rc;
  }
  L.status = p->status_dev;
  *out = p;
  return SMB_OK;
}

}  // namespace

extern "C" int smb_bf16_plan_create(smb_bf16_plan** out, const void* a, const void* bt, void* d,
                                    int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldd,
                                    unsigned flags) {
  return bf16_plan_create_impl(out, a, bt, d, M, N, K, lda, ldb, ldd, flags, nullptr);
}

extern "C" int smb_bf16_grouped_plan_create(smb_bf16_plan** out, const void* a, const void* bt_stacked,
                                            void* d, int M_total, int N, int K, int groups,
                                            const int* mtile_group_dev, unsigned flags) {
  if (groups < 1) return set_error(SMB_ERR_INVALID, "grouped plan: at least one group");
  if (mtile_group_dev == nullptr) return set_error(SMB_ERR_INVALID, "grouped plan: null tile-to-group map");
  if (M_total <= 0 || M_total % 256 != 0)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "grouped plan: every group's rows must be padded to a multiple of 256 (M_total=%d)", M_total);
  if (static_cast<long long>(groups) * N > 0x7FFFFFFFLL)
    return set_error(SMB_ERR_UNSUPPORTED, "grouped plan: groups * N too large");
  return bf16_plan_create_impl(out, a, bt_stacked, d, M_total, N, K, K, K, N, flags, nullptr, groups,
                               mtile_group_dev);
}

namespace smb {
// Row tiles of a grouped problem whose groups have any number of rows: group g owns rows
// [offsets[g], offsets[g + 1]) and is cut into tiles of 256 rows from its own first row; the last
// tile of a group reads on into the next group's rows (or past the end of A, where the loads
// return zeros) and stores only its own.  Builds [first row | end of group | group id] for every
// tile on the host and copies it to the device.  `align`: required multiple of every offset.
int build_group_tiles(const int* offsets, int groups, int align, int** table_dev, int* tiles_out, int* m_total) {
  if (offsets == nullptr || groups < 1) return set_error(SMB_ERR_INVALID, "grouped plan: null offsets or no group");
  if (offsets[0] != 0) return set_error(SMB_ERR_INVALID, "grouped plan: offsets must start at 0");
  std::vector<int> row0, row_end, group;
  for (int g = 0; g < groups; ++g) {
    const int lo = offsets[g], hi = offsets[g + 1];
    if (hi < lo) return set_error(SMB_ERR_INVALID, "grouped plan: offsets must not decrease (group %d)", g);
    if (lo % align != 0)
      return set_error(SMB_ERR_UNSUPPORTED, "grouped plan: group %d starts at row %d, not a multiple of %d", g, lo, align);
    for (int r = lo; r < hi; r += 256) {
      row0.push_back(r);
      row_end.push_back(hi);
      group.push_back(g);
    }
  }
  const int tiles = static_cast<int>(row0.size());
  if (tiles == 0) return set_error(SMB_ERR_INVALID, "grouped plan: every group is empty");
  std::vector<int> table;
  table.insert(table.end(), row0.begin(), row0.end());
  table.insert(table.end(), row_end.begin(), row_end.end());
  table.insert(table.end(), group.begin(), group.end());
  int* dev = nullptr;
  cudaError_t e = cudaMalloc(&dev, table.size() * sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpy(dev, table.data(), table.size() * sizeof(int), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    if (dev) cudaFree(dev);
    return set_cuda_error(e, "grouped plan: tile table");
  }
  *table_dev = dev;
  *tiles_out = tiles;
  *m_total = offsets[groups];
  return SMB_OK;
}
}  // namespace smb

extern "C" int smb_bf16_grouped_plan_create_offsets(smb_bf16_plan** out, const void* a, const void* bt_stacked,
                                                    void* d, int N, int K, int groups, const int* group_offsets,
                                                    unsigned flags) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "grouped plan: null output handle");
  *out = nullptr;
  if (static_cast<long long>(groups) * N > 0x7FFFFFFFLL)
    return set_error(SMB_ERR_UNSUPPORTED, "grouped plan: groups * N too large");
  int* table = nullptr;
  int tiles = 0, m_total = 0;
  int rc = build_group_tiles(group_offsets, groups, 1, &table, &tiles, &m_total);
  if (rc != SMB_OK) return rc;
  rc = bf16_plan_create_impl(out, a, bt_stacked, d, m_total, N, K, K, K,
                             (flags & SMB_FLAG_EPILOGUE_SWIGLU) ? N / 2 : N, flags, nullptr, groups, table + 2 * tiles);
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

extern "C" int smb_bf16_plan_tune(smb_bf16_plan* plan, int group_m, int max_clusters) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "plan: null handle");
  if (group_m < 0 || max_clusters < 0) return set_error(SMB_ERR_INVALID, "plan: negative tuning value");
  plan->launch.group_m = group_m;
  plan->launch.max_clusters = max_clusters;
  return SMB_OK;
}

extern "C" int smb_bf16_plan_set_peer_copies(smb_bf16_plan* plan, int count, void* const* dst,
                                             int64_t ld) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "plan: null handle");
  return set_peer_copies(&plan->launch.peers, plan->launch.tma_store, count, dst, ld,
                         plan->launch.swiglu ? plan->launch.N / 2 : plan->launch.N);
}

extern "C" int smb_bf16_plan_set_row_route(smb_bf16_plan* plan, int blocks, void* const* dst,
                                           int rows_per_block, int64_t ld, int first_block) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "plan: null handle");
  return set_row_route(&plan->launch.peers, plan->launch.tma_store, blocks, dst, rows_per_block, ld, first_block,
                       plan->launch.M, plan->launch.swiglu ? plan->launch.N / 2 : plan->launch.N);
}

extern "C" int smb_bf16_plan_set_profile(smb_bf16_plan* plan, long long* counters) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "plan: null handle");
  plan->launch.prof = counters;
  return SMB_OK;
}

extern "C" int smb_bf16_plan_run(smb_bf16_plan* plan, void* stream) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "plan: null handle");
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device != plan->device)
    return set_error(SMB_ERR_INVALID, "plan: created on device %d, run with device %d current", plan->device,
                     device);
  Bf16Launch& L = plan->launch;
  // Peer copies and row routes belong to the whole-tile kernel's epilogue.
  if (L.streamk_partial != nullptr && L.peers.count == 0 && L.peers.route_rows == 0) {
    if (++plan->launches == 0) ++plan->launches;   // 0 is what the cleared flags hold
    L.streamk_epoch = plan->launches;
    return bf16_streamk_launch(L, static_cast<cudaStream_t>(stream));
  }
  return bf16_launch(L, static_cast<cudaStream_t>(stream));
}

extern "C" int smb_bf16_plan_check(smb_bf16_plan* plan, void* stream) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "plan: null handle");
  cudaError_t e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return set_cuda_error(e, "plan check: stream synchronize");
  int status = 0;
  e = cudaMemcpy(&status, plan->status_dev, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return set_cuda_error(e, "plan check: status read");
  if (status != 0) {
    cudaMemset(plan->status_dev, 0, sizeof(int));
    return set_error(SMB_ERR_DEVICE, "bf16 GEMM kernel reported status %d: %s", status,
                     device_status_name(status));
  }
  return SMB_OK;
}

extern "C" int smb_bf16_plan_describe(smb_bf16_plan* plan, char* out, size_t capacity) {
  if (plan == nullptr || out == nullptr || capacity == 0)
    return set_error(SMB_ERR_INVALID, "plan describe: null argument");
  const Bf16Launch& L = plan->launch;
  const bool narrow_pair = L.tile_n <= 128 && L.operands_static && !L.swiglu;
  const bool streamk = L.streamk_partial != nullptr && L.peers.count == 0 && L.peers.route_rows == 0;
  snprintf(out, capacity, "bf16 tile 256x%d store=%s resident=%d%s", L.tile_n * L.sub_blocks,
           L.swiglu ? "swiglu" : (L.tma_store ? "tma" : "plain"), narrow_pair ? 2 : 1, streamk ? " stream-k" : "");
  return SMB_OK;
}

extern "C" int smb_bf16_plan_wait_probe(smb_bf16_plan* plan, long long budget_cycles, void* stream) {
  if (plan == nullptr) return set_error(SMB_ERR_INVALID, "plan: null handle");
  return wait_probe_launch(plan->status_dev, budget_cycles, nullptr, static_cast<cudaStream_t>(stream));
}

extern "C" int smb_bf16_plan_destroy(smb_bf16_plan* plan) {
  if (plan == nullptr) return SMB_OK;
  if (plan->status_dev && plan->owns_status) cudaFree(plan->status_dev);
  if (plan->tile_table_dev) cudaFree(plan->tile_table_dev);
  if (plan->launch.streamk_partial) cudaFree(plan->launch.streamk_partial);
  if (plan->launch.streamk_flags) cudaFree(plan->launch.streamk_flags);
  delete plan;
  return SMB_OK;
}

extern "C" int smb_dense_gemm_bf16(const void* a, const void* bt, void* d, int M, int N, int K,
                                   void* stream) {
  smb_bf16_plan* plan = nullptr;
  int rc = smb_bf16_plan_create(&plan, a, bt, d, M, N, K, K, K, N, SMB_FLAG_NONE);
  if (rc != SMB_OK) return rc;
  rc = smb_bf16_plan_run(plan, stream);
  if (rc == SMB_OK) rc = smb_bf16_plan_check(plan, stream);
  smb_bf16_plan_destroy(plan);
  return rc;
}

// ------------------------------------------------------------------------------------
// Host-buffer context: device buffers, plans, streams and events are created once; every
// run uploads A and BT, computes and downloads D.  The work is cut into row chunks of A
// so that the three legs overlap: while chunk i is being multiplied, chunk i+1 of A is on its
// way up and chunk i-1 of D on its way down (PCIe is full duplex).  BT goes up first.
// What cannot overlap is the last chunk's GEMM and download, so the chunks shrink towards the
// end: 1024 rows while much is left, then a quarter of the rest, never less than 256.
// All chunk GEMMs report into one status word, read once per run together with the last download.
// ------------------------------------------------------------------------------------
#include <vector>

namespace {
constexpr int kHostChunkRows = 1024;
constexpr int kHostChunkMinRows = 256;

int next_chunk_rows(int rows_left) {
  if (rows_left >= 4 * kHostChunkRows) return kHostChunkRows;
  int rows = (rows_left / 4 + kHostChunkMinRows - 1) / kHostChunkMinRows * kHostChunkMinRows;
  if (rows < kHostChunkMinRows) rows = kHostChunkMinRows;
  return rows < rows_left ? rows : rows_left;
}
}  // namespace

struct smb_bf16_host_ctx {
  int M, N, K;
  int64_t ldd;
  void *da, *db, *dd;
  int* status_dev;
  int* status_host;   // pinned
  std::vector<smb_bf16_plan*> plans;   // one per row chunk
  std::vector<int> chunk_row0, chunk_rows;
  std::vector<cudaEvent_t> uploaded, computed;
  cudaStream_t up, compute, down;
  // Sharded form: this rank uploads only its M / world rows of A; the ranks complete A over
  // NVLink with an all-gather on the compute stream.
  smb_comm* comm;
  cudaEvent_t a_block_up, operands_up;
};

extern "C" int smb_bf16_host_ctx_destroy(smb_bf16_host_ctx* ctx) {
  if (ctx == nullptr) return SMB_OK;
  for (smb_bf16_plan* p : ctx->plans) smb_bf16_plan_destroy(p);
  for (cudaEvent_t e : ctx->uploaded) cudaEventDestroy(e);
  for (cudaEvent_t e : ctx->computed) cudaEventDestroy(e);
  if (ctx->a_block_up) cudaEventDestroy(ctx->a_block_up);
  if (ctx->operands_up) cudaEventDestroy(ctx->operands_up);
  if (ctx->da) cudaFree(ctx->da);
  if (ctx->db) cudaFree(ctx->db);
  if (ctx->dd) cudaFree(ctx->dd);
  if (ctx->status_dev) cudaFree(ctx->status_dev);
  if (ctx->status_host) cudaFreeHost(ctx->status_host);
  if (ctx->up) cudaStreamDestroy(ctx->up);
  if (ctx->compute) cudaStreamDestroy(ctx->compute);
  if (ctx->down) cudaStreamDestroy(ctx->down);
  delete ctx;
  return SMB_OK;
}

namespace {
int bf16_host_ctx_create_impl(smb_bf16_host_ctx** out, int M, int N, int K, smb_comm* comm);
}

extern "C" int smb_bf16_host_ctx_create(smb_bf16_host_ctx** out, int M, int N, int K) {
  return bf16_host_ctx_create_impl(out, M, N, K, nullptr);
}

extern "C" int smb_bf16_host_ctx_create_sharded(smb_bf16_host_ctx** out, int M, int n_local, int K,
                                                smb_comm* comm) {
  if (comm == nullptr) return set_error(SMB_ERR_INVALID, "sharded host context: null communicator");
  if (M <= 0 || M % comm_world(comm) != 0)
    return set_error(SMB_ERR_INVALID, "sharded host context: M=%d is not divisible by %d ranks", M,
                     comm_world(comm));
  return bf16_host_ctx_create_impl(out, M, n_local, K, comm);
}

namespace {
int bf16_host_ctx_create_impl(smb_bf16_host_ctx** out, int M, int N, int K, smb_comm* comm) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "host context: null output handle");
  *out = nullptr;
  if (M <= 0 || N <= 0 || K <= 0) return set_error(SMB_ERR_INVALID, "host context: bad dimensions");
  smb_bf16_host_ctx* c = new (std::nothrow) smb_bf16_host_ctx();
  if (c == nullptr) return set_error(SMB_ERR_NOMEM, "host context: out of host memory");
  c->comm = comm;
  c->a_block_up = c->operands_up = nullptr;
  c->M = M;
  c->N = N;
  c->K = K;
  // Pad rows of D to 8 elements so that the TMA-store epilogue is always usable.
  c->ldd = (static_cast<int64_t>(N) + 7) / 8 * 8;
  c->da = c->db = c->dd = nullptr;
  c->status_dev = c->status_host = nullptr;
  c->up = c->compute = c->down = nullptr;
  int rc = SMB_OK;
  cudaError_t e = cudaStreamCreateWithFlags(&c->up, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->compute, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->down, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(&c->da, static_cast<size_t>(M) * K * 2);
  if (e == cudaSuccess) e = cudaMalloc(&c->db, static_cast<size_t>(N) * K * 2);
  if (e == cudaSuccess) e = cudaMalloc(&c->dd, static_cast<size_t>(M) * c->ldd * 2);
  if (e == cudaSuccess) e = cudaMalloc(&c->status_dev, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->status_dev, 0, sizeof(int));
  if (e == cudaSuccess) e = cudaMallocHost(&c->status_host, sizeof(int));
  if (e == cudaSuccess && comm != nullptr) e = cudaEventCreateWithFlags(&c->a_block_up, cudaEventDisableTiming);
  if (e == cudaSuccess && comm != nullptr) e = cudaEventCreateWithFlags(&c->operands_up, cudaEventDisableTiming);
  if (e != cudaSuccess) rc = set_cuda_error(e, "host context: allocation");
  for (int row0 = 0; rc == SMB_OK && row0 < M;) {
    const int rows = next_chunk_rows(M - row0);
    smb_bf16_plan* plan = nullptr;
    // The operands of a chunk's GEMM come from host copies ordered by events, never from the
    // GEMM launched before it, so consecutive chunk GEMMs may overlap.
    rc = bf16_plan_create_impl(&plan, static_cast<char*>(c->da) + static_cast<size_t>(row0) * K * 2,
                               c->db, static_cast<char*>(c->dd) + static_cast<size_t>(row0) * c->ldd * 2,
                               rows, N, K, K, K, c->ldd, SMB_FLAG_OPERANDS_STATIC, c->status_dev);
    if (rc != SMB_OK) break;
    c->plans.push_back(plan);
    c->chunk_row0.push_back(row0);
    c->chunk_rows.push_back(rows);
    cudaEvent_t ev_up = nullptr, ev_done = nullptr;
    e = cudaEventCreateWithFlags(&ev_up, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&ev_done, cudaEventDisableTiming);
    if (ev_up) c->uploaded.push_back(ev_up);
    if (ev_done) c->computed.push_back(ev_done);
    if (e != cudaSuccess) rc = set_cuda_error(e, "host context: event creation");
    row0 += rows;
  }
  if (rc != SMB_OK) {
    smb_bf16_host_ctx_destroy(c);
    return rc;
  }
  *out = c;
  return SMB_OK;
}
}  // namespace

namespace {
// An error in the middle of a run: nothing may still be reading or writing the caller's buffers
// when the call returns.
int host_ctx_abort(smb_bf16_host_ctx* c, int rc) {
  cudaStreamSynchronize(c->up);
  cudaStreamSynchronize(c->compute);
  cudaStreamSynchronize(c->down);
  return rc;
}
}  // namespace

extern "C" int smb_bf16_host_ctx_run(smb_bf16_host_ctx* c, const uint16_t* a, const uint16_t* bt,
                                     uint16_t* d) {
  if (c == nullptr) return set_error(SMB_ERR_INVALID, "host context: null handle");
  if (a == nullptr || bt == nullptr || d == nullptr)
    return set_error(SMB_ERR_INVALID, "host context: null operand pointer");
  const size_t row_bytes_a = static_cast<size_t>(c->K) * 2;
  cudaError_t e = cudaSuccess;
  const bool sharded = c->comm != nullptr;
  if (sharded) {
    // `a` holds this rank's M / world rows.  They go up first so that the all-gather over NVLink
    // runs while BT is still crossing PCIe; the GEMMs wait for both.
    const size_t block_bytes = static_cast<size_t>(c->M / comm_world(c->comm)) * row_bytes_a;
    e = cudaMemcpyAsync(static_cast<char*>(c->da) + static_cast<size_t>(comm_rank(c->comm)) * block_bytes, a,
                        block_bytes, cudaMemcpyHostToDevice, c->up);
    if (e == cudaSuccess) e = cudaEventRecord(c->a_block_up, c->up);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->compute, c->a_block_up, 0);
    if (e != cudaSuccess) return host_ctx_abort(c, set_cuda_error(e, "host context: upload of the A block"));
    int rc = comm_allgather_inplace(c->comm, c->da, block_bytes, c->compute);
    if (rc != SMB_OK) return host_ctx_abort(c, rc);
  }
  e = cudaMemcpyAsync(c->db, bt, static_cast<size_t>(c->N) * c->K * 2, cudaMemcpyHostToDevice, c->up);
  if (e != cudaSuccess) return host_ctx_abort(c, set_cuda_error(e, "host context: upload of BT"));
  if (sharded) {
    e = cudaEventRecord(c->operands_up, c->up);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->compute, c->operands_up, 0);
    if (e != cudaSuccess) return host_ctx_abort(c, set_cuda_error(e, "host context: upload order"));
  }
  const size_t chunks = c->plans.size();
  for (size_t i = 0; i < chunks; ++i) {
    const size_t row0 = static_cast<size_t>(c->chunk_row0[i]);
    const size_t rows = static_cast<size_t>(c->chunk_rows[i]);
    if (!sharded) {
      e = cudaMemcpyAsync(static_cast<char*>(c->da) + row0 * row_bytes_a,
                          reinterpret_cast<const char*>(a) + row0 * row_bytes_a, rows * row_bytes_a,
                          cudaMemcpyHostToDevice, c->up);
      if (e == cudaSuccess) e = cudaEventRecord(c->uploaded[i], c->up);
      if (e == cudaSuccess) e = cudaStreamWaitEvent(c->compute, c->uploaded[i], 0);
    }
    if (e != cudaSuccess) return host_ctx_abort(c, set_cuda_error(e, "host context: upload of A"));
    int rc = smb_bf16_plan_run(c->plans[i], c->compute);
    if (rc != SMB_OK) return host_ctx_abort(c, rc);
    e = cudaEventRecord(c->computed[i], c->compute);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->down, c->computed[i], 0);
    if (e == cudaSuccess) {
      char* dst = reinterpret_cast<char*>(d) + row0 * static_cast<size_t>(c->N) * 2;
      const char* src = static_cast<char*>(c->dd) + row0 * static_cast<size_t>(c->ldd) * 2;
      if (c->ldd == c->N) {
        e = cudaMemcpyAsync(dst, src, rows * static_cast<size_t>(c->N) * 2, cudaMemcpyDeviceToHost,
                            c->down);
      } else {
        e = cudaMemcpy2DAsync(dst, static_cast<size_t>(c->N) * 2, src,
                              static_cast<size_t>(c->ldd) * 2, static_cast<size_t>(c->N) * 2, rows,
                              cudaMemcpyDeviceToHost, c->down);
      }
    }
    if (e != cudaSuccess) return host_ctx_abort(c, set_cuda_error(e, "host context: download of D"));
  }
  // The download stream has waited for every GEMM: the status word is final when it gets there.
  e = cudaMemcpyAsync(c->status_host, c->status_dev, sizeof(int), cudaMemcpyDeviceToHost, c->down);
  if (e == cudaSuccess) e = cudaStreamSynchronize(c->down);
  if (e != cudaSuccess) return host_ctx_abort(c, set_cuda_error(e, "host context: synchronize"));
  // The next run overwrites A and BT on the upload stream: every GEMM must be done by then (it
  // is: the download stream waited for all of them).
  const int status = *c->status_host;
  if (status != 0) {
    cudaMemset(c->status_dev, 0, sizeof(int));
    return set_error(SMB_ERR_DEVICE, "bf16 GEMM kernel reported status %d: %s", status,
                     device_status_name(status));
  }
  return SMB_OK;
}

extern "C" int smb_dense_gemm_bf16_host(const uint16_t* a, const uint16_t* bt, uint16_t* d, int M,
                                        int N, int K) {
  if (a == nullptr || bt == nullptr || d == nullptr)
    return set_error(SMB_ERR_INVALID, "host GEMM: null operand pointer");
  smb_bf16_host_ctx* ctx = nullptr;
  int rc = smb_bf16_host_ctx_create(&ctx, M, N, K);
  if (rc != SMB_OK) return rc;
  rc = smb_bf16_host_ctx_run(ctx, a, bt, d);
  smb_bf16_host_ctx_destroy(ctx);
  return rc;
}
