// Error plumbing and tensor-map encoding shared by every entry point.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "gemm_common.cuh"

namespace smb {

namespace {
thread_local char g_error[512] = {0};
}

const char* last_error_message() { return g_error; }
void clear_error() { g_error[0] = 0; }

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

int set_cuda_error(cudaError_t e, const char* what) {
  snprintf(g_error, sizeof(g_error), "%s: %s (%s)", what, cudaGetErrorString(e), cudaGetErrorName(e));
  return SMB_ERR_CUDA;
}

int device_cluster_slots() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return 0;
  }
  return sms / 2;
}

int set_peer_copies(PeerCopies* out, bool tma_store, int count, void* const* dst, long long ld, int N) {
  if (count < 0 || count > kMaxPeerCopies - 1)
    return set_error(SMB_ERR_INVALID, "peer copies: count %d outside 0..%d", count, kMaxPeerCopies - 1);
  out->route_rows = 0;
  out->first_block = 0;
  if (count == 0) {
    out->count = 0;
    return SMB_OK;
  }
  if (dst == nullptr) return set_error(SMB_ERR_INVALID, "peer copies: null destination list");
  if (!tma_store)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "peer copies need the 16-byte-aligned store path (D 16-byte aligned, ldd %% 8 == 0)");
  if (N % 8 != 0) return set_error(SMB_ERR_UNSUPPORTED, "peer copies: N=%d must be a multiple of 8", N);
  if (ld < N || ld % 8 != 0)
    return set_error(SMB_ERR_INVALID, "peer copies: row pitch %lld must be >= N and a multiple of 8", ld);
  for (int i = 0; i < count; ++i) {
    if (dst[i] == nullptr || reinterpret_cast<uintptr_t>(dst[i]) % 16 != 0)
      return set_error(SMB_ERR_INVALID, "peer copies: destination %d (%p) is null or not 16-byte aligned", i,
                       dst[i]);
  }
  out->count = count;
  out->ld = ld;
  for (int i = 0; i < count; ++i) out->base[i] = static_cast<uint16_t*>(dst[i]);
  return SMB_OK;
}

int set_row_route(PeerCopies* out, bool tma_store, int blocks, void* const* dst, int rows_per_block, long long ld,
                  int first_block, int M, int N) {
  if (blocks == 0) {
    out->count = 0;
    out->route_rows = 0;
    out->first_block = 0;
    return SMB_OK;
  }
  if (blocks < 0 || blocks > kMaxPeerCopies)
    return set_error(SMB_ERR_INVALID, "row route: %d blocks outside 1..%d", blocks, kMaxPeerCopies);
  if (dst == nullptr) return set_error(SMB_ERR_INVALID, "row route: null destination list");
  if (!tma_store)
    return set_error(SMB_ERR_UNSUPPORTED,
                     "row route needs the 16-byte-aligned store path (D 16-byte aligned, ldd %% 8 == 0)");
  if (rows_per_block <= 0 || rows_per_block % 256 != 0)
    return set_error(SMB_ERR_UNSUPPORTED, "row route: %d rows per block is not a multiple of 256", rows_per_block);
  if (static_cast<long long>(blocks) * rows_per_block < M)
    return set_error(SMB_ERR_INVALID, "row route: %d blocks of %d rows do not cover M=%d", blocks, rows_per_block, M);
  if (N % 8 != 0 || ld < N || ld % 8 != 0)
    return set_error(SMB_ERR_INVALID, "row route: N and the row pitch must be multiples of 8, pitch >= N");
  for (int i = 0; i < blocks; ++i) {
    if (dst[i] == nullptr || reinterpret_cast<uintptr_t>(dst[i]) % 16 != 0)
      return set_error(SMB_ERR_INVALID, "row route: destination %d (%p) is null or not 16-byte aligned", i, dst[i]);
  }
  if (first_block < 0 || first_block >= blocks)
    return set_error(SMB_ERR_INVALID, "row route: first block %d outside 0..%d", first_block, blocks - 1);
  out->count = blocks;
  out->first_block = first_block;
  out->route_rows = rows_per_block;
  out->ld = ld;
  for (int i = 0; i < blocks; ++i) out->base[i] = static_cast<uint16_t*>(dst[i]);
  return SMB_OK;
}

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up at run time so that the library links against the
// CUDA runtime only and still loads on a machine without a driver.
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn != nullptr) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || sym == nullptr) {
    (void)cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

}  // namespace

int encode_tmap_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                   uint64_t rows, uint64_t cols, uint64_t ld_bytes, uint32_t box_rows,
                   uint32_t box_cols, bool swizzle128) {
  if (base == nullptr) return set_error(SMB_ERR_INVALID, "tensor map: null base pointer");
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "tensor map: base pointer %p is not 16-byte aligned", base);
  if (ld_bytes % 16 != 0)
    return set_error(SMB_ERR_INVALID, "tensor map: row pitch %llu bytes is not a multiple of 16",
                     static_cast<unsigned long long>(ld_bytes));
  if (box_rows == 0 || box_rows > 256 || box_cols == 0 || box_cols > 256)
    return set_error(SMB_ERR_INVALID, "tensor map: box %u x %u out of range", box_rows, box_cols);
  if ((static_cast<uint64_t>(box_cols) * elem_bytes) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "tensor map: box row of %u bytes is not a multiple of 16",
                     box_cols * elem_bytes);
  if (swizzle128 && box_cols * elem_bytes != 128)
    return set_error(SMB_ERR_INVALID, "tensor map: 128-byte swizzle needs 128-byte box rows");
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr)
    return set_error(SMB_ERR_CUDA, "cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  if (const char* env = getenv("SMB_TUNE_L2_PROMO")) {   // tuning sweeps: 0, 64, 128 or 256 bytes
    const int v = atoi(env);
    promo = v == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                   : (v == 64 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                              : (v == 128 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B : CU_TENSOR_MAP_L2_PROMOTION_L2_256B));
  }
  CUresult r = fn(out, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, promo,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(SMB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return SMB_OK;
}

}  // namespace smb

extern "C" int smb_column_shard(int n_total, int world, int rank, int* n0, int* n_local) {
  using namespace smb;
  if (n0 == nullptr || n_local == nullptr) return set_error(SMB_ERR_INVALID, "column shard: null output");
  if (n_total <= 0) return set_error(SMB_ERR_INVALID, "column shard: N=%d must be positive", n_total);
  if (world < 1 || rank < 0 || rank >= world)
    return set_error(SMB_ERR_INVALID, "column shard: rank %d outside world of %d", rank, world);
  if (n_total % world != 0)
    return set_error(SMB_ERR_INVALID, "column shard: N=%d is not divisible by %d ranks", n_total, world);
  const int local = n_total / world;
  if (local % 8 != 0)
    return set_error(SMB_ERR_INVALID, "column shard: N/g=%d must be a multiple of 8 (16-byte rows of D)", local);
  *n0 = rank * local;
  *n_local = local;
  return SMB_OK;
}
