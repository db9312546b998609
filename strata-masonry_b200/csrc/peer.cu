// Multi-GPU plumbing of the column-sharded GEMM: device memory that the other processes of the
// box can map (CUDA IPC), and the copy that turns an all-gathered [g, M, N/g] buffer into
// row-major [M, N].  The reference is single-GPU; nothing here has a counterpart there.
#include <cstring>

#include "gemm_common.cuh"

using namespace smb;

static_assert(sizeof(cudaIpcMemHandle_t) == SMB_PEER_HANDLE_BYTES, "handle size of the C ABI");

extern "C" int smb_peer_alloc(void** ptr, size_t bytes) {
  if (ptr == nullptr || bytes == 0) return set_error(SMB_ERR_INVALID, "peer alloc: bad arguments");
  *ptr = nullptr;
  // cudaMalloc, not a pool: only whole cudaMalloc allocations can be exported.
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return set_cuda_error(e, "peer alloc");
  return SMB_OK;
}

extern "C" int smb_peer_export(void* ptr, unsigned char handle[SMB_PEER_HANDLE_BYTES]) {
  if (ptr == nullptr || handle == nullptr) return set_error(SMB_ERR_INVALID, "peer export: null argument");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return set_cuda_error(e, "peer export");
  std::memcpy(handle, &h, sizeof(h));
  return SMB_OK;
}

extern "C" int smb_peer_open(const unsigned char handle[SMB_PEER_HANDLE_BYTES], void** ptr) {
  if (ptr == nullptr || handle == nullptr) return set_error(SMB_ERR_INVALID, "peer open: null argument");
  *ptr = nullptr;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return set_cuda_error(e, "peer open");
  return SMB_OK;
}

extern "C" int smb_peer_close(void* ptr) {
  if (ptr == nullptr) return SMB_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return set_cuda_error(e, "peer close");
  return SMB_OK;
}

extern "C" int smb_peer_free(void* ptr) {
  if (ptr == nullptr) return SMB_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return set_cuda_error(e, "peer free");
  return SMB_OK;
}

extern "C" int smb_device_synchronize(void) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return set_cuda_error(e, "device synchronize");
  return SMB_OK;
}

namespace {

// One 16-byte chunk per thread and step: chunk c of output row m comes from slab c / chunks_local.
// HBM-bound copy: 2 * M * N * 2 bytes moved; consecutive threads read and write consecutive
// chunks (a slab row is n_local * 2 >= 16 contiguous bytes on the read side).
__global__ void __launch_bounds__(256) unshard_columns_kernel(const uint4* __restrict__ gathered,
                                                              uint4* __restrict__ d, int g, int M,
                                                              int chunks_local, long long ld_chunks) {
  const long long chunks_row = static_cast<long long>(g) * chunks_local;
  const long long total = static_cast<long long>(M) * chunks_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long long m = i / chunks_row;
    const int c = static_cast<int>(i - m * chunks_row);
    const int r = c / chunks_local;
    const int cl = c - r * chunks_local;
    d[m * ld_chunks + c] = gathered[(static_cast<long long>(r) * M + m) * chunks_local + cl];
  }
}

}  // namespace

namespace {

// D[i] = bf16_rne( sum over the `count` slots, in slot order, of slot[s][i] ), fp32 accumulation.
// Eight bf16 per thread and step.  HBM-bound: (count + 1) * elems * 2 bytes moved.
__global__ void __launch_bounds__(256) sum_slots_bf16_kernel(const uint4* __restrict__ slots,
                                                             uint4* __restrict__ d, int count,
                                                             long long chunks_per_slot) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < chunks_per_slot;
       i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < count; ++s) {
      const uint4 q = slots[static_cast<long long>(s) * chunks_per_slot + i];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        acc[2 * t] += __uint_as_float(w[t] << 16);
        acc[2 * t + 1] += __uint_as_float(w[t] & 0xFFFF0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int t = 0; t < 4; ++t) {
      asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(o[t]) : "f"(acc[2 * t + 1]), "f"(acc[2 * t]));
    }
    d[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace

extern "C" int smb_sum_slots_bf16_device(const void* slots, void* d, int count, int64_t elems, void* stream) {
  if (slots == nullptr || d == nullptr) return set_error(SMB_ERR_INVALID, "sum slots: null pointer");
  if (count <= 0 || elems <= 0 || elems % 8 != 0)
    return set_error(SMB_ERR_INVALID, "sum slots: count and elems must be positive, elems a multiple of 8");
  if (reinterpret_cast<uintptr_t>(slots) % 16 != 0 || reinterpret_cast<uintptr_t>(d) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "sum slots: buffers must be 16-byte aligned");
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return set_error(SMB_ERR_CUDA, "sum slots: no CUDA device");
  const long long chunks = elems / 8;
  long long blocks = (chunks + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 8;
  if (blocks > cap) blocks = cap;
  sum_slots_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(slots), static_cast<uint4*>(d), count, chunks);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "sum slots launch");
  return SMB_OK;
}

extern "C" int smb_unshard_columns_device(const void* gathered, void* d, int g, int M, int n_local,
                                          int64_t ldd, void* stream) {
  if (gathered == nullptr || d == nullptr) return set_error(SMB_ERR_INVALID, "unshard: null pointer");
  if (g <= 0 || M <= 0 || n_local <= 0) return set_error(SMB_ERR_INVALID, "unshard: bad dimensions");
  if (n_local % 8 != 0 || ldd % 8 != 0 || ldd < static_cast<int64_t>(g) * n_local)
    return set_error(SMB_ERR_INVALID, "unshard: n_local and ldd must be multiples of 8, ldd >= g * n_local");
  if (reinterpret_cast<uintptr_t>(gathered) % 16 != 0 || reinterpret_cast<uintptr_t>(d) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "unshard: buffers must be 16-byte aligned");
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return set_error(SMB_ERR_CUDA, "unshard: no CUDA device");
  const long long total = static_cast<long long>(M) * g * (n_local / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(sms) * 8;   // a multiple of the SM count
  if (blocks > cap) blocks = cap;
  unshard_columns_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(gathered), static_cast<uint4*>(d), g, M, n_local / 8, ldd / 8);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "unshard launch");
  return SMB_OK;
}
