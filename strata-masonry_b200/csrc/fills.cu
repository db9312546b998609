// Input generators on the device and on the host (bit-identical by construction: both call
// the same functions of formats.cuh).  The reference fills operands on the host with a
// single thread (dense_gemm_bf16.cu:298-304); at the 32768 x 57344 x 8192 size that takes
// minutes, so the drivers here generate on the device.
#include <cstring>

#include "formats.cuh"
#include "gemm_common.cuh"
#include "ptx.cuh"

namespace smb {

namespace {

__global__ void fill_bf16_kernel(uint16_t* out, int64_t rows, int64_t cols, int64_t ld,
                                 uint32_t index0, uint32_t rs, uint32_t cs, int fill, uint32_t seed) {
  const int64_t total = rows * cols;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / cols;
    const int64_t c = i - r * cols;
    const uint32_t index = index0 + static_cast<uint32_t>(r) * rs + static_cast<uint32_t>(c) * cs;
    out[r * ld + c] = fmt::f32_to_bf16(fmt::bf16_fill_value(index, fill, seed));
  }
}

int check_fill_args(const void* out, int64_t rows, int64_t cols, int64_t ld, int fill) {
  if (out == nullptr) return set_error(SMB_ERR_INVALID, "fill: null output pointer");
  if (rows < 0 || cols < 0 || ld < cols) return set_error(SMB_ERR_INVALID, "fill: bad extents");
  if (fill < 1 || fill > 7) return set_error(SMB_ERR_INVALID, "fill: mode %d not in 1..7", fill);
  return SMB_OK;
}

}  // namespace

}  // namespace smb

using namespace smb;

extern "C" int smb_fill_bf16_device(uint16_t* out, int64_t rows, int64_t cols, int64_t ld,
                                    uint64_t index0, uint64_t index_row_stride,
                                    uint64_t index_col_stride, int fill, uint32_t seed, void* stream) {
  if (int rc = check_fill_args(out, rows, cols, ld, fill)) return rc;
  if (rows == 0 || cols == 0) return SMB_OK;
  const int64_t total = rows * cols;
  int blocks = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  fill_bf16_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      out, rows, cols, ld, static_cast<uint32_t>(index0), static_cast<uint32_t>(index_row_stride),
      static_cast<uint32_t>(index_col_stride), fill, seed);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "bf16 fill launch");
  return SMB_OK;
}

extern "C" int smb_fill_bf16_host(uint16_t* out, int64_t rows, int64_t cols, int64_t ld,
                                  uint64_t index0, uint64_t index_row_stride,
                                  uint64_t index_col_stride, int fill, uint32_t seed) {
  if (int rc = check_fill_args(out, rows, cols, ld, fill)) return rc;
  const uint32_t i0 = static_cast<uint32_t>(index0);
  const uint32_t rs = static_cast<uint32_t>(index_row_stride);
  const uint32_t cs = static_cast<uint32_t>(index_col_stride);
  for (int64_t r = 0; r < rows; ++r) {
    for (int64_t c = 0; c < cols; ++c) {
      const uint32_t index = i0 + static_cast<uint32_t>(r) * rs + static_cast<uint32_t>(c) * cs;
      out[r * ld + c] = fmt::f32_to_bf16(fmt::bf16_fill_value(index, fill, seed));
    }
  }
  return SMB_OK;
}

// ------------------------------------------------------------------------------------
// E2M1 + UE8M0 operands
// ------------------------------------------------------------------------------------
namespace smb {
namespace {

// Codes and scale byte of one 32-element block (row `grow` of the logical operand, k-block `kb`).
SMB_HD void fp4_block(uint32_t grow, uint32_t kb, uint32_t K, int fill, int which, uint8_t* codes16,
                      uint8_t* scale_byte) {
  const uint32_t seed = which == 0 ? fmt::kSeedFp4A : fmt::kSeedFp4B;
  const uint32_t base = grow * K + kb * 32u;
  uint32_t codes[32];
  int e;
  if (fill <= 4) {
    for (int i = 0; i < 32; ++i) codes[i] = fmt::fp4_fill_code(base + i, fill, seed);
    e = fmt::fp4_fill_scale_exp(grow, kb, fill, which);
  } else {
    float v[32];
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i) {
      v[i] = fmt::fp4_source_value(base + i, fill, seed);
      const float a = v[i] < 0.0f ? -v[i] : v[i];
      amax = a > amax ? a : amax;
    }
    e = fmt::ue8m0_exponent(amax);
    const float inv = fmt::exp2i(-e);
    for (int i = 0; i < 32; ++i) codes[i] = fmt::e2m1_encode(fmt::mul_rn(v[i], inv));
  }
  for (int i = 0; i < 16; ++i)
    codes16[i] = static_cast<uint8_t>(codes[2 * i] | (codes[2 * i + 1] << 4));
  *scale_byte = static_cast<uint8_t>(e + 127);
}

// Quantise one block of 32 fp32 values (formats.cuh).
SMB_HD void quantize_block(const float* v, uint8_t* codes16, uint8_t* scale_byte) {
  fmt::quantize_mx_block(v, codes16, scale_byte);
}

__global__ void fill_fp4_kernel(uint8_t* data, int64_t ld_bytes, uint8_t* sf_packed,
                                uint8_t* sf_rowmajor, int64_t rows, uint32_t K, uint32_t row0,
                                int fill, int which) {
  const uint32_t kblocks = K / 32u;
  const int64_t total = rows * kblocks;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / kblocks;
    const uint32_t kb = static_cast<uint32_t>(i - r * kblocks);
    uint8_t codes[16];
    uint8_t sb;
    fp4_block(row0 + static_cast<uint32_t>(r), kb, K, fill, which, codes, &sb);
    uint4 packed;
    memcpy(&packed, codes, 16);
    *reinterpret_cast<uint4*>(data + r * ld_bytes + kb * 16) = packed;
    if (sf_packed) sf_packed[fmt::sf_packed_offset(static_cast<uint32_t>(r), kb, kblocks)] = sb;
    if (sf_rowmajor) sf_rowmajor[r * kblocks + kb] = sb;
  }
}

__global__ void quantize_mx_kernel(const float* src, int64_t ld_src, uint8_t* data, int64_t ld_bytes,
                                   uint8_t* sf_packed, uint8_t* sf_rowmajor, int64_t rows, uint32_t K) {
  const uint32_t kblocks = K / 32u;
  const int64_t total = rows * kblocks;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / kblocks;
    const uint32_t kb = static_cast<uint32_t>(i - r * kblocks);
    float v[32];
    const float4* s4 = reinterpret_cast<const float4*>(src + r * ld_src + kb * 32);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float4 q = s4[j];
      v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
    }
    uint8_t codes[16];
    uint8_t sb;
    quantize_block(v, codes, &sb);
    uint4 packed;
    memcpy(&packed, codes, 16);
    *reinterpret_cast<uint4*>(data + r * ld_bytes + kb * 16) = packed;
    if (sf_packed) sf_packed[fmt::sf_packed_offset(static_cast<uint32_t>(r), kb, kblocks)] = sb;
    if (sf_rowmajor) sf_rowmajor[r * kblocks + kb] = sb;
  }
}

// BF16 source (the activations a model hands to the decode GEMM).  `chained`: launched with
// programmatic stream serialisation in front of a GEMM; lets the GEMM start its weight loads at
// once and itself waits for the previous kernel on the stream (which may still read the codes
// and scales this kernel overwrites) before it writes anything.
__global__ void quantize_mx_bf16_kernel(const uint16_t* src, int64_t ld_src, uint8_t* data,
                                        int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor,
                                        int64_t rows, uint32_t K, int chained) {
  if (chained) {
    griddep_launch_dependents();
    griddep_wait();
  }
  const uint32_t kblocks = K / 32u;
  const int64_t total = rows * kblocks;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / kblocks;
    const uint32_t kb = static_cast<uint32_t>(i - r * kblocks);
    float v[32];
    const uint4* s4 = reinterpret_cast<const uint4*>(src + r * ld_src + kb * 32);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 q = s4[j];
      const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        v[8 * j + 2 * t] = __uint_as_float(w[t] << 16);
        v[8 * j + 2 * t + 1] = __uint_as_float(w[t] & 0xFFFF0000u);
      }
    }
    uint8_t codes[16];
    uint8_t sb;
    quantize_block(v, codes, &sb);
    uint4 packed;
    memcpy(&packed, codes, 16);
    *reinterpret_cast<uint4*>(data + r * ld_bytes + kb * 16) = packed;
    if (sf_packed) sf_packed[fmt::sf_packed_offset(static_cast<uint32_t>(r), kb, kblocks)] = sb;
    if (sf_rowmajor) sf_rowmajor[r * kblocks + kb] = sb;
  }
}

// NVFP4 proper: one thread per 16-value block (64 bytes in, 8 + 1 bytes out).
__global__ void quantize_nvf4_kernel(const float* src, int64_t ld_src, float gs, uint8_t* data,
                                     int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor,
                                     int64_t rows, uint32_t K) {
  const uint32_t kblocks = K / 16u;
  const int64_t total = rows * kblocks;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / kblocks;
    const uint32_t kb = static_cast<uint32_t>(i - r * kblocks);
    float v[16];
    const float4* s4 = reinterpret_cast<const float4*>(src + r * ld_src + kb * 16);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 q = s4[j];
      v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
    }
    uint8_t codes[8];
    uint8_t sb;
    fmt::quantize_nvf4_block(v, gs, codes, &sb);
    uint2 packed;
    memcpy(&packed, codes, 8);
    *reinterpret_cast<uint2*>(data + r * ld_bytes + kb * 8) = packed;
    if (sf_packed) sf_packed[fmt::sf_packed_offset(static_cast<uint32_t>(r), kb, kblocks)] = sb;
    if (sf_rowmajor) sf_rowmajor[r * kblocks + kb] = sb;
  }
}

int check_fp4_args(const void* data, int64_t rows, int64_t K, int64_t ld_bytes) {
  if (data == nullptr) return set_error(SMB_ERR_INVALID, "fp4: null data pointer");
  if (rows < 0 || K <= 0 || K % 32 != 0)
    return set_error(SMB_ERR_INVALID, "fp4: K=%lld must be a positive multiple of 32",
                     static_cast<long long>(K));
  if (ld_bytes < K / 2 || ld_bytes % 16 != 0 || reinterpret_cast<uintptr_t>(data) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "fp4: data rows must be 16-byte aligned and at least K/2 bytes");
  return SMB_OK;
}

int grid_for(int64_t total) {
  const int64_t b = (total + 255) / 256;
  return static_cast<int>(b < 148 * 16 ? (b > 0 ? b : 1) : 148 * 16);
}

}  // namespace

int quantize_bf16_launch(const void* src, int64_t ld_src, void* data, int64_t ld_bytes, void* sf_packed,
                         void* sf_rowmajor, int64_t rows, int64_t K, bool chained, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid_for(rows * (K / 32))), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute pdl;
  pdl.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &pdl;
  cfg.numAttrs = chained ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, quantize_mx_bf16_kernel, static_cast<const uint16_t*>(src), ld_src,
                                     static_cast<uint8_t*>(data), ld_bytes, static_cast<uint8_t*>(sf_packed),
                                     static_cast<uint8_t*>(sf_rowmajor), rows, static_cast<uint32_t>(K),
                                     chained ? 1 : 0);
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "bf16 quantize launch");
  return SMB_OK;
}

}  // namespace smb

extern "C" size_t smb_sf_packed_bytes(int64_t rows, int64_t kblocks) {
  if (rows <= 0 || kblocks <= 0) return 0;
  return fmt::sf_packed_bytes(static_cast<uint64_t>(rows), static_cast<uint64_t>(kblocks));
}

extern "C" int smb_sf_pack_host(const uint8_t* sf_rowmajor, int64_t rows, int64_t kblocks,
                                uint8_t* packed) {
  if (sf_rowmajor == nullptr || packed == nullptr || rows <= 0 || kblocks <= 0)
    return set_error(SMB_ERR_INVALID, "sf_pack: bad arguments");
  memset(packed, 127, smb_sf_packed_bytes(rows, kblocks));
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < kblocks; ++j)
      packed[fmt::sf_packed_offset(static_cast<uint32_t>(r), static_cast<uint32_t>(j),
                                   static_cast<uint32_t>(kblocks))] = sf_rowmajor[r * kblocks + j];
  return SMB_OK;
}

extern "C" int smb_fill_fp4_host(uint8_t* data, int64_t ld_bytes, uint8_t* sf_packed,
                                 uint8_t* sf_rowmajor, int64_t rows, int64_t K, uint64_t row0,
                                 int fill, int which) {
  if (int rc = check_fp4_args(data, rows, K, ld_bytes)) return rc;
  if (fill < 1 || fill > 6) return set_error(SMB_ERR_INVALID, "fp4 fill: mode %d not in 1..6", fill);
  if (which != 0 && which != 1) return set_error(SMB_ERR_INVALID, "fp4 fill: operand must be 0 (A) or 1 (B)");
  const uint32_t kblocks = static_cast<uint32_t>(K / 32);
  if (sf_packed) memset(sf_packed, 127, smb_sf_packed_bytes(rows, kblocks));
  for (int64_t r = 0; r < rows; ++r) {
    for (uint32_t kb = 0; kb < kblocks; ++kb) {
      uint8_t sb;
      fp4_block(static_cast<uint32_t>(row0) + static_cast<uint32_t>(r), kb, static_cast<uint32_t>(K),
                fill, which, data + r * ld_bytes + kb * 16, &sb);
      if (sf_packed) sf_packed[fmt::sf_packed_offset(static_cast<uint32_t>(r), kb, kblocks)] = sb;
      if (sf_rowmajor) sf_rowmajor[r * kblocks + kb] = sb;
    }
  }
  return SMB_OK;
}

extern "C" int smb_fill_fp4_device(uint8_t* data, int64_t ld_bytes, uint8_t* sf_packed,
                                   uint8_t* sf_rowmajor, int64_t rows, int64_t K, uint64_t row0,
                                   int fill, int which, void* stream) {
  if (int rc = check_fp4_args(data, rows, K, ld_bytes)) return rc;
  if (fill < 1 || fill > 6) return set_error(SMB_ERR_INVALID, "fp4 fill: mode %d not in 1..6", fill);
  if (which != 0 && which != 1) return set_error(SMB_ERR_INVALID, "fp4 fill: operand must be 0 (A) or 1 (B)");
  if (rows == 0) return SMB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t kblocks = K / 32;
  if (sf_packed) {
    cudaError_t e = cudaMemsetAsync(sf_packed, 127, smb_sf_packed_bytes(rows, kblocks), st);
    if (e != cudaSuccess) return set_cuda_error(e, "fp4 fill: scale buffer memset");
  }
  fill_fp4_kernel<<<grid_for(rows * kblocks), 256, 0, st>>>(data, ld_bytes, sf_packed, sf_rowmajor, rows,
                                                            static_cast<uint32_t>(K),
                                                            static_cast<uint32_t>(row0), fill, which);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "fp4 fill launch");
  return SMB_OK;
}

extern "C" int smb_quantize_mx_host(const float* src, int64_t ld_src, uint8_t* data, int64_t ld_bytes,
                                    uint8_t* sf_packed, uint8_t* sf_rowmajor, int64_t rows, int64_t K) {
  if (src == nullptr) return set_error(SMB_ERR_INVALID, "quantize: null source");
  if (int rc = check_fp4_args(data, rows, K, ld_bytes)) return rc;
  if (ld_src < K) return set_error(SMB_ERR_INVALID, "quantize: source pitch smaller than K");
  const uint32_t kblocks = static_cast<uint32_t>(K / 32);
  if (sf_packed) memset(sf_packed, 127, smb_sf_packed_bytes(rows, kblocks));
  for (int64_t r = 0; r < rows; ++r) {
    for (uint32_t kb = 0; kb < kblocks; ++kb) {
      uint8_t sb;
      quantize_block(src + r * ld_src + kb * 32, data + r * ld_bytes + kb * 16, &sb);
      if (sf_packed) sf_packed[fmt::sf_packed_offset(static_cast<uint32_t>(r), kb, kblocks)] = sb;
      if (sf_rowmajor) sf_rowmajor[r * kblocks + kb] = sb;
    }
  }
  return SMB_OK;
}

extern "C" int smb_quantize_mx_device(const float* src, int64_t ld_src, uint8_t* data,
                                      int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor,
                                      int64_t rows, int64_t K, void* stream) {
  if (src == nullptr) return set_error(SMB_ERR_INVALID, "quantize: null source");
  if (int rc = check_fp4_args(data, rows, K, ld_bytes)) return rc;
  if (ld_src < K || ld_src % 4 != 0 || reinterpret_cast<uintptr_t>(src) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "quantize: source rows must be 16-byte aligned");
  if (rows == 0) return SMB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t kblocks = K / 32;
  if (sf_packed) {
    cudaError_t e = cudaMemsetAsync(sf_packed, 127, smb_sf_packed_bytes(rows, kblocks), st);
    if (e != cudaSuccess) return set_cuda_error(e, "quantize: scale buffer memset");
  }
  quantize_mx_kernel<<<grid_for(rows * kblocks), 256, 0, st>>>(src, ld_src, data, ld_bytes, sf_packed,
                                                               sf_rowmajor, rows, static_cast<uint32_t>(K));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "quantize launch");
  return SMB_OK;
}

extern "C" int smb_quantize_mx_bf16_device(const uint16_t* src, int64_t ld_src, uint8_t* data,
                                           int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor,
                                           int64_t rows, int64_t K, void* stream) {
  if (src == nullptr) return set_error(SMB_ERR_INVALID, "quantize: null source");
  if (int rc = check_fp4_args(data, rows, K, ld_bytes)) return rc;
  if (ld_src < K || ld_src % 8 != 0 || reinterpret_cast<uintptr_t>(src) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "quantize: source rows must be 16-byte aligned");
  if (rows == 0) return SMB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (sf_packed) {
    cudaError_t e = cudaMemsetAsync(sf_packed, 127, smb_sf_packed_bytes(rows, K / 32), st);
    if (e != cudaSuccess) return set_cuda_error(e, "quantize: scale buffer memset");
  }
  return quantize_bf16_launch(src, ld_src, data, ld_bytes, sf_packed, sf_rowmajor, rows, K, false, st);
}

extern "C" int smb_quantize_nvf4_host(const float* src, int64_t ld_src, float global_scale, uint8_t* data,
                                      int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor,
                                      int64_t rows, int64_t K) {
  if (src == nullptr) return set_error(SMB_ERR_INVALID, "quantize: null source");
  if (int rc = check_fp4_args(data, rows, K, ld_bytes)) return rc;
  if (ld_src < K) return set_error(SMB_ERR_INVALID, "quantize: source pitch smaller than K");
  if (!(global_scale > 0.0f)) return set_error(SMB_ERR_INVALID, "quantize: global scale must be positive");
  const uint32_t kblocks = static_cast<uint32_t>(K / 16);
  if (sf_packed) memset(sf_packed, 0, smb_sf_packed_bytes(rows, kblocks));
  for (int64_t r = 0; r < rows; ++r) {
    for (uint32_t kb = 0; kb < kblocks; ++kb) {
      uint8_t sb;
      fmt::quantize_nvf4_block(src + r * ld_src + kb * 16, global_scale, data + r * ld_bytes + kb * 8, &sb);
      if (sf_packed) sf_packed[fmt::sf_packed_offset(static_cast<uint32_t>(r), kb, kblocks)] = sb;
      if (sf_rowmajor) sf_rowmajor[r * kblocks + kb] = sb;
    }
  }
  return SMB_OK;
}

extern "C" int smb_quantize_nvf4_device(const float* src, int64_t ld_src, float global_scale, uint8_t* data,
                                        int64_t ld_bytes, uint8_t* sf_packed, uint8_t* sf_rowmajor,
                                        int64_t rows, int64_t K, void* stream) {
  if (src == nullptr) return set_error(SMB_ERR_INVALID, "quantize: null source");
  if (int rc = check_fp4_args(data, rows, K, ld_bytes)) return rc;
  if (ld_src < K || ld_src % 4 != 0 || reinterpret_cast<uintptr_t>(src) % 16 != 0)
    return set_error(SMB_ERR_INVALID, "quantize: source rows must be 16-byte aligned");
  if (!(global_scale > 0.0f)) return set_error(SMB_ERR_INVALID, "quantize: global scale must be positive");
  if (rows == 0) return SMB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t kblocks = K / 16;
  if (sf_packed) {
    // Padding rows of the last 128-row band: scale 0 (they multiply zero-filled data).
    cudaError_t e = cudaMemsetAsync(sf_packed, 0, smb_sf_packed_bytes(rows, kblocks), st);
    if (e != cudaSuccess) return set_cuda_error(e, "quantize: scale buffer memset");
  }
  quantize_nvf4_kernel<<<grid_for(rows * kblocks), 256, 0, st>>>(src, ld_src, global_scale, data, ld_bytes,
                                                                 sf_packed, sf_rowmajor, rows,
                                                                 static_cast<uint32_t>(K));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_cuda_error(e, "nvf4 quantize launch");
  return SMB_OK;
}

// ------------------------------------------------------------------------------------
// Bit-pattern helpers exported for the host-side known-answer tests.
// ------------------------------------------------------------------------------------

extern "C" uint64_t smb_debug_smem_desc(uint32_t smem_addr, uint32_t sbo_bytes, uint32_t lbo_bytes,
                                        uint32_t swizzle_mode) {
  return smb::make_smem_desc(smem_addr, sbo_bytes, lbo_bytes, swizzle_mode);
}
extern "C" uint32_t smb_debug_idesc_bf16(int mma_m, int mma_n) { return smb::make_idesc_bf16(mma_m, mma_n); }
extern "C" uint32_t smb_debug_idesc_mxf4(int mma_m, int mma_n, uint32_t sf_id_a, uint32_t sf_id_b,
                                         int ue8m0) {
  return smb::make_idesc_mxf4(mma_m, mma_n, sf_id_a, sf_id_b, ue8m0 != 0);
}
extern "C" void smb_debug_tile_coords(int t, int tiles_m, int tiles_n, int group_m, int* tm, int* tn) {
  smb::tile_coords(t, tiles_m, tiles_n, group_m, *tm, *tn);
}
extern "C" uint64_t smb_debug_sf_offset(uint32_t row, uint32_t kblock, uint32_t kblocks) {
  return fmt::sf_packed_offset(row, kblock, kblocks);
}
