// Input generators on the device and on the host (bit-identical by construction: both call
// the same functions of formats.cuh).  The reference fills operands on the host with a
// single thread (dense_gemm_bf16.cu:298-304); at the 32768 x 57344 x 8192 size that takes
// minutes, so the drivers here generate on the device.
#include "formats.cuh"
#include "gemm_common.cuh"

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
