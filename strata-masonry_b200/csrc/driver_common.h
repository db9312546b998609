// Helpers shared by the two command-line drivers.  The drivers reproduce the command-line
// contract of the reference executables of the same names (flags, stdout lines, raw bf16 dump
// file, exit codes) on top of the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/strata_masonry_b200.h"

#define DRV_CUDA(expr)                                                                      \
  do {                                                                                      \
    cudaError_t e__ = (expr);                                                               \
    if (e__ != cudaSuccess) {                                                               \
      std::fprintf(stderr, "CUDA error %s at %s:%d: %s\n", cudaGetErrorName(e__), __FILE__, \
                   __LINE__, cudaGetErrorString(e__));                                      \
      std::exit(1);                                                                         \
    }                                                                                       \
  } while (0)

#define DRV_SMB(expr)                                                                 \
  do {                                                                                \
    int rc__ = (expr);                                                                \
    if (rc__ != SMB_OK) {                                                             \
      std::fprintf(stderr, "error %d at %s:%d: %s\n", rc__, __FILE__, __LINE__,       \
                   smb_last_error());                                                 \
      std::exit(1);                                                                   \
    }                                                                                 \
  } while (0)

// Batch-mean latency of `launch` in milliseconds: warm-up launches, then timed launches between
// two events on `stream` (the reference's method: 10 + 100, mean not median, L2-warm;
// dense_gemm_bf16_benchmark.cuh:24-49 there).
template <class Launch>
double measure_mean_ms(cudaStream_t stream, Launch&& launch, int warmup = 10, int timed = 100) {
  cudaEvent_t begin, end;
  DRV_CUDA(cudaEventCreate(&begin));
  DRV_CUDA(cudaEventCreate(&end));
  for (int i = 0; i < warmup; ++i) DRV_SMB(launch());
  DRV_CUDA(cudaEventRecord(begin, stream));
  for (int i = 0; i < timed; ++i) DRV_SMB(launch());
  DRV_CUDA(cudaEventRecord(end, stream));
  DRV_CUDA(cudaStreamSynchronize(stream));
  float ms = 0.0f;
  DRV_CUDA(cudaEventElapsedTime(&ms, begin, end));
  DRV_CUDA(cudaEventDestroy(begin));
  DRV_CUDA(cudaEventDestroy(end));
  return static_cast<double>(ms) / timed;
}

inline void dump_bf16(const void* dev, size_t count, const char* path) {
  std::vector<uint16_t> host(count);
  DRV_CUDA(cudaMemcpy(host.data(), dev, count * 2, cudaMemcpyDeviceToHost));
  FILE* f = std::fopen(path, "wb");
  if (!f || std::fwrite(host.data(), 2, host.size(), f) != host.size()) {
    if (f) std::fclose(f);
    std::fprintf(stderr, "failed to write %s\n", path);
    std::exit(1);
  }
  std::fclose(f);
  std::printf("  wrote %zu BF16 values to %s\n", host.size(), path);
}

inline float bf16_bits_to_float(uint16_t h) {
  uint32_t b = static_cast<uint32_t>(h) << 16;
  float v;
  std::memcpy(&v, &b, 4);
  return v;
}

inline void write_json(const char* path, const char* kernel, int M, int N, int K, int fill,
                       double ms, double tflops, bool timed) {
  if (path == nullptr) return;
  FILE* f = std::fopen(path, "w");
  if (!f) {
    std::fprintf(stderr, "failed to write %s\n", path);
    std::exit(1);
  }
  std::fprintf(f,
               "{\"kernel\": \"%s\", \"M\": %d, \"N\": %d, \"K\": %d, \"fill\": %d, \"timed\": %s, "
               "\"mean_ms\": %.6f, \"tflops\": %.3f}\n",
               kernel, M, N, K, fill, timed ? "true" : "false", ms, tflops);
  std::fclose(f);
}

// --shard=RANK/WORLD and --device=INDEX (beyond the reference, which is single-GPU): the process
// computes and dumps the column slab D[:, n0 : n0 + n_local) of the logical [M, N] problem, with
// the operands generated from their global indices, so that the slabs of the WORLD processes of a
// box, set side by side, are the single-process output bit for bit.
struct Shard {
  int rank = 0, world = 1, device = 0;
  int n0 = 0, n_local = 0;   // set by resolve()
  bool parse(const char* arg) {
    if (std::strncmp(arg, "--shard=", 8) == 0) {
      char tail = 0;
      if (std::sscanf(arg + 8, "%d/%d%c", &rank, &world, &tail) != 2 || world < 1 || rank < 0 || rank >= world) {
        std::fprintf(stderr, "--shard must be RANK/WORLD with 0 <= RANK < WORLD\n");
        std::exit(1);
      }
      return true;
    }
    if (std::strncmp(arg, "--device=", 9) == 0) {
      char tail = 0;
      if (std::sscanf(arg + 9, "%d%c", &device, &tail) != 1 || device < 0) {
        std::fprintf(stderr, "--device must be a device index\n");
        std::exit(1);
      }
      return true;
    }
    return false;
  }
  void resolve(int N) {
    if (smb_column_shard(N, world, rank, &n0, &n_local) != SMB_OK) {
      std::fprintf(stderr, "unsupported --shard for this shape: %s\n", smb_last_error());
      std::exit(1);
    }
    if (world > 1)
      std::printf("  shard %d/%d: columns [%d, %d) of N=%d on device %d\n", rank, world, n0, n0 + n_local, N,
                  device);
  }
};
