// Helpers shared by the two command-line drivers.  The drivers reproduce the command-line
// contract of the reference executables of the same names (flags, stdout lines, raw bf16 dump
// file, exit codes) on top of the C ABI.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
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

// --gpus=G [--allgather] (beyond the reference, which is single-GPU): ONE process drives G devices
// of the box; device g computes the column slab of rank g of G, exactly what G processes started
// with --shard=g/G --device=g compute.  The box time of a launch is the slowest device's.  With
// --allgather the slabs are then exchanged (smb_allgather_columns_multi: NCCL all-gather over
// NVLink + unshard copy), timed apart from the GEMM, and every device ends up with the full
// row-major D; --dump-output writes that full D (without --allgather it is assembled from the
// slabs on the host).  The dump equals the single-GPU dump bit for bit.
struct BoxOptions {
  int gpus = 0;            // 0: single-device mode
  bool allgather = false;
  bool parse(const char* arg) {
    if (std::strncmp(arg, "--gpus=", 7) == 0) {
      char tail = 0;
      if (std::sscanf(arg + 7, "%d%c", &gpus, &tail) != 1 || gpus < 1 || gpus > 64) {
        std::fprintf(stderr, "--gpus must be a device count between 1 and 64\n");
        std::exit(1);
      }
      return true;
    }
    if (std::strcmp(arg, "--allgather") == 0) {
      allgather = true;
      return true;
    }
    return false;
  }
};

// One device's share of a box run.  The driver fills these in (operands, plan) with `device`
// current; run_box() only launches, times, gathers and dumps.
struct BoxSlab {
  int device = 0, n0 = 0, n_local = 0;
  cudaStream_t stream = nullptr;
  uint16_t* d = nullptr;               // [M, n_local] bf16 on `device`
  std::function<int()> launch;         // enqueue one GEMM on `stream`
  std::function<int()> check;          // synchronise and read the kernel status
  std::function<int()> verify;         // the driver's self-check of this slab (0 = passed), may be empty
  std::function<void()> destroy;
};

inline double run_box(std::vector<BoxSlab>& slabs, int M, int n_total, int K, bool benchmark, bool allgather,
                      const char* dump, const char* line_format) {
  const int G = static_cast<int>(slabs.size());
  auto on_all = [&](const std::function<void(BoxSlab&)>& fn) {
    for (BoxSlab& s : slabs) {
      DRV_CUDA(cudaSetDevice(s.device));
      fn(s);
    }
  };
  double ms = 0.0;
  if (benchmark) {
    std::vector<cudaEvent_t> begin(G), end(G);
    on_all([&](BoxSlab& s) {
      const int i = static_cast<int>(&s - slabs.data());
      DRV_CUDA(cudaEventCreate(&begin[i]));
      DRV_CUDA(cudaEventCreate(&end[i]));
    });
    for (int it = 0; it < 10; ++it) on_all([&](BoxSlab& s) { DRV_SMB(s.launch()); });
    on_all([&](BoxSlab& s) { DRV_CUDA(cudaStreamSynchronize(s.stream)); });
    on_all([&](BoxSlab& s) { DRV_CUDA(cudaEventRecord(begin[&s - slabs.data()], s.stream)); });
    for (int it = 0; it < 100; ++it) on_all([&](BoxSlab& s) { DRV_SMB(s.launch()); });
    on_all([&](BoxSlab& s) { DRV_CUDA(cudaEventRecord(end[&s - slabs.data()], s.stream)); });
    on_all([&](BoxSlab& s) {
      const int i = static_cast<int>(&s - slabs.data());
      DRV_CUDA(cudaStreamSynchronize(s.stream));
      float t = 0.0f;
      DRV_CUDA(cudaEventElapsedTime(&t, begin[i], end[i]));
      if (t / 100.0 > ms) ms = t / 100.0;   // the box is as fast as its slowest device
      DRV_CUDA(cudaEventDestroy(begin[i]));
      DRV_CUDA(cudaEventDestroy(end[i]));
    });
  } else {
    on_all([&](BoxSlab& s) { DRV_SMB(s.launch()); });
  }
  // The dumped output comes from one more launch, as in the reference driver.
  on_all([&](BoxSlab& s) { DRV_SMB(s.launch()); });
  on_all([&](BoxSlab& s) { DRV_SMB(s.check()); });
  double tflops = 0.0;
  if (benchmark) {
    tflops = 2.0 * M * n_total * K / (ms * 1e-3) / 1e12;
    std::printf(line_format, M, n_total, K, ms, tflops);
    std::printf("  box of %d GPUs, N column-parallel, %d columns each: %.1f per GPU\n", G, n_total / G, tflops / G);
  } else {
    std::printf("  shape (%6d, %6d, %4d): untimed\n", M, n_total, K);
  }
  const int n_local = slabs[0].n_local;
  std::vector<uint16_t*> gathered(G, nullptr), full(G, nullptr);
  if (allgather) {
    std::vector<smb_comm*> comms(G, nullptr);
    std::vector<int> devices(G);
    for (int i = 0; i < G; ++i) devices[i] = slabs[i].device;
    DRV_SMB(smb_comm_create_all(comms.data(), G, devices.data()));
    std::vector<const void*> send(G);
    std::vector<void*> recv(G), out(G), streams(G);
    on_all([&](BoxSlab& s) {
      const int i = static_cast<int>(&s - slabs.data());
      DRV_CUDA(cudaMalloc(&gathered[i], static_cast<size_t>(G) * M * n_local * 2));
      DRV_CUDA(cudaMalloc(&full[i], static_cast<size_t>(M) * n_total * 2));
      send[i] = s.d;
      recv[i] = gathered[i];
      out[i] = full[i];
      streams[i] = s.stream;
    });
    auto gather = [&](bool unshard) {
      DRV_SMB(smb_allgather_columns_multi(comms.data(), G, send.data(), recv.data(), unshard ? out.data() : nullptr,
                                          M, n_local, n_total, streams.data()));
    };
    auto timed = [&](bool unshard) {
      std::vector<cudaEvent_t> b(G), e(G);
      for (int it = 0; it < 2; ++it) gather(unshard);
      on_all([&](BoxSlab& s) {
        const int i = static_cast<int>(&s - slabs.data());
        DRV_CUDA(cudaStreamSynchronize(s.stream));
        DRV_CUDA(cudaEventCreate(&b[i]));
        DRV_CUDA(cudaEventCreate(&e[i]));
        DRV_CUDA(cudaEventRecord(b[i], s.stream));
      });
      for (int it = 0; it < 5; ++it) gather(unshard);
      double worst = 0.0;
      on_all([&](BoxSlab& s) {
        const int i = static_cast<int>(&s - slabs.data());
        DRV_CUDA(cudaEventRecord(e[i], s.stream));
        DRV_CUDA(cudaStreamSynchronize(s.stream));
        float t = 0.0f;
        DRV_CUDA(cudaEventElapsedTime(&t, b[i], e[i]));
        if (t / 5.0 > worst) worst = t / 5.0;
        DRV_CUDA(cudaEventDestroy(b[i]));
        DRV_CUDA(cudaEventDestroy(e[i]));
      });
      return worst;
    };
    const double ag_ms = timed(false);
    const double both_ms = timed(true);
    const double recv_bytes = static_cast<double>(G - 1) * M * n_local * 2;
    std::printf("  all-gather of D over %d GPUs: %.6f ms (%.1f GB/s received per GPU); with unshard copy %.6f ms\n",
                G, ag_ms, recv_bytes / (ag_ms * 1e-3) / 1e9, both_ms);
    for (smb_comm* c : comms) smb_comm_destroy(c);
  }
  if (dump != nullptr) {
    if (allgather) {
      DRV_CUDA(cudaSetDevice(slabs[0].device));
      dump_bf16(full[0], static_cast<size_t>(M) * n_total, dump);
    } else {
      std::vector<uint16_t> host(static_cast<size_t>(M) * n_total), part(static_cast<size_t>(M) * n_local);
      for (BoxSlab& s : slabs) {
        DRV_CUDA(cudaSetDevice(s.device));
        DRV_CUDA(cudaMemcpy(part.data(), s.d, part.size() * 2, cudaMemcpyDeviceToHost));
        for (int m = 0; m < M; ++m)
          std::memcpy(&host[static_cast<size_t>(m) * n_total + s.n0], &part[static_cast<size_t>(m) * n_local],
                      static_cast<size_t>(n_local) * 2);
      }
      FILE* f = std::fopen(dump, "wb");
      if (!f || std::fwrite(host.data(), 2, host.size(), f) != host.size()) {
        if (f) std::fclose(f);
        std::fprintf(stderr, "failed to write %s\n", dump);
        std::exit(1);
      }
      std::fclose(f);
      std::printf("  wrote %zu BF16 values to %s\n", host.size(), dump);
    }
  }
  int rc = 0;
  on_all([&](BoxSlab& s) {
    if (s.verify && s.verify() != 0) rc = 1;
  });
  on_all([&](BoxSlab& s) {
    const int i = static_cast<int>(&s - slabs.data());
    if (gathered[i]) cudaFree(gathered[i]);
    if (full[i]) cudaFree(full[i]);
    s.destroy();
  });
  if (rc != 0) std::exit(1);
  return tflops;
}
