// kernel_sm100a_dense_gemm_bf16 -- command-line driver with the contract of the reference
// executable of the same name (main() of src/kernels/gemm/sm100a/dense_gemm_bf16.cu:485-565):
//   --shape=M,K,N  --fill=N  --no-benchmark  --no-gpu-verify  --raster=along-m|along-n
//   --dump-output=PATH          (raw little-endian bf16, M*N values, row-major, no header)
// No arguments: the reference's built-in shape inventory with the GPU self-check.
// Beyond the reference: any positive M and N, any K that is a multiple of 8, fills 5..7
// (Gaussian stand-ins), --json=PATH, --ordered-launches (stores of a launch wait for the
// previous launch; by default the timing loop's launches are independent, as the reference's
// are), --shard=RANK/WORLD and --device=INDEX (one process per GPU computes and dumps its column
// slab of D), --gpus=G [--allgather] (one process drives G devices, times the box, optionally
// exchanges the slabs with an NCCL all-gather timed apart, and dumps the full D).  Operands are
// generated on the device.
#include "driver_common.h"

namespace {

// CUDA-core reference for --gpu-verify: one block per row, fp32 dot products.
__global__ void reference_gemm_bf16(const uint16_t* a, const uint16_t* bt, uint16_t* d, int M, int N,
                                    int K) {
  const int m = blockIdx.x;
  if (m >= M) return;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) {
      acc += __uint_as_float(static_cast<uint32_t>(a[static_cast<size_t>(m) * K + k]) << 16) *
             __uint_as_float(static_cast<uint32_t>(bt[static_cast<size_t>(n) * K + k]) << 16);
    }
    uint32_t b = __float_as_uint(acc);
    d[static_cast<size_t>(m) * N + n] = static_cast<uint16_t>((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
  }
}

const char* fill_label(int fill) {
  switch (fill) {
    case 1: return "[-0.5,0.5) /256";
    case 2: return "[-1.0,1.0) /2048";
    case 3: return "const 1.0";
    case 4: return "int{-3..3} /7 (profiler)";
    case 5: return "gauss12 * 0.1";
    case 6: return "gauss12 * 0.05";
    case 7: return "gauss12";
    default: return "unknown";
  }
}

struct Options {
  int fill = 1;
  bool benchmark = true;
  bool verify = true;
  int raster = 0;   // 0 default grouping, 1 along-n, 2 along-m
  const char* dump = nullptr;
  const char* json = nullptr;
  // false (default): launches of the timing loop are independent of one another, as the
  // reference kernels' are; true: every launch orders its stores after the previous launch.
  bool ordered = false;
  Shard shard;
  BoxOptions box;
};

// Operands, output and plan of one device's share: columns [n0, n0 + N) of the logical problem.
struct Case {
  int M = 0, N = 0, K = 0, n0 = 0, n_total = 0;
  uint16_t *a = nullptr, *bt = nullptr, *d = nullptr;
  cudaStream_t stream = nullptr;
  smb_bf16_plan* plan = nullptr;
};

// On the current device.
Case make_case(int M, int n_total, int K, int n0, int n_local, const Options& o) {
  Case c;
  c.M = M;
  c.N = n_local;
  c.K = K;
  c.n0 = n0;
  c.n_total = n_total;
  const int N = n_local;
  DRV_CUDA(cudaMalloc(&c.a, static_cast<size_t>(M) * K * 2));
  DRV_CUDA(cudaMalloc(&c.bt, static_cast<size_t>(N) * K * 2));
  DRV_CUDA(cudaMalloc(&c.d, static_cast<size_t>(M) * N * 2));
  DRV_CUDA(cudaMemset(c.d, 0, static_cast<size_t>(M) * N * 2));
  DRV_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
  // A: index m*K + k, seed 1.  BT[n][k] = B[k][n]: index k*N + n, seed 2.
  DRV_SMB(smb_fill_bf16_device(c.a, M, K, K, 0, static_cast<uint64_t>(K), 1, o.fill, 1, c.stream));
  DRV_SMB(smb_fill_bf16_device(c.bt, N, K, K, static_cast<uint64_t>(n0), 1, static_cast<uint64_t>(n_total),
                               o.fill, 2, c.stream));
  DRV_CUDA(cudaStreamSynchronize(c.stream));
  DRV_SMB(smb_bf16_plan_create(&c.plan, c.a, c.bt, c.d, M, N, K, K, K, N,
                               o.ordered ? SMB_FLAG_OPERANDS_STATIC : SMB_FLAG_LAUNCH_INDEPENDENT));
  if (o.raster == 1) DRV_SMB(smb_bf16_plan_tune(c.plan, 1, 0));
  if (o.raster == 2) DRV_SMB(smb_bf16_plan_tune(c.plan, (M + 255) / 256, 0));
  return c;
}

// The driver's self-check of one slab against the CUDA-core reference; 0 = passed.
int verify_case(const Case& c) {
  const int M = c.M, N = c.N, K = c.K;
  uint16_t* ref = nullptr;
  DRV_CUDA(cudaMalloc(&ref, static_cast<size_t>(M) * N * 2));
  reference_gemm_bf16<<<M, 256>>>(c.a, c.bt, ref, M, N, K);
  DRV_CUDA(cudaDeviceSynchronize());
  std::vector<uint16_t> got(static_cast<size_t>(M) * N), want(got.size());
  DRV_CUDA(cudaMemcpy(got.data(), c.d, got.size() * 2, cudaMemcpyDeviceToHost));
  DRV_CUDA(cudaMemcpy(want.data(), ref, want.size() * 2, cudaMemcpyDeviceToHost));
  float max_diff = 0.0f;
  bool ok = true;
  for (size_t i = 0; i < got.size(); ++i) {
    const float g = bf16_bits_to_float(got[i]), w = bf16_bits_to_float(want[i]);
    const float diff = fabsf(g - w);
    if (!(diff <= max_diff)) max_diff = diff;
    if (!(diff <= 0.05f + 0.05f * fabsf(w))) ok = false;
  }
  std::printf("  verify (M=%d,N=%d,K=%d): max_diff=%.3f tight=%s\n", M, N, K, max_diff, ok ? "OK" : "FAIL");
  cudaFree(ref);
  return ok ? 0 : 1;
}

void free_case(Case& c) {
  smb_bf16_plan_destroy(c.plan);
  cudaStreamDestroy(c.stream);
  cudaFree(c.a);
  cudaFree(c.bt);
  cudaFree(c.d);
}

double run_one(int M, int n_total, int K, const Options& o) {
  if (o.box.gpus > 0) {
    // One process, several devices: device g holds the slab of rank g.
    int have = 0;
    DRV_CUDA(cudaGetDeviceCount(&have));
    if (o.box.gpus > have) {
      std::fprintf(stderr, "--gpus=%d but only %d device(s) are visible\n", o.box.gpus, have);
      std::exit(1);
    }
    std::vector<Case> cases(o.box.gpus);
    std::vector<BoxSlab> slabs(o.box.gpus);
    for (int g = 0; g < o.box.gpus; ++g) {
      int n0 = 0, n_local = 0;
      if (smb_column_shard(n_total, o.box.gpus, g, &n0, &n_local) != SMB_OK) {
        std::fprintf(stderr, "unsupported --gpus for this shape: %s\n", smb_last_error());
        std::exit(1);
      }
      DRV_CUDA(cudaSetDevice(g));
      cases[g] = make_case(M, n_total, K, n0, n_local, o);
      Case* c = &cases[g];
      BoxSlab& s = slabs[g];
      s.device = g;
      s.n0 = n0;
      s.n_local = n_local;
      s.stream = c->stream;
      s.d = c->d;
      s.launch = [c]() { return smb_bf16_plan_run(c->plan, c->stream); };
      s.check = [c]() { return smb_bf16_plan_check(c->plan, c->stream); };
      if (o.verify) s.verify = [c]() { return verify_case(*c); };
      s.destroy = [c]() { free_case(*c); };
    }
    const double tflops = run_box(slabs, M, n_total, K, o.benchmark, o.box.allgather, o.dump,
                                  "  shape (%6d, %6d, %4d): %.6f ms  %7.1f TFLOPS\n");
    DRV_CUDA(cudaSetDevice(0));
    return tflops;
  }
  Shard shard = o.shard;
  shard.resolve(n_total);
  const int N = shard.n_local;   // everything below works on this process's slab
  Case c = make_case(M, n_total, K, shard.n0, N, o);
  cudaStream_t stream = c.stream;
  auto launch = [&]() { return smb_bf16_plan_run(c.plan, stream); };
  double ms = 0.0;
  if (o.benchmark) {
    ms = measure_mean_ms(stream, launch);
  } else {
    DRV_SMB(launch());
  }
  // The dumped output comes from one more launch, as in the reference driver.
  DRV_SMB(launch());
  DRV_SMB(smb_bf16_plan_check(c.plan, stream));
  double tflops = 0.0;
  if (o.benchmark) {
    tflops = 2.0 * M * N * K / (ms * 1e-3) / 1e12;
    std::printf("  shape (%6d, %6d, %4d): %.6f ms  %7.1f TFLOPS\n", M, N, K, ms, tflops);
  } else {
    std::printf("  shape (%6d, %6d, %4d): untimed\n", M, N, K);
  }
  write_json(o.json, "dense_gemm_bf16", M, N, K, o.fill, ms, tflops, o.benchmark);
  if (o.dump) dump_bf16(c.d, static_cast<size_t>(M) * N, o.dump);
  const int rc = o.verify ? verify_case(c) : 0;
  free_case(c);
  if (rc != 0) std::exit(rc);
  return tflops;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  int M = 0, K = 0, N = 0;
  for (int i = 1; i < argc; ++i) {
    if (std::strncmp(argv[i], "--fill=", 7) == 0) {
      o.fill = std::atoi(argv[i] + 7);
      if (o.fill < 1 || o.fill > 7) {
        std::fprintf(stderr, "--fill must be 1, 2, 3, or 4 (5, 6, 7: Gaussian stand-ins)\n");
        return 1;
      }
    } else if (std::strncmp(argv[i], "--shape=", 8) == 0) {
      if (std::sscanf(argv[i] + 8, "%d,%d,%d", &M, &K, &N) != 3) {
        std::fprintf(stderr, "--shape must be M,K,N\n");
        return 1;
      }
    } else if (std::strcmp(argv[i], "--no-benchmark") == 0) {
      o.benchmark = false;
    } else if (std::strcmp(argv[i], "--no-gpu-verify") == 0) {
      o.verify = false;
    } else if (std::strcmp(argv[i], "--ordered-launches") == 0) {
      o.ordered = true;
    } else if (std::strcmp(argv[i], "--raster=along-m") == 0) {
      o.raster = 2;
    } else if (std::strcmp(argv[i], "--raster=along-n") == 0) {
      o.raster = 1;
    } else if (std::strncmp(argv[i], "--dump-output=", 14) == 0) {
      o.dump = argv[i] + 14;
    } else if (std::strncmp(argv[i], "--json=", 7) == 0) {
      o.json = argv[i] + 7;
    } else if (o.shard.parse(argv[i])) {
    } else if (o.box.parse(argv[i])) {
    } else {
      std::fprintf(stderr, "unknown argument: %s\n", argv[i]);
      return 1;
    }
  }
  if (o.box.allgather && o.box.gpus < 1) {
    std::fprintf(stderr, "--allgather requires --gpus=G\n");
    return 1;
  }
  if (o.box.gpus > 0 && o.shard.world > 1) {
    std::fprintf(stderr, "--gpus and --shard exclude each other\n");
    return 1;
  }
  DRV_CUDA(cudaSetDevice(o.shard.device));
  DRV_CUDA(cudaFree(0));
  std::printf("K0 dense_gemm_bf16 (Blackwell B200, sm_100a) -- fill=%d %s\n", o.fill,
              fill_label(o.fill));
  std::printf("=============================================\n");

  if (M || K || N) {
    if (M <= 0 || K <= 0 || N <= 0) {
      std::fprintf(stderr, "--shape dimensions must be positive\n");
      return 1;
    }
    if (K % 8 != 0) {
      std::fprintf(stderr, "unsupported --shape for this kernel (K must be a multiple of 8)\n");
      return 1;
    }
    run_one(M, N, K, o);
    return 0;
  }
  if (o.dump) {
    std::fprintf(stderr, "--dump-output requires --shape=M,K,N\n");
    return 1;
  }

  // The reference driver's shape inventory (M padded to 14080 for the UND rows).
  struct Shape { const char* label; int M, K, N; };
  const Shape shapes[] = {
      {"und-gate", 14080, 2048, 128},  {"und-qkv", 14080, 2048, 5120}, {"und-o", 14080, 4096, 2048},
      {"gen-gate", 30720, 2048, 128},  {"gen-qkv", 30720, 2048, 5120}, {"gen-o", 30720, 4096, 2048},
  };
  std::printf("\n[V0 shape inventory]\n");
  for (const Shape& s : shapes) {
    std::printf("\n[%s]\n", s.label);
    Options along = o;
    std::printf("  AlongN:\n");
    along.raster = 1;
    run_one(s.M, s.N, s.K, along);
    std::printf("  AlongM:\n");
    along.raster = 2;
    run_one(s.M, s.N, s.K, along);
  }
  return 0;
}
