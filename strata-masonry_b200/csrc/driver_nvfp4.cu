// kernel_sm100a_dense_gemm_nvfp4 -- command-line driver with the contract of the reference
// executable of the same name (main() of src/kernels/gemm/sm100a/nvfp4/dense_gemm_nvfp4.cu:2941-3258):
//   --shape=M,K,N  --fill=N  --no-benchmark  --no-gpu-verify  --dump-output=PATH  --help
// Single-case output line:  "  shape (M, N, K): mean=X ms  Y NVFP4_TFLOPS".
// The built-in check follows the reference: fills 1 and 3 are checked over the whole output
// against the closed form (exact), the other fills on 2048 hashed samples against a host fp32
// reference with tolerance max(0.8 % |ref|, 16).  FILL environment variable as default fill.
// Beyond the reference: any positive M and N, any K that is a multiple of 32, fills 5 and 6
// (quantised Gaussian stand-ins), --json=PATH, --ordered-launches, --shard=RANK/WORLD and
// --device=INDEX (one process per GPU computes its column slab of D), --gpus=G [--allgather] (one
// process drives G devices, times the box, optionally exchanges the slabs with an NCCL all-gather
// timed apart, and dumps the full D); no arguments runs a short shape list.
#include <cmath>

#include "driver_common.h"

namespace {

const float kE2m1[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                         -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

uint32_t hash32(uint32_t x) {
  x *= 2654435761u;
  x ^= x >> 16;
  x *= 2246822519u;
  x ^= x >> 13;
  return x;
}

struct Options {
  int fill = 1;
  bool benchmark = true;
  bool verify = true;
  const char* dump = nullptr;
  const char* json = nullptr;
  // false (default): launches of the timing loop are independent of one another, as the
  // reference kernels' are; true: every launch orders its stores after the previous launch.
  bool ordered = false;
  Shard shard;
  BoxOptions box;
};

// One logical row of an operand on the host: values (code * scale) as floats.
void host_row(std::vector<float>& out, int row, int K, int fill, int which) {
  std::vector<uint8_t> data(K / 2 + 16), sf(K / 32);
  // 16-byte aligned scratch for the generator.
  uint8_t* aligned = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(data.data()) + 15) & ~uintptr_t(15));
  DRV_SMB(smb_fill_fp4_host(aligned, (K / 2 + 15) / 16 * 16, nullptr, sf.data(), 1, K,
                            static_cast<uint64_t>(row), fill, which));
  out.resize(K);
  for (int k = 0; k < K; ++k) {
    const uint8_t byte = aligned[k / 2];
    const uint32_t code = (k & 1) ? (byte >> 4) : (byte & 15);
    out[k] = kE2m1[code] * std::exp2(static_cast<float>(static_cast<int>(sf[k / 32]) - 127));
  }
}

// Operands, output and plan of one device's share: columns [n0, n0 + N) of the logical problem.
struct Case {
  int M = 0, N = 0, K = 0, n0 = 0, fill = 1;
  uint8_t *a = nullptr, *b = nullptr, *sfa = nullptr, *sfb = nullptr;
  uint16_t* d = nullptr;
  cudaStream_t stream = nullptr;
  smb_fp4_plan* plan = nullptr;
};

// On the current device.
Case make_case(int M, int K, int n0, int n_local, const Options& o) {
  Case c;
  c.M = M;
  c.N = n_local;
  c.K = K;
  c.n0 = n0;
  c.fill = o.fill;
  const int N = n_local;
  const size_t sfa_bytes = smb_sf_packed_bytes(M, K / 32), sfb_bytes = smb_sf_packed_bytes(N, K / 32);
  DRV_CUDA(cudaMalloc(&c.a, static_cast<size_t>(M) * K / 2));
  DRV_CUDA(cudaMalloc(&c.b, static_cast<size_t>(N) * K / 2));
  DRV_CUDA(cudaMalloc(&c.sfa, sfa_bytes));
  DRV_CUDA(cudaMalloc(&c.sfb, sfb_bytes));
  DRV_CUDA(cudaMalloc(&c.d, static_cast<size_t>(M) * N * 2));
  DRV_CUDA(cudaMemset(c.d, 0, static_cast<size_t>(M) * N * 2));
  DRV_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
  DRV_SMB(smb_fill_fp4_device(c.a, K / 2, c.sfa, nullptr, M, K, 0, o.fill, 0, c.stream));
  DRV_SMB(smb_fill_fp4_device(c.b, K / 2, c.sfb, nullptr, N, K, static_cast<uint64_t>(n0), o.fill, 1, c.stream));
  DRV_CUDA(cudaStreamSynchronize(c.stream));
  DRV_SMB(smb_fp4_plan_create(&c.plan, c.a, c.sfa, c.b, c.sfb, c.d, M, N, K, K / 2, K / 2, N,
                              o.ordered ? SMB_FLAG_OPERANDS_STATIC : SMB_FLAG_LAUNCH_INDEPENDENT));
  return c;
}

void free_case(Case& c) {
  smb_fp4_plan_destroy(c.plan);
  cudaStreamDestroy(c.stream);
  cudaFree(c.a);
  cudaFree(c.b);
  cudaFree(c.sfa);
  cudaFree(c.sfb);
  cudaFree(c.d);
}

// The driver's self-check of one slab (global column = n0 + n); 0 = passed.
int verify_case(const Case& c) {
  const int M = c.M, N = c.N, K = c.K, n0 = c.n0, fill = c.fill;
  int rc = 0;
  std::vector<uint16_t> host(static_cast<size_t>(M) * N);
  DRV_CUDA(cudaMemcpy(host.data(), c.d, host.size() * 2, cudaMemcpyDeviceToHost));
  if (fill == 1 || fill == 3) {
    // D[m][n] = p K 2^((m % 5) - 2) 2^((n % 3) - 1), p = 16 (fill 1) or 1 (fill 3): exact.
    const float per_product = (fill == 3) ? 1.0f : 16.0f;
    float max_rel = 0.0f;
    int nan_count = 0, bad_m = -1, bad_n = -1;
    for (int m = 0; m < M; ++m) {
      const float sa = std::exp2(static_cast<float>(m % 5 - 2));
      for (int n = 0; n < N; ++n) {
        const float v = bf16_bits_to_float(host[static_cast<size_t>(m) * N + n]);
        if (std::isnan(v) || std::isinf(v)) { ++nan_count; continue; }
        const float expected = per_product * K * sa * std::exp2(static_cast<float>((n0 + n) % 3 - 1));
        const float rel = std::fabs(v - expected) / expected;
        if (rel > max_rel) { max_rel = rel; bad_m = m; bad_n = n; }
      }
    }
    const bool ok = nan_count == 0 && max_rel < 1e-3f;
    std::printf("  verify M=%d,N=%d,K=%d (real scales): max_rel=%.2e nan=%d %s", M, N, K, max_rel,
                nan_count, ok ? "OK" : "FAIL");
    if (!ok && bad_m >= 0) std::printf(" [worst at m=%d n=%d]", bad_m, bad_n);
    std::printf("\n");
    if (!ok) rc = 1;
  } else {
    int fail = 0, nan_count = 0, bad_m = -1, bad_n = -1;
    float max_err = 0.0f, max_ref = 0.0f, max_got = 0.0f;
    std::vector<float> ra, rb;
    for (int smp = 0; smp < 2048; ++smp) {
      const int m = static_cast<int>(hash32(2u * smp + 1u) % static_cast<uint32_t>(M));
      const int n = static_cast<int>(hash32(2u * smp + 2u) % static_cast<uint32_t>(N));
      host_row(ra, m, K, fill, 0);
      host_row(rb, n0 + n, K, fill, 1);
      float acc = 0.0f;
      for (int k = 0; k < K; ++k) acc += ra[k] * rb[k];
      uint32_t bits;
      std::memcpy(&bits, &acc, 4);
      const float ref = bf16_bits_to_float(static_cast<uint16_t>((bits + 0x7FFFu + ((bits >> 16) & 1u)) >> 16));
      const float got = bf16_bits_to_float(host[static_cast<size_t>(m) * N + n]);
      if (std::isnan(got) || std::isinf(got)) { ++nan_count; continue; }
      const float err = std::fabs(got - ref);
      const float floor_abs = (fill <= 4) ? 16.0f : 0.25f;
      if (err > std::fmax(0.008f * std::fabs(ref), floor_abs)) {
        ++fail;
        if (err > max_err) { max_err = err; bad_m = m; bad_n = n; max_ref = ref; max_got = got; }
      }
    }
    const bool ok = nan_count == 0 && fail == 0;
    std::printf("  verify M=%d,N=%d,K=%d (FILL=%d sampled ref x2048): fail=%d nan=%d %s", M, N, K,
                fill, fail, nan_count, ok ? "OK" : "FAIL");
    if (!ok && bad_m >= 0)
      std::printf(" [worst at m=%d n=%d: got %.3f ref %.3f]", bad_m, bad_n, max_got, max_ref);
    std::printf("\n");
    if (!ok) rc = 1;
  }
  return rc;
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
      cases[g] = make_case(M, K, n0, n_local, o);
      Case* c = &cases[g];
      BoxSlab& s = slabs[g];
      s.device = g;
      s.n0 = n0;
      s.n_local = n_local;
      s.stream = c->stream;
      s.d = c->d;
      s.launch = [c]() { return smb_fp4_plan_run(c->plan, c->stream); };
      s.check = [c]() { return smb_fp4_plan_check(c->plan, c->stream); };
      if (o.verify) s.verify = [c]() { return verify_case(*c); };
      s.destroy = [c]() { free_case(*c); };
    }
    const double tflops = run_box(slabs, M, n_total, K, o.benchmark, o.box.allgather, o.dump,
                                  "  shape (%6d, %6d, %4d): mean=%.6f ms  %7.1f NVFP4_TFLOPS\n");
    DRV_CUDA(cudaSetDevice(0));
    return tflops;
  }
  Shard shard = o.shard;
  shard.resolve(n_total);
  const int N = shard.n_local;   // everything below works on this process's slab; global column = n0 + n
  Case c = make_case(M, K, shard.n0, N, o);
  cudaStream_t stream = c.stream;
  auto launch = [&]() { return smb_fp4_plan_run(c.plan, stream); };
  double ms = 0.0;
  if (o.benchmark) {
    ms = measure_mean_ms(stream, launch);
  } else {
    DRV_SMB(launch());
  }
  DRV_SMB(launch());
  DRV_SMB(smb_fp4_plan_check(c.plan, stream));
  double tflops = 0.0;
  if (o.benchmark) {
    tflops = 2.0 * M * N * K / (ms * 1e-3) / 1e12;
    std::printf("  shape (%6d, %6d, %4d): mean=%.6f ms  %7.1f NVFP4_TFLOPS\n", M, N, K, ms, tflops);
  } else {
    std::printf("  shape (%6d, %6d, %4d): untimed\n", M, N, K);
  }
  write_json(o.json, "dense_gemm_nvfp4", M, N, K, o.fill, ms, tflops, o.benchmark);
  if (o.dump) dump_bf16(c.d, static_cast<size_t>(M) * N, o.dump);
  const int rc = o.verify ? verify_case(c) : 0;
  free_case(c);
  if (rc != 0) std::exit(EXIT_FAILURE);
  return tflops;
}

bool parse_positive(const char*& text, int& out) {
  char* end = nullptr;
  const long v = std::strtol(text, &end, 10);
  if (end == text || v <= 0 || v > 2147483647L) return false;
  out = static_cast<int>(v);
  text = end;
  return true;
}

}  // namespace

int main(int argc, char** argv) {
  Options o;
  if (const char* env = std::getenv("FILL")) {
    const int f = std::atoi(env);
    if (f >= 1 && f <= 6) o.fill = f;
  }
  int M = 0, K = 0, N = 0;
  for (int i = 1; i < argc; ++i) {
    if (std::strncmp(argv[i], "--shape=", 8) == 0) {
      const char* text = argv[i] + 8;
      if (!parse_positive(text, M) || *text++ != ',' || !parse_positive(text, K) || *text++ != ',' ||
          !parse_positive(text, N) || *text != '\0') {
        std::fprintf(stderr, "--shape must be positive integers M,K,N\n");
        return 1;
      }
    } else if (std::strncmp(argv[i], "--fill=", 7) == 0) {
      const char* text = argv[i] + 7;
      if (!parse_positive(text, o.fill) || *text || o.fill > 6) {
        std::fprintf(stderr, "--fill must be 1, 2, 3, or 4 (5, 6: quantised Gaussian stand-ins)\n");
        return 1;
      }
    } else if (std::strcmp(argv[i], "--no-benchmark") == 0) {
      o.benchmark = false;
    } else if (std::strcmp(argv[i], "--no-gpu-verify") == 0) {
      o.verify = false;
    } else if (std::strcmp(argv[i], "--ordered-launches") == 0) {
      o.ordered = true;
    } else if (std::strncmp(argv[i], "--dump-output=", 14) == 0 && argv[i][14]) {
      o.dump = argv[i] + 14;
    } else if (o.shard.parse(argv[i])) {
    } else if (o.box.parse(argv[i])) {
    } else if (std::strncmp(argv[i], "--json=", 7) == 0 && argv[i][7]) {
      o.json = argv[i] + 7;
    } else if (std::strcmp(argv[i], "--help") == 0) {
      std::printf("Usage: %s [--shape=M,K,N [--fill=1..6] [--no-benchmark]\n"
                  "       [--no-gpu-verify] [--dump-output=PATH] [--json=PATH]\n"
                  "       [--shard=RANK/WORLD] [--device=INDEX] [--gpus=G [--allgather]]]\n"
                  "No arguments: short sweep (FILL environment variable supported).\n", argv[0]);
      return 0;
    } else {
      std::fprintf(stderr, "unknown or empty argument: %s\n", argv[i]);
      return 1;
    }
  }
  if (argc > 1) {
    if (!M || !N || !K || K % 32 != 0) {
      std::fprintf(stderr, "require --shape=M,K,N: positive M and N, K a multiple of 32\n");
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
  std::printf("K1 dense_gemm_nvfp4 (sm_100a, B200) -- block32 UE8M0\n\n");
  if (argc > 1) {
    run_one(M, N, K, o);
    return 0;
  }
  struct Shape { const char* label; int M, K, N; };
  const Shape shapes[] = {
      {"und-gate", 14080, 2048, 128},  {"und-qkv", 14080, 2048, 5120}, {"und-o", 14080, 4096, 2048},
      {"gen-gate", 30720, 2048, 128},  {"gen-qkv", 30720, 2048, 5120}, {"gen-o", 30720, 4096, 2048},
      {"gen-o-2K", 30720, 8192, 2048}, {"2K+2N", 30720, 8192, 4096},   {"8192^3", 8192, 8192, 8192},
      {"16384^3", 16384, 16384, 16384},
  };
  for (const Shape& s : shapes) {
    std::printf("[%s]\n", s.label);
    run_one(s.M, s.N, s.K, o);
  }
  return 0;
}
