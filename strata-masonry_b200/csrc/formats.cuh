// Number formats and input generators of the dense GEMM path, written once for host and
// device so that the CUDA fills, the C++ host fills and the drivers cannot drift apart.
// The NumPy oracle restates the same rules independently and the tests compare the two
// bit for bit.
//
// Reference definitions these follow:
//   BF16 fills 1-4      src/kernels/gemm/sm100a/dense_gemm_bf16.cu:268-279
//                       dense_gemm_bf16_cpu_verifier.py:32-44
//   bf16 rounding       dense_gemm_bf16_cpu_verifier.py:26-29
//   hash, FP4 fills     nvfp4/dense_gemm_nvfp4.cu:2271-2290, verifier :27-63
//   scale exponents     nvfp4/dense_gemm_nvfp4.cu:2287-2290, :2436-2437, verifier :66-77
//   scale packing       nvfp4/dense_gemm_nvfp4.cu:2418-2435
// The Gaussian fills (5-7) and the FP32 -> E2M1/UE8M0 quantiser have no counterpart in the
// reference; they are defined here and in the oracle.
#pragma once

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define SMB_HD __host__ __device__ __forceinline__
#else
#define SMB_HD inline
#endif

namespace smb {
namespace fmt {

constexpr uint32_t kSeedFp4A = 0x9E3779B9u;
constexpr uint32_t kSeedFp4B = 0x7F4A7C15u;

SMB_HD uint32_t f32_bits(float v) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(v);
#else
  uint32_t b;
  std::memcpy(&b, &v, 4);
  return b;
#endif
}
SMB_HD float bits_f32(uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(b);
#else
  float v;
  std::memcpy(&v, &b, 4);
  return v;
#endif
}

// fp32 -> bf16, round to nearest even (finite inputs).
SMB_HD uint16_t f32_to_bf16(float v) {
  const uint32_t b = f32_bits(v);
  return static_cast<uint16_t>((b + 0x7FFFu + ((b >> 16) & 1u)) >> 16);
}
SMB_HD float bf16_to_f32(uint16_t h) { return bits_f32(static_cast<uint32_t>(h) << 16); }

// Two rounds of multiply / xor-shift, 32-bit wrap-around.
SMB_HD uint32_t hash32(uint32_t x) {
  x *= 2654435761u;
  x ^= x >> 16;
  x *= 2246822519u;
  x ^= x >> 13;
  return x;
}

// Gaussian stand-in: twelve 16-bit uniform fields of six counter-hash words, summed and
// centred.  Mean 0, variance 1 (to 2^-32), range (-6, 6), every value a multiple of 2^-16.
SMB_HD float gauss12(uint32_t index, uint32_t seed) {
  const uint32_t base = index * 6u + seed * 0x632BE5ABu;
  uint32_t sum = 0;
  for (uint32_t j = 0; j < 6; ++j) {
    const uint32_t w = hash32(base + j);
    sum += (w & 0xFFFFu) + (w >> 16);
  }
  return static_cast<float>(static_cast<int32_t>(sum) - 393210) * (1.0f / 65536.0f);
}

SMB_HD float mul_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fmul_rn(a, b);
#else
  return a * b;
#endif
}

// Value of BF16 fill `fill` at flat index `index`, before rounding to bf16.
SMB_HD float bf16_fill_value(uint32_t index, int fill, uint32_t seed) {
  const uint32_t x = index * 2654435761u + seed;
  switch (fill) {
    case 1: return static_cast<float>(x % 256u) / 256.0f - 0.5f;
    case 2: return static_cast<float>(x % 2048u) / 1024.0f - 1.0f;
    case 3: return 1.0f;
    case 4: return static_cast<float>(static_cast<int>(x % 7u) - 3);
    case 5: return mul_rn(gauss12(index, seed), 0.1f);
    case 6: return mul_rn(gauss12(index, seed), 0.05f);
    case 7: return gauss12(index, seed);
    default: return 0.0f;
  }
}

// ------------------------------------------------------------------------------- E2M1
SMB_HD float e2m1_decode(uint32_t code) {
  const float mags[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  const float m = mags[code & 7u];
  return (code & 8u) ? -m : m;
}

// Nearest E2M1 code of `v` (|v| <= 6 expected, larger saturates), ties to the even code.
SMB_HD uint32_t e2m1_encode(float v) {
  const float a = v < 0.0f ? -v : v;
  const uint32_t mag = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) +
                       (a >= 3.5f) + (a > 5.0f);
  return mag | (v < 0.0f ? 8u : 0u);
}

// UE8M0 exponent for a block with absolute maximum `amax`: the smallest e with
// 6 * 2^e >= amax, clamped to [-126, 127]; 0 for an all-zero block.
SMB_HD int ue8m0_exponent(float amax) {
  if (!(amax > 0.0f)) return 0;
  const uint32_t b = f32_bits(amax);
  int biased = static_cast<int>((b >> 23) & 0xFFu);
  uint32_t mant = b & 0x7FFFFFu;
  if (biased == 0) {
    // Subnormal: any such block clamps to the smallest exponent.
    return -126;
  }
  // amax = (1 + mant / 2^23) * 2^(biased - 127).  amax / 6 <= 2^e  <=>
  // (1 + mant/2^23) <= 1.5 * 2^(e - (biased - 127) + 2).
  const int x = biased - 127;
  int e = (mant <= 0x400000u) ? (x - 2) : (x - 1);
  if (e < -126) e = -126;
  if (e > 127) e = 127;
  return e;
}
SMB_HD float exp2i(int e) { return bits_f32(static_cast<uint32_t>(e + 127) << 23); }

// ------------------------------------------------------------------------------- E4M3 (unsigned use)
// OCP FP8 E4M3: bias 7, three mantissa bits, subnormals m * 2^-9, largest finite value 448
// (0x7E); 0x7F is NaN and never produced.  Scale bytes of NVFP4 (one per 16 K) use the
// non-negative half.
SMB_HD float add_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fadd_rn(a, b);
#else
  return a + b;
#endif
}
SMB_HD float div_rn(float a, float b) {
#if defined(__CUDA_ARCH__)
  return __fdiv_rn(a, b);
#else
  return a / b;
#endif
}

// Nearest E4M3 code of x >= 0 (round to nearest even, saturating at 448).
SMB_HD uint32_t e4m3_encode(float x) {
  if (!(x > 0.0f)) return 0u;
  if (x >= 464.0f) return 0x7Eu;                     // above the rounding boundary of 448
  if (x < 0.015625f) {                                // below 2^-6: subnormal grid of 2^-9
    const float t = add_rn(mul_rn(x, 512.0f), 12582912.0f);   // 1.5 * 2^23: rounds to an integer
    return f32_bits(t) & 0xFu;                        // 0..8; 8 is the smallest normal, code 0x08
  }
  const uint32_t b = f32_bits(x);
  const uint32_t r = b + 0x7FFFFu + ((b >> 20) & 1u);  // round the mantissa to three bits
  const uint32_t code = ((((r >> 23) & 0xFFu) - 120u) << 3) | ((r >> 20) & 7u);
  return code > 0x7Eu ? 0x7Eu : code;
}

SMB_HD float e4m3_decode(uint32_t code) {
  const uint32_t e = (code >> 3) & 0xFu, m = code & 7u;
  if (e == 0) return static_cast<float>(m) * 0.001953125f;                  // m * 2^-9
  return mul_rn(1.0f + static_cast<float>(m) * 0.125f, exp2i(static_cast<int>(e) - 7));
}

// FP32 -> E2M1 + UE8M0, one block of 32 values: scale exponent = the smallest e with
// 6 * 2^e >= max|v|, codes = nearest E2M1 value of v * 2^-e (ties to the even code), two codes per
// byte with the even element in the low nibble.
SMB_HD void quantize_mx_block(const float* v, uint8_t* codes16, uint8_t* scale_byte) {
  float amax = 0.0f;
  for (int i = 0; i < 32; ++i) {
    const float a = v[i] < 0.0f ? -v[i] : v[i];
    amax = a > amax ? a : amax;
  }
  const int e = ue8m0_exponent(amax);
  const float inv = exp2i(-e);
  for (int i = 0; i < 16; ++i) {
    const uint32_t lo = e2m1_encode(mul_rn(v[2 * i], inv));
    const uint32_t hi = e2m1_encode(mul_rn(v[2 * i + 1], inv));
    codes16[i] = static_cast<uint8_t>(lo | (hi << 4));
  }
  *scale_byte = static_cast<uint8_t>(e + 127);
}

// NVFP4 proper: 16 values share one E4M3 scale; `gs` is the caller's per-tensor factor
// (typically 448 * 6 / max|tensor|).  scale = e4m3(max|v| * gs / 6); code = e2m1(v * gs / scale).
// The represented value is e2m1(code) * e4m3(scale) / gs.
SMB_HD void quantize_nvf4_block(const float* v, float gs, uint8_t* codes8, uint8_t* scale_byte) {
  float amax = 0.0f;
  for (int i = 0; i < 16; ++i) {
    const float a = v[i] < 0.0f ? -v[i] : v[i];
    amax = a > amax ? a : amax;
  }
  const uint32_t sb = e4m3_encode(div_rn(mul_rn(amax, gs), 6.0f));
  const float s = e4m3_decode(sb);
  for (int i = 0; i < 8; ++i) {
    uint32_t lo = 0, hi = 0;
    if (s > 0.0f) {
      lo = e2m1_encode(div_rn(mul_rn(v[2 * i], gs), s));
      hi = e2m1_encode(div_rn(mul_rn(v[2 * i + 1], gs), s));
    }
    codes8[i] = static_cast<uint8_t>(lo | (hi << 4));
  }
  *scale_byte = static_cast<uint8_t>(sb);
}

// ------------------------------------------------------------------------------- FP4 fills
// E2M1 code of reference fills 1-4 for element `index` (= row * K + k, 32-bit wrap).
SMB_HD uint32_t fp4_fill_code(uint32_t index, int fill, uint32_t seed) {
  if (fill == 1) return 6u;   // 4.0
  if (fill == 3) return 2u;   // 1.0
  const uint32_t h = hash32(index * 2u + seed);
  if (fill == 2) return h & 15u;
  const uint32_t mags[4] = {0u, 2u, 4u, 5u};
  return mags[h & 3u] | (((h >> 5) & 1u) << 3);
}

// Scale exponent of reference fills 1-4 for (row, k-block); which = 0 for A, 1 for B.
SMB_HD int fp4_fill_scale_exp(uint32_t row, uint32_t kblock, int fill, int which) {
  if (fill == 1 || fill == 3) {
    return which == 0 ? static_cast<int>(row % 5u) - 2 : static_cast<int>(row % 3u) - 1;
  }
  const uint32_t raw = row * 131071u + kblock * 8191u + static_cast<uint32_t>(which) * 977u;
  return static_cast<int>(hash32(raw) % 5u) - 2;
}

// FP32 source value of the quantised fills (5, 6) for element `index`.
//   fill 5: Gaussian, sigma 1.   fill 6: the same value rounded to bf16 first.
SMB_HD float fp4_source_value(uint32_t index, int fill, uint32_t seed) {
  const float g = gauss12(index, seed);
  return fill == 6 ? bf16_to_f32(f32_to_bf16(g)) : g;
}

// ------------------------------------------------------------------------------- scale packing
// Byte offset of scale (row r, k-block j) in the packed scale buffer of a matrix with
// `kblocks` = K / 32 scale columns (padded up to a multiple of 4).  Rows are grouped in
// bands of 128; a band holds kchunks = ceil(kblocks / 4) chunks of 512 bytes; chunk c is 32
// lines of 16 bytes, line i = rows i, i + 32, i + 64, i + 96 (4 bytes each = 4 k-blocks).
// One chunk is what a single tcgen05.cp.32x128b.warpx4 moves into 4 TMEM columns.
SMB_HD size_t sf_packed_offset(uint32_t r, uint32_t j, uint32_t kblocks) {
  const size_t kchunks = (kblocks + 3u) / 4u;
  const size_t band = r / 128u;
  const uint32_t rr = r % 128u;
  return (band * kchunks + j / 4u) * 512u + (rr % 32u) * 16u + (rr / 32u) * 4u + (j % 4u);
}
SMB_HD size_t sf_packed_bytes(uint64_t rows, uint64_t kblocks) {
  return static_cast<size_t>(((rows + 127u) / 128u) * ((kblocks + 3u) / 4u) * 512u);
}

}  // namespace fmt
}  // namespace smb
