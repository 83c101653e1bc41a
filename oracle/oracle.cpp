// CPU oracle for the quantized-Linear path of slopfab's DiT.
//
// TEST INFRASTRUCTURE ONLY. Nothing in the product package links, imports or
// calls this file; it exists so that the CUDA kernels can be checked against an
// independent statement of the reference arithmetic, and so that a host
// baseline can be timed. Every function names the reference source it restates
// (paths are relative to the reference project root).
//
// Parity status: every decode/quantize/epilogue rule here is pinned against the
// reference's own golden cases by the CPU test-suite (tests/test_oracle_*.py)
// and, where the reference sources are available, against the reference's own
// code compiled into oracle/_ref/. The W4A8/W6A8/INT8 *encoders* live in the
// product (they have no counterpart in the reference tree) and are therefore
// "parity unpinned" in the encode direction; their decode is fully pinned.
//
// Build: see oracle/Makefile (g++ -O2 -fopenmp -ffp-contract=off).
// All fused multiply-adds the GPU code performs are written as explicit fmaf
// calls, and nothing else may contract, hence -ffp-contract=off.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace {

inline uint32_t bits_of(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
inline float float_of(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// ---------------------------------------------------------------------------
// Scalar conversions. include/slopfab/dtype.h:46-188.
// ---------------------------------------------------------------------------

inline float bf16_to_f32(uint16_t v) { return float_of(uint32_t(v) << 16); }

// Round to nearest even by adding 0x7FFF plus the kept LSB (dtype.h:54-60).
inline uint16_t f32_to_bf16(float f) {
  const uint32_t u = bits_of(f);
  return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

// IEEE binary16 <-> binary32 (dtype.h:62-121), written from the format rather
// than from that file: widen exactly; narrow with round-to-nearest-even,
// overflow to infinity, NaNs keep a quiet payload bit.
inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = uint32_t(h & 0x8000u) << 16;
  const int e = (h >> 10) & 31;
  const uint32_t m = h & 0x3FFu;
  if (e == 31) return float_of(sign | 0x7F800000u | (m << 13));
  if (e == 0) {
    const float mag = std::ldexp(float(m), -24);  // subnormals and zero, exact
    return float_of(bits_of(mag) | sign);
  }
  return float_of(sign | (uint32_t(e + 112) << 23) | (m << 13));
}
inline uint16_t f32_to_f16(float f) {
  const uint32_t u = bits_of(f);
  const uint16_t sign = uint16_t((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return uint16_t(sign | 0x7C00u | ((a & 0x7FFFFFu) ? 0x0200u : 0u));
  const int e = int(a >> 23) - 127;
  if (e >= 16) return uint16_t(sign | 0x7C00u);
  if (e < -25) return sign;  // below half of the smallest subnormal
  // Scale so that one unit is the target's ulp, then round to even.
  const int ulp_exp = e >= -14 ? e - 10 : -24;
  const double scaled = std::ldexp(double(float_of(a)), -ulp_exp);
  double r = std::nearbyint(scaled);  // default rounding mode is to-nearest-even
  uint32_t q = uint32_t(r);
  if (e >= -14) {
    // q in [1024, 2048]; 2048 means the significand carried into the next binade.
    uint32_t out = (uint32_t(e + 15) << 10) + (q - 1024u);
    return uint16_t(sign | out);  // carry propagates into the exponent; 0x7C00 is infinity
  }
  return uint16_t(sign | q);  // subnormal; q == 1024 lands on the smallest normal
}

// E4M3 "fn": bias 7, no infinities, S.1111.111 is NaN (dtype.h:123-151).
inline float e4m3_to_f32(uint8_t v) {
  const int e = (v >> 3) & 15;
  const int m = v & 7;
  float mag;
  if (e == 15 && m == 7)
    return float_of((uint32_t(v & 0x80u) << 24) | 0x7FC00000u);
  if (e == 0)
    mag = std::ldexp(float(m), -9);
  else
    mag = std::ldexp(float(8 + m), e - 10);
  return (v & 0x80u) ? -mag : mag;
}

// Round-to-nearest-even, saturating at 448, NaN -> 0x7F
// (src/cuda/linear_weights.cu:41-68; the hardware's cvt.rn.satfinite.e4m3).
inline uint8_t f32_to_e4m3(float f) {
  const uint8_t sign = uint8_t((bits_of(f) >> 24) & 0x80u);
  if (std::isnan(f)) return uint8_t(sign | 0x7Fu);
  float a = std::fabs(f);
  if (a >= 448.0f) return uint8_t(sign | 0x7Eu);
  if (a == 0.0f) return sign;
  int e = std::ilogb(a);
  if (e < -6) e = -6;
  // One unit of the scaled value is the spacing of the binade: 2^(e-3).
  int q = int(std::nearbyint(std::ldexp(double(a), 3 - e)));
  if (q == 16) {
    q = 8;
    ++e;
  }
  if (e > 8 || (e == 8 && q > 14)) return uint8_t(sign | 0x7Eu);
  if (q < 8) return uint8_t(sign | q);  // subnormal binade (only reachable with e == -6)
  return uint8_t(sign | ((e + 7) << 3) | (q - 8));
}

// The same encoder by exhaustive search over the non-negative codes, ties to
// the even code (tests/detail/nn_weight_fixture.h:286-297). Used by the NVFP4
// fixture packer; kept separate so the two can be compared.
inline uint8_t e4m3_nearest_nonneg(float v) {
  uint8_t best = 0;
  double best_d = 1e300;
  for (int c = 0; c < 0x7F; ++c) {
    const double d = std::fabs(double(e4m3_to_f32(uint8_t(c))) - double(v));
    if (d < best_d || (d == best_d && (c & 1) == 0)) {
      best_d = d;
      best = uint8_t(c);
    }
  }
  return best;
}

const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

inline float e2m1_to_f32(uint8_t nib) {  // dtype.h:155-161
  const float m = kE2M1[nib & 7];
  return (nib & 8) ? -m : m;
}

// Nearest magnitude, ties to the even code, saturate at 6, sign carried even
// onto zero (tests/detail/nn_weight_fixture.h:299-315; cvt.rn.satfinite.e2m1x2).
inline uint8_t f32_to_e2m1(float v) {
  const double a = std::fabs(double(v));
  int mag = 0;
  double best = 1e300;
  for (int c = 0; c < 8; ++c) {
    const double d = std::fabs(double(kE2M1[c]) - a);
    if (d < best || (d == best && (c & 1) == 0)) {
      best = d;
      mag = c;
    }
  }
  return uint8_t(mag | (std::signbit(v) ? 8 : 0));
}

// ---------------------------------------------------------------------------
// NVFP4 scale tiling. src/cuda/linear_weights.cu:111-115,
// tests/detail/nn_weight_fixture.h:35-44.
// Tiles of 128 rows x 4 blocks, 512 bytes each, row-major over (row tile, block
// tile); inside a tile the 128 rows are four groups of 32.
// ---------------------------------------------------------------------------
inline size_t nvfp4_scale_slot(int row, int blk, int blocks_per_row) {
  const size_t tile = size_t(row / 128) * size_t(blocks_per_row / 4) + size_t(blk / 4);
  const int r = row % 128;
  return tile * 512 + size_t(r % 32) * 16 + size_t(r / 32) * 4 + size_t(blk % 4);
}

// ---------------------------------------------------------------------------
// Integer-exact reciprocal square root used by the norm kernels.
// include/slopfab/cuda/deterministic_math.cuh:26-197.
//
// mean = RNE(sum / dim); base = RNE(mean + eps); result = Newton iteration in
// unsigned Q30 fixed point with round-half-even shifts, six steps from a seed
// that depends on the exponent's parity, rounded to 24 bits.
// ---------------------------------------------------------------------------
inline uint64_t shift_rne(uint64_t v, unsigned s) {
  const uint64_t q = v >> s;
  const uint64_t rem = v & ((uint64_t(1) << s) - 1);
  const uint64_t half = uint64_t(1) << (s - 1);
  return q + ((rem > half || (rem == half && (q & 1))) ? 1 : 0);
}
inline int top_bit(uint64_t v) {
  int t = 0;
  while (v >>= 1) ++t;
  return t;
}

// sum / divisor for a positive finite float and a positive integer, rounded to
// nearest even. For a divisor below 2^24 this equals IEEE division by
// float(divisor); it is computed in double (exact quotient rounding is safe
// because the double quotient of a 24-bit by a 24-bit significand cannot sit
// within half a float-ulp of a rounding boundary without being exact) and
// checked against the integer form in the tests.
inline float div_rne(float sum, uint32_t divisor) {
  if (sum == 0.0f) return 0.0f;
  if (std::isinf(sum) || std::isnan(sum)) return sum;
  return sum / float(divisor);
}

inline float rsqrt_q30(float value) {
  const uint32_t bits = bits_of(value);
  const uint32_t mag = bits & 0x7FFFFFFFu;
  if (mag == 0) return float_of((bits & 0x80000000u) | 0x7F800000u);
  if ((bits & 0x80000000u) || mag > 0x7F800000u) return float_of(0x7FC00000u);
  if (mag == 0x7F800000u) return 0.0f;
  uint32_t sig = mag & 0x007FFFFFu;
  int expo;
  if (mag < 0x00800000u) {
    const int t = top_bit(sig);
    expo = t - 149;
    sig <<= unsigned(23 - t);
  } else {
    expo = int(mag >> 23) - 127;
    sig |= 0x00800000u;
  }
  const int odd = expo & 1;
  const uint64_t m = uint64_t(sig) << (7 + odd);  // Q30, in [1,4)
  const int out_scale = -(expo - odd) / 2;
  uint64_t y = odd ? 637534208ull : 872415232ull;
  for (int it = 0; it < 6; ++it) {
    const uint64_t y2 = shift_rne(y * y, 30);
    const uint64_t my2 = shift_rne(m * y2, 30);
    const uint64_t corr = 3ull * (1ull << 30) - my2;
    y = shift_rne(y * corr, 31);
  }
  int t = top_bit(y);
  uint64_t r = shift_rne(y, unsigned(t - 23));
  if (r == (1ull << 24)) {
    r >>= 1;
    ++t;
  }
  const int e = t - 30 + out_scale;
  return float_of((uint32_t(e + 127) << 23) | (uint32_t(r) & 0x007FFFFFu));
}

inline float norm_rsqrt(float sum, uint32_t dim, float eps) {
  const float mean = div_rne(sum, dim);
  const float base = mean + eps;  // IEEE add == the reference's integer add for these operands
  return rsqrt_q30(base);
}

// Sum of squares in the order the block kernel uses
// (src/cuda/nn_kernels.cu:160-168, src/cuda/nn_internal.cuh:21-43):
// 256 threads, thread t owns 8-element packs t, t+256, ...; each thread
// accumulates with fused multiply-add; lanes fold with shfl_down 16,8,4,2,1;
// warp leaders fold the same way in warp 0.
float block_sum_sq(const uint16_t* x, int dim) {
  const int threads = 256;
  float part[256];
  const int packs = dim / 8;
  for (int t = 0; t < threads; ++t) {
    float s = 0.0f;
    for (int p = t; p < packs; p += threads)
      for (int i = 0; i < 8; ++i) {
        const float v = bf16_to_f32(x[p * 8 + i]);
        s = std::fmaf(v, v, s);
      }
    part[t] = s;
  }
  float warp_tot[8];
  for (int w = 0; w < 8; ++w) {
    float lane[32];
    for (int l = 0; l < 32; ++l) lane[l] = part[w * 32 + l];
    for (int off = 16; off > 0; off >>= 1)
      for (int l = 0; l < 32; ++l)
        lane[l] = lane[l] + (l + off < 32 ? lane[l + off] : lane[l]);  // out-of-range shfl_down returns own value
    warp_tot[w] = lane[0];
  }
  float lane[32];
  for (int l = 0; l < 32; ++l) lane[l] = l < 8 ? warp_tot[l] : 0.0f;
  for (int off = 16; off > 0; off >>= 1)
    for (int l = 0; l < 32; ++l) lane[l] = lane[l] + (l + off < 32 ? lane[l + off] : lane[l]);
  return lane[0];
}

// One radix-4 stage of the regular-Hadamard butterfly
// (src/cuda/linear_weights.cu:444-465): left-to-right fp32 additions.
inline void h4_stage(float* v, int n, int stride) {
  for (int base = 0; base < n; base += 4 * stride)
    for (int i = 0; i < stride; ++i) {
      const int j = base + i;
      const float a = v[j], b = v[j + stride], c = v[j + 2 * stride], d = v[j + 3 * stride];
      v[j] = ((a + b) + c) - d;
      v[j + stride] = ((a + b) - c) + d;
      v[j + 2 * stride] = ((a - b) + c) + d;
      v[j + 3 * stride] = ((-a + b) + c) + d;
    }
}

inline int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }
// __float2int_rn: round half to even, saturating.
inline int rint_sat(float f) {
  if (std::isnan(f)) return 0;
  if (f >= 2147483648.0f) return INT32_MAX;
  if (f <= -2147483648.0f) return INT32_MIN;
  return int(std::nearbyint(f));
}

}  // namespace

// ===========================================================================
// Exported scalar conversions
// ===========================================================================
ORC_API uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
ORC_API float orc_bf16_to_f32(uint16_t v) { return bf16_to_f32(v); }
ORC_API uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
ORC_API float orc_f16_to_f32(uint16_t v) { return f16_to_f32(v); }
ORC_API float orc_e4m3_to_f32(uint8_t v) { return e4m3_to_f32(v); }
ORC_API uint8_t orc_f32_to_e4m3(float f) { return f32_to_e4m3(f); }
ORC_API uint8_t orc_e4m3_nearest_nonneg(float f) { return e4m3_nearest_nonneg(f); }
ORC_API float orc_e2m1_to_f32(uint8_t v) { return e2m1_to_f32(v); }
ORC_API uint8_t orc_f32_to_e2m1(float f) { return f32_to_e2m1(f); }
ORC_API uint64_t orc_nvfp4_scale_slot(int row, int blk, int blocks_per_row) {
  return nvfp4_scale_slot(row, blk, blocks_per_row);
}
ORC_API float orc_norm_rsqrt(float sum, uint32_t dim, float eps) { return norm_rsqrt(sum, dim, eps); }
ORC_API float orc_rsqrt_q30(float v) { return rsqrt_q30(v); }

ORC_API void orc_f32_to_bf16_n(const float* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = f32_to_bf16(in[i]);
}
ORC_API void orc_bf16_to_f32_n(const uint16_t* in, float* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = bf16_to_f32(in[i]);
}

// Deterministic test data: xorshift32 mapped to (-scale, scale)
// (tests/harness.cpp:198-208) and Box-Muller over it
// (tests/detail/nn_weight_fixture.h:395-403).
ORC_API void orc_make_data(float* out, size_t n, uint32_t seed, float scale) {
  uint32_t s = seed | 1u;
  for (size_t i = 0; i < n; ++i) {
    s ^= s << 13;
    s ^= s >> 17;
    s ^= s << 5;
    out[i] = ((float(s & 0xFFFFFFu) / 16777216.0f) - 0.5f) * 2.0f * scale;
  }
}
ORC_API void orc_make_gaussian(float* out, size_t n, uint32_t seed, float sigma) {
  std::vector<float> u(2 * n);
  orc_make_data(u.data(), 2 * n, seed, 0.5f);
  for (size_t i = 0; i < n; ++i) {
    const float a = std::max(1e-7f, u[2 * i] + 0.5f);
    out[i] = sigma * std::sqrt(-2.0f * std::log(a)) * std::cos(6.2831853f * (u[2 * i + 1] + 0.5f));
  }
}

// ===========================================================================
// NVFP4
// ===========================================================================

// Quantize a dense [rows, cols] fp32 matrix to the checkpoint's storage form
// (tests/detail/nn_weight_fixture.h:333-360). `dense` (optional) receives what
// the stored bytes mean: e2m1 * (e4m3 * global).
ORC_API void orc_nvfp4_pack(const float* w, int rows, int cols, float global, int high_even,
                            int swizzled, uint8_t* data, uint8_t* scale, float* dense) {
  const int kb = cols / 16;
  std::memset(data, 0, size_t(rows) * cols / 2);
  std::memset(scale, 0, size_t(rows) * kb);
  for (int r = 0; r < rows; ++r)
    for (int b = 0; b < kb; ++b) {
      const float* blk = w + size_t(r) * cols + b * 16;
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) amax = std::max(amax, std::fabs(blk[i]));
      const uint8_t s8 = e4m3_nearest_nonneg(amax / 6.0f / global);
      const float sd = e4m3_to_f32(s8) * global;
      const float inv = sd > 0.0f ? 1.0f / sd : 0.0f;
      scale[swizzled ? nvfp4_scale_slot(r, b, kb) : size_t(r) * kb + b] = s8;
      for (int i = 0; i < 16; ++i) {
        const int col = b * 16 + i;
        const size_t flat = size_t(r) * cols + col;
        const uint8_t q = f32_to_e2m1(blk[i] * inv);
        const bool hi = ((col % 2) == 0) == (high_even != 0);
        data[flat / 2] |= uint8_t(q << (hi ? 4 : 0));
        if (dense) dense[flat] = e2m1_to_f32(q) * sd;
      }
    }
}

// Stored bytes -> bf16, the order of operations of the dequantisation kernel
// (src/cuda/linear_weights.cu:216-245): s = e4m3(scale) * global, then
// e2m1 * s, rounded to bf16. Even element in the high nibble, tiled scales.
ORC_API void orc_nvfp4_dequant_bf16(const uint8_t* data, const uint8_t* scale, float global, int rows,
                                    int cols, uint16_t* out) {
  const int kb = cols / 16;
#pragma omp parallel for
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      const uint8_t byte = data[(size_t(r) * cols + c) / 2];
      const uint8_t nib = (c % 2 == 0) ? uint8_t(byte >> 4) : uint8_t(byte & 15);
      const float s = e4m3_to_f32(scale[nvfp4_scale_slot(r, c / 16, kb)]) * global;
      out[size_t(r) * cols + c] = f32_to_bf16(e2m1_to_f32(nib) * s);
    }
}

// Activation quantizer (src/cuda/nvfp4_gemm.cu:107-158; host twin
// tests/detail/nn_weight_fixture.h:365-383). Low nibble = even element,
// scales row-major [rows, dim/16]. `dense` (optional) = decoded values.
ORC_API void orc_nvfp4_quantize_act(const uint16_t* x, int rows, int dim, uint8_t* packed,
                                    uint8_t* scales, float* dense) {
  const int kb = dim / 16;
#pragma omp parallel for
  for (int r = 0; r < rows; ++r)
    for (int b = 0; b < kb; ++b) {
      float v[16];
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) {
        v[i] = bf16_to_f32(x[size_t(r) * dim + b * 16 + i]);
        amax = std::fmax(amax, std::fabs(v[i]));
      }
      const uint8_t s8 = f32_to_e4m3(amax * (1.0f / 6.0f));
      const float sd = e4m3_to_f32(s8);
      const float inv = sd > 0.0f ? 1.0f / sd : 0.0f;
      if (scales) scales[size_t(r) * kb + b] = s8;
      for (int i = 0; i < 16; i += 2) {
        const uint8_t q0 = f32_to_e2m1(v[i] * inv), q1 = f32_to_e2m1(v[i + 1] * inv);
        if (packed) packed[(size_t(r) * dim + b * 16 + i) / 2] = uint8_t(q0 | (q1 << 4));
        if (dense) {
          dense[size_t(r) * dim + b * 16 + i] = e2m1_to_f32(q0) * sd;
          dense[size_t(r) * dim + b * 16 + i + 1] = e2m1_to_f32(q1) * sd;
        }
      }
    }
}

// ===========================================================================
// W4A8 / W6A8 / INT8 weight decode
// ===========================================================================

// src/cuda/w4a8.cu:44-68. byte = even | odd << 4; q = clamp(rint(codebook[c] * e4m3(s)), -127, 127).
ORC_API void orc_w4a8_decode(const uint8_t* packed, const uint8_t* group_scale, const float* codebook,
                             int rows, int cols, int group, int8_t* out) {
#pragma omp parallel for
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c) {
      const uint8_t byte = packed[size_t(r) * (cols / 2) + c / 2];
      const int code = (c & 1) ? (byte >> 4) : (byte & 15);
      const float s = e4m3_to_f32(group_scale[size_t(r) * (cols / group) + c / group]);
      out[size_t(r) * cols + c] = int8_t(clampi(rint_sat(codebook[code] * s), -127, 127));
    }
}

// src/cuda/w4a8.cu:15-29. Row = cols/2 low-nibble bytes then cols/4 bytes of
// 2-bit highs (shifts 0,2,4,6); level = code - 32.
ORC_API void orc_w6a8_decode(const uint8_t* packed, const uint8_t* group_scale, int rows, int cols,
                             int group, int8_t* out) {
#pragma omp parallel for
  for (int r = 0; r < rows; ++r) {
    const uint8_t* row = packed + size_t(r) * (cols * 3 / 4);
    for (int c = 0; c < cols; ++c) {
      const int lo = (row[c / 2] >> ((c & 1) * 4)) & 15;
      const int hi = (row[cols / 2 + c / 4] >> ((c & 3) * 2)) & 3;
      const int level = (lo | (hi << 4)) - 32;
      const float s = e4m3_to_f32(group_scale[(size_t(r) * cols + c) / group]);
      out[size_t(r) * cols + c] = int8_t(clampi(rint_sat(float(level) * s), -127, 127));
    }
  }
}

// src/cuda/linear_weights.cu:177-192: bf16(int8 * scale[row]).
ORC_API void orc_int8_dequant_bf16(const int8_t* codes, const float* scale, int rows, int cols,
                                   uint16_t* out) {
  for (int r = 0; r < rows; ++r)
    for (int c = 0; c < cols; ++c)
      out[size_t(r) * cols + c] = f32_to_bf16(float(codes[size_t(r) * cols + c]) * scale[r]);
}

// src/core/int8_weight.cpp:66-100: inverse-rotate an int8 ConvRot weight into
// fp16. group in {1,4,16,64,256}; normalisation 1/sqrt(group) folded into the
// row scale; optional flush of fp16 subnormals to signed zero.
ORC_API void orc_int8_unpack_f16(const int8_t* codes, const float* scales, int rows, int cols,
                                 int group, int flush_subnormals, uint16_t* out) {
  const float norm = 1.0f / std::sqrt(float(group));
  for (int r = 0; r < rows; ++r)
    for (int c0 = 0; c0 < cols; c0 += group) {
      float v[256];
      for (int i = 0; i < group; ++i) v[i] = float(codes[size_t(r) * cols + c0 + i]);
      for (int stride = 1; stride < group; stride *= 4) h4_stage(v, group, stride);
      const float factor = scales[r] * norm;
      for (int i = 0; i < group; ++i) {
        uint16_t h = f32_to_f16(v[i] * factor);
        if (flush_subnormals && (h & 0x7C00u) == 0) h &= 0x8000u;
        out[size_t(r) * cols + c0 + i] = h;
      }
    }
}

// src/cuda/linear_weights.cu:150-162: bf16(f8_e4m3(v) * scale), one fp32 scale for the tensor.
ORC_API void orc_f8_dequant_bf16(const uint8_t* src, float scale, size_t n, uint16_t* out) {
  for (size_t i = 0; i < n; ++i) out[i] = f32_to_bf16(e4m3_to_f32(src[i]) * scale);
}

// src/cuda/linear_weights.cu:273-315: bitsandbytes NF4 with double-quantized block scales. High nibble is
// the even element; scale(block) = nested_map[absmax[block]] * nested_absmax[block / nested_block] + offset;
// value = map[code] * scale, rounded to bf16.
ORC_API void orc_nf4_dequant_bf16(const uint8_t* src, const uint8_t* absmax, const float* map, const float* nested_map,
                                  const float* nested_absmax, int block, int nested_block, float offset, size_t n,
                                  uint16_t* out) {
  for (size_t i = 0; i < n; ++i) {
    const size_t b = i / size_t(block);
    // the device compiler contracts this multiply-add into one fused operation
    const float scale = std::fmaf(nested_map[absmax[b]], nested_absmax[b / size_t(nested_block)], offset);
    const uint8_t byte = src[i / 2];
    const int code = (i % 2 == 0) ? (byte >> 4) : (byte & 15);
    out[i] = f32_to_bf16(map[code] * scale);
  }
}

// src/cuda/linear_weights.cu:366-384: f16 -> bf16 through fp32.
ORC_API void orc_f16_to_bf16_n(const uint16_t* in, uint16_t* out, size_t n) {
  for (size_t i = 0; i < n; ++i) out[i] = f32_to_bf16(f16_to_f32(in[i]));
}

// src/cuda/linear_weights.cu:499-509: AWQ activation pre-scale, dst[r, i] = bf16(src[r, i] * scale[i]).
ORC_API void orc_pre_quant_scale_bf16(const uint16_t* x, const uint16_t* scale, int rows, int dim, uint16_t* out) {
  for (int r = 0; r < rows; ++r)
    for (int i = 0; i < dim; ++i)
      out[size_t(r) * dim + i] = f32_to_bf16(bf16_to_f32(x[size_t(r) * dim + i]) * bf16_to_f32(scale[i]));
}

// ===========================================================================
// ConvRot, int8 activation quantizer, integer GEMM, epilogues
// ===========================================================================

// The butterfly in the kernel's own order (src/cuda/linear_weights.cu:422-471):
// fp32 stages with strides 1,4,16,..., then * (1/sqrt(group)) and a bf16 store.
ORC_API void orc_convrot_bf16(const uint16_t* in, int rows, int dim, int group, uint16_t* out) {
  int stages = 0;
  for (int n = 1; n < group; n *= 4) ++stages;
  const float norm = 1.0f / float(1 << stages);
#pragma omp parallel for
  for (int r = 0; r < rows; ++r)
    for (int g0 = 0; g0 < dim; g0 += group) {
      float v[1024];
      for (int i = 0; i < group; ++i) v[i] = bf16_to_f32(in[size_t(r) * dim + g0 + i]);
      for (int stride = 1; stride < group; stride *= 4) h4_stage(v, group, stride);
      for (int i = 0; i < group; ++i) out[size_t(r) * dim + g0 + i] = f32_to_bf16(v[i] * norm);
    }
}

// The same rotation as an explicit matrix product, H = kron^4(h4)/16 with the
// regular (not Sylvester) h4 (docs/convrot_notes.md:5-16;
// tests/detail/nn_kernels_fixture.h:337-366). fp32 in/out, double accumulate.
ORC_API void orc_convrot_dense_f32(const float* in, int rows, int dim, int group, float* out) {
  static const int h4[4][4] = {{1, 1, 1, -1}, {1, 1, -1, 1}, {1, -1, 1, 1}, {-1, 1, 1, 1}};
  int stages = 0;
  for (int n = 1; n < group; n *= 4) ++stages;
  std::vector<float> H(size_t(group) * group);
  for (int i = 0; i < group; ++i)
    for (int j = 0; j < group; ++j) {
      int s = 1, a = i, b = j;
      for (int t = 0; t < stages; ++t) {
        s *= h4[a & 3][b & 3];
        a >>= 2;
        b >>= 2;
      }
      H[size_t(i) * group + j] = float(s) / float(1 << stages);
    }
  for (int r = 0; r < rows; ++r)
    for (int g0 = 0; g0 < dim; g0 += group)
      for (int i = 0; i < group; ++i) {
        double acc = 0.0;
        for (int j = 0; j < group; ++j)
          acc += double(H[size_t(i) * group + j]) * in[size_t(r) * dim + g0 + j];
        out[size_t(r) * dim + g0 + i] = float(acc);
      }
}

// Per-token dynamic int8 (src/cuda/w4a8.cu:193-216): scale = max(amax/127, 1e-30)
// kept in fp32 for the output; the divisor is that scale rounded to bf16; the
// quotient is rounded to bf16 before the nearest-even integer conversion.
ORC_API void orc_quantize_int8_token(const uint16_t* x, int rows, int width, int8_t* q, float* scales) {
#pragma omp parallel for
  for (int r = 0; r < rows; ++r) {
    float amax = 0.0f;
    for (int i = 0; i < width; ++i) amax = std::fmax(amax, std::fabs(bf16_to_f32(x[size_t(r) * width + i])));
    const float scale = std::fmax(amax / 127.0f, 1e-30f);
    scales[r] = scale;
    const float rounded = round_bf16(scale);
    for (int i = 0; i < width; ++i) {
      const float quo = round_bf16(bf16_to_f32(x[size_t(r) * width + i]) / rounded);
      q[size_t(r) * width + i] = int8_t(clampi(rint_sat(quo), -128, 127));
    }
  }
}

// The fp16 / VAE variant with the rotation fused (src/cuda/w4a8.cu:70-124):
// 0.5 per radix-4 stage, amax clamped to 65504 and *multiplied* by 1/127,
// value, scale and quotient rounded through fp16.
ORC_API void orc_quantize_int8_token_f16(const uint16_t* x, int rows, int width, int8_t* q, float* scales) {
  for (int r = 0; r < rows; ++r) {
    std::vector<float> row(width);
    for (int i = 0; i < width; ++i) row[i] = f16_to_f32(x[size_t(r) * width + i]);
    for (int g0 = 0; g0 < width; g0 += 256) {
      float tmp[256];
      float* src = row.data() + g0;
      for (int stage = 0; stage < 4; ++stage) {
        const int stride = 1 << (2 * stage);
        for (int t = 0; t < 256; ++t) {
          const int digit = (t / stride) & 3;
          const int base = t - digit * stride;
          const float x0 = src[base], x1 = src[base + stride], x2 = src[base + 2 * stride], x3 = src[base + 3 * stride];
          float s;
          switch (digit) {
            case 0: s = ((x0 + x1) + x2) - x3; break;
            case 1: s = ((x0 + x1) - x2) + x3; break;
            case 2: s = ((x0 - x1) + x2) + x3; break;
            default: s = ((-x0 + x1) + x2) + x3; break;
          }
          tmp[t] = 0.5f * s;
        }
        std::memcpy(src, tmp, sizeof(tmp));
      }
    }
    float amax = 0.0f;
    for (int i = 0; i < width; ++i) amax = std::fmax(amax, std::fabs(row[i]));
    const float scale = std::fmax(std::fmin(amax, 65504.0f) * (1.0f / 127.0f), 1.0e-30f);
    scales[r] = scale;
    const float rs = f16_to_f32(f32_to_f16(scale));
    for (int i = 0; i < width; ++i) {
      const float rv = f16_to_f32(f32_to_f16(row[i]));
      const float quo = f16_to_f32(f32_to_f16(rv / rs));
      q[size_t(r) * width + i] = int8_t(clampi(rint_sat(quo), -128, 127));
    }
  }
}

// acc[m, n] = sum_k a[m, k] * w[n, k]  (the cuBLAS int8 GemmEx of src/cuda/linear.cu:202-203; exact).
ORC_API void orc_int8_gemm(const int8_t* a, const int8_t* w, int M, int N, int K, int32_t* acc) {
#pragma omp parallel for collapse(2)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const int8_t* ar = a + size_t(m) * K;
      const int8_t* wr = w + size_t(n) * K;
      int32_t s = 0;
      for (int k = 0; k < K; ++k) s += int32_t(ar[k]) * int32_t(wr[k]);
      acc[size_t(m) * N + n] = s;
    }
}

// src/cuda/w4a8.cu:218-223: bf16((float(acc) * row) * channel).
ORC_API void orc_w4a8_output_bf16(const int32_t* acc, const float* row_scale, const float* chan_scale,
                                  int M, int N, uint16_t* y) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n)
      y[size_t(m) * N + n] = f32_to_bf16((float(acc[size_t(m) * N + n]) * row_scale[m]) * chan_scale[n]);
}

// src/cuda/linear_weights.cu:483-491: y = bf16(float(y) + bias[n]); the bias
// is fp32 (bias_is_bf16 == 0) or bf16.
ORC_API void orc_add_bias_bf16(uint16_t* y, const void* bias, int bias_is_bf16, int M, int N) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      const float b = bias_is_bf16 ? bf16_to_f32(static_cast<const uint16_t*>(bias)[n])
                                   : static_cast<const float*>(bias)[n];
      y[size_t(m) * N + n] = f32_to_bf16(bf16_to_f32(y[size_t(m) * N + n]) + b);
    }
}

// src/cuda/nn_pointwise.cu:74-81, in place on bf16. The device code contracts
// v + c*v*v*v into one fused multiply-add; tanhf here is the host library's,
// which may differ from the device's in the last ulp, so this one is a
// tolerance reference (one bf16 ulp), not a bit-exact one.
ORC_API void orc_gelu_tanh_bf16(uint16_t* y, size_t n) {
  for (size_t i = 0; i < n; ++i) {
    const float v = bf16_to_f32(y[i]);
    const float inner = std::fmaf((0.044715f * v) * v, v, v);
    y[i] = f32_to_bf16((0.5f * v) * (1.0f + std::tanh(0.7978845608028654f * inner)));
  }
}

// src/cuda/nn_pointwise.cu:46-64: silu(fused[:, :inner]) * fused[:, inner:].
ORC_API void orc_swiglu_bf16(const uint16_t* fused, int rows, int inner, uint16_t* out) {
  for (int r = 0; r < rows; ++r)
    for (int i = 0; i < inner; ++i) {
      const float g = bf16_to_f32(fused[size_t(r) * 2 * inner + i]);
      const float v = bf16_to_f32(fused[size_t(r) * 2 * inner + inner + i]);
      out[size_t(r) * inner + i] = f32_to_bf16((g / (1.0f + std::exp(-g))) * v);
    }
}

// src/cuda/nn_pointwise.cu:15-37: x = bf16(fma(gate[a[r]], branch, x)).
ORC_API void orc_add_gated_bf16(uint16_t* x, const uint16_t* branch, const float* gate, const int32_t* a,
                                int rows, int dim) {
  for (int r = 0; r < rows; ++r)
    for (int i = 0; i < dim; ++i) {
      const float g = gate[size_t(a[r]) * dim + i];
      x[size_t(r) * dim + i] =
          f32_to_bf16(std::fmaf(g, bf16_to_f32(branch[size_t(r) * dim + i]), bf16_to_f32(x[size_t(r) * dim + i])));
    }
}

// Head-wise RMSNorm on the warp-per-row path (rmsnorm_warp_kernel, src/cuda/nn_kernels.cu:100-136: 16 lanes x 8 channels,
// per-lane fma chain, xor butterfly 16, 8, 4, 2, 1 over 32 lanes of which 16 hold zero) followed by MM-RoPE
// (rope_h3_kernel, src/cuda/nn_position.cu:15-68) on x [rows, heads, 128] with a row pitch; w and cos may be null.
static float rope_flush(float v) {
  uint32_t b; std::memcpy(&b, &v, 4);
  if ((b & 0x7fffffffu) < 0x00800000u) { b &= 0x80000000u; std::memcpy(&v, &b, 4); }
  return v;
}
static float rope_bf16_in(uint16_t bits) { return (bits & 0x7fffu) < 0x0080u ? bf16_to_f32(uint16_t(bits & 0x8000u)) : bf16_to_f32(bits); }
static uint16_t rope_bf16_out(float v) {
  const uint16_t bits = f32_to_bf16(v);
  return (bits & 0x7fffu) < 0x0080u ? uint16_t(bits & 0x8000u) : bits;
}
ORC_API void orc_head_norm_rope(uint16_t* x, int ld, const uint16_t* w, const float* cos_tab, const float* sin_tab, int rows, int heads,
                                float eps) {
#pragma omp parallel for collapse(2)
  for (int row = 0; row < rows; ++row)
    for (int head = 0; head < heads; ++head) {
      uint16_t* v = x + size_t(row) * ld + head * 128;
      if (w != nullptr) {
        float lane_sum[32] = {};
        for (int lane = 0; lane < 16; ++lane)
          for (int i = 0; i < 8; ++i) {
            const float b = bf16_to_f32(v[lane * 8 + i]);
            lane_sum[lane] = std::fmaf(b, b, lane_sum[lane]);
          }
        for (int offset = 16; offset > 0; offset >>= 1) {
          float next[32];
          for (int lane = 0; lane < 32; ++lane) next[lane] = lane_sum[lane] + lane_sum[lane ^ offset];
          std::memcpy(lane_sum, next, sizeof(next));
        }
        const float inv = norm_rsqrt(lane_sum[0], 128u, eps);
        for (int c = 0; c < 128; ++c) v[c] = f32_to_bf16((bf16_to_f32(v[c]) * inv) * bf16_to_f32(w[c]));
      }
      if (cos_tab != nullptr) {
        for (int j = 0; j < 48; ++j) {
          const float c = rope_flush(cos_tab[size_t(row) * 96 + j]), s = rope_flush(sin_tab[size_t(row) * 96 + j]);
          const float lo = rope_bf16_in(v[j]), hi = rope_bf16_in(v[j + 48]);
          const float left = rope_flush(lo * c), right = rope_flush(hi * s), base = rope_flush(hi * c);
          const float product = lo * s;
          uint32_t pb, ab, bb;
          std::memcpy(&pb, &product, 4); std::memcpy(&ab, &lo, 4); std::memcpy(&bb, &s, 4);
          const bool tiny = (pb & 0x7fffffffu) < 0x00800000u && (ab & 0x7fffffffu) != 0u && (bb & 0x7fffffffu) != 0u;
          v[j] = rope_bf16_out(left - right);
          v[j + 48] = rope_bf16_out(tiny ? base : std::fmaf(lo, s, base));
        }
      }
    }
}

// Dense attention, no mask (cpu_attention, tests/detail/nn_kernels_fixture.h:193-231): fp64 scores, softmax and
// weighted sum; q is [seq_q, heads*dim], k and v are [seq_kv, kv_heads*dim], all fp32 holding bf16 values.
ORC_API void orc_attention(const float* q, const float* k, const float* v, int seq_q, int seq_kv, int heads, int kv_heads,
                           int head_dim, float scale, float* out) {
  const int qld = heads * head_dim, kvld = kv_heads * head_dim, group = heads / kv_heads;
#pragma omp parallel for collapse(2)
  for (int h = 0; h < heads; ++h)
    for (int i = 0; i < seq_q; ++i) {
      const int kv = h / group;
      std::vector<double> p(seq_kv);
      double m = -1e300;
      for (int j = 0; j < seq_kv; ++j) {
        double dot = 0.0;
        for (int d = 0; d < head_dim; ++d) dot += double(q[size_t(i) * qld + h * head_dim + d]) * k[size_t(j) * kvld + kv * head_dim + d];
        p[j] = dot * scale;
        m = std::max(m, p[j]);
      }
      double sum = 0.0;
      for (int j = 0; j < seq_kv; ++j) {
        p[j] = std::exp(p[j] - m);
        sum += p[j];
      }
      for (int d = 0; d < head_dim; ++d) {
        double acc = 0.0;
        for (int j = 0; j < seq_kv; ++j) acc += p[j] * v[size_t(j) * kvld + kv * head_dim + d];
        out[size_t(i) * qld + h * head_dim + d] = float(acc / sum);
      }
    }
}

// adaLN table expansion, src/cuda/dit_kernels.cu:61-90: acc = bias[p]; acc = fmaf(w[p,k], code[t,k], acc), k ascending;
// destination [param][t][modality][channel] with p = (modality * num_param + param) * channels + channel.
ORC_API void orc_adaln_expand(const float* w, const float* bias, const float* code, float* out, int num_t, int num_modality,
                              int num_param, int channels, int rank) {
  const int features = num_modality * num_param * channels;
  for (int ti = 0; ti < num_t; ++ti)
#pragma omp parallel for
    for (int p = 0; p < features; ++p) {
      float acc = bias[p];
      for (int k = 0; k < rank; ++k) acc = std::fmaf(w[size_t(p) * rank + k], code[size_t(ti) * rank + k], acc);
      const int channel = p % channels, rest = p / channels;
      const int param = rest % num_param, modality = rest / num_param;
      out[(size_t(param) * num_t * num_modality + size_t(ti) * num_modality + modality) * channels + channel] = acc;
    }
}

// LoRA side branch, the CPU statement the reference's own test holds its kernels to
// (tests/test_lora_backends.cu:84-101): sequential fma in index order, hidden rounded to bf16, the product
// rounded to bf16, then added to y and rounded again. a: [rank, in] and b: [out_total, rank] as fp32 (rounded
// to bf16 here, as LoraRunner::attach does, src/cuda/lora.cu:25-27); rows [offset, offset + out) of b are used.
ORC_API void orc_lora_apply(const uint16_t* x, int rows, const float* a, const float* b, int rank, int in, int offset,
                            int out, uint16_t* y) {
  std::vector<float> ab(size_t(rank) * in), bb(size_t(out) * rank);
  for (size_t i = 0; i < ab.size(); ++i) ab[i] = bf16_to_f32(f32_to_bf16(a[i]));
  for (int o = 0; o < out; ++o)
    for (int r = 0; r < rank; ++r) bb[size_t(o) * rank + r] = bf16_to_f32(f32_to_bf16(b[size_t(o + offset) * rank + r]));
#pragma omp parallel for
  for (int row = 0; row < rows; ++row) {
    std::vector<float> mid(rank);
    for (int r = 0; r < rank; ++r) {
      float sum = 0.0f;
      for (int i = 0; i < in; ++i) sum = std::fmaf(bf16_to_f32(x[size_t(row) * in + i]), ab[size_t(r) * in + i], sum);
      mid[r] = bf16_to_f32(f32_to_bf16(sum));
    }
    for (int o = 0; o < out; ++o) {
      float sum = 0.0f;
      for (int r = 0; r < rank; ++r) sum = std::fmaf(mid[r], bb[size_t(o) * rank + r], sum);
      const size_t i = size_t(row) * out + o;
      y[i] = f32_to_bf16(bf16_to_f32(y[i]) + bf16_to_f32(f32_to_bf16(sum)));
    }
  }
}

// ===========================================================================
// RMSNorm and adaLN modulation
// ===========================================================================

// Bit-level restatement of the block kernels (src/cuda/nn_kernels.cu:13-48,
// 153-198) for dim % 8 == 0: out = bf16(((x * inv) * w)) or
// bf16(fma((x * inv) * w, 1 + scale[a[r]], shift[a[r]])).
ORC_API void orc_rmsnorm_bf16(const uint16_t* x, const uint16_t* w, const float* scale, const float* shift,
                              const int32_t* a, int rows, int dim, float eps, uint16_t* out) {
#pragma omp parallel for
  for (int r = 0; r < rows; ++r) {
    const uint16_t* xr = x + size_t(r) * dim;
    const float inv = norm_rsqrt(block_sum_sq(xr, dim), uint32_t(dim), eps);
    for (int i = 0; i < dim; ++i) {
      float n = (bf16_to_f32(xr[i]) * inv) * bf16_to_f32(w[i]);
      if (scale) {
        const size_t mod = size_t(a[r]) * dim + i;
        n = std::fmaf(n, 1.0f + scale[mod], shift[mod]);
      }
      out[size_t(r) * dim + i] = f32_to_bf16(n);
    }
  }
}

// The specification form in double (tests/detail/nn_kernels_fixture.h:155-189),
// fp32 in/out, for tolerance checks that do not depend on reduction order.
ORC_API void orc_rmsnorm_spec_f32(const float* x, const float* w, const float* scale, const float* shift,
                                  const int32_t* a, int rows, int dim, float eps, float* out) {
  for (int r = 0; r < rows; ++r) {
    double ss = 0.0;
    for (int i = 0; i < dim; ++i) ss += double(x[size_t(r) * dim + i]) * x[size_t(r) * dim + i];
    const double inv = 1.0 / std::sqrt(ss / dim + eps);
    for (int i = 0; i < dim; ++i) {
      float n = float(x[size_t(r) * dim + i] * inv * w[i]);
      if (scale) {
        const size_t mod = size_t(a[r]) * dim + i;
        n = n * (1.0f + scale[mod]) + shift[mod];
      }
      out[size_t(r) * dim + i] = n;
    }
  }
}

// ===========================================================================
// Dense reference products
// ===========================================================================

// C = A * B^T with double accumulation (tests/detail/nn_kernels_fixture.h:323-335).
ORC_API void orc_matmul_nt(const float* A, const float* B, int M, int N, int K, float* C) {
#pragma omp parallel for collapse(2)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      double acc = 0.0;
      const float* ar = A + size_t(m) * K;
      const float* br = B + size_t(n) * K;
      for (int k = 0; k < K; ++k) acc += double(ar[k]) * br[k];
      C[size_t(m) * N + n] = float(acc);
    }
}

// fp32-accumulate blocked product used for the timed host baseline: the
// reference's host path is "decode to a dense fp32 matrix, then x * W^T"; this
// is that product with all cores, and is only ever timed, never checked against.
ORC_API void orc_matmul_nt_fast(const float* A, const float* B, int M, int N, int K, float* C) {
  const int BN = 64, BK = 256;
#pragma omp parallel for collapse(2) schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n0 = 0; n0 < N; n0 += BN) {
      float acc[BN];
      const int nb = std::min(BN, N - n0);
      for (int j = 0; j < nb; ++j) acc[j] = 0.0f;
      for (int k0 = 0; k0 < K; k0 += BK) {
        const int kb = std::min(BK, K - k0);
        const float* ar = A + size_t(m) * K + k0;
        for (int j = 0; j < nb; ++j) {
          const float* br = B + size_t(n0 + j) * K + k0;
          float s = 0.0f;
#pragma omp simd reduction(+ : s)
          for (int k = 0; k < kb; ++k) s += ar[k] * br[k];
          acc[j] += s;
        }
      }
      for (int j = 0; j < nb; ++j) C[size_t(m) * N + n0 + j] = acc[j];
    }
}

// Sets the OpenMP team size of the timed host path. A launcher such as torch.distributed.run exports
// OMP_NUM_THREADS=1 to its workers; the CPU baseline must state, and use, the cores the box really has.
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORC_API int orc_num_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// ===========================================================================
// Whole-Linear oracles
// ===========================================================================

enum { ORC_ACT_NONE = 0, ORC_ACT_GELU_TANH = 1 };

// NVFP4 Linear with fp4 activations ("oracle B"): the arithmetic definition of
// the native kernel (src/cuda/nvfp4_gemm.cu:346-485): y = bf16(global *
// sum(a_q * w_q)) with a_q the quantized activation and w_q = e2m1 * e4m3
// (no global), accumulated here in double; then the bias re-rounding of
// src/cuda/linear_weights.cu:483-491 and the optional in-place GELU.
ORC_API void orc_nvfp4_linear(const uint16_t* x, int M, const uint8_t* wdata, const uint8_t* wscale,
                              float global, int N, int K, const float* bias, int act, uint16_t* y) {
  std::vector<float> a(size_t(M) * K), w(size_t(N) * K);
  orc_nvfp4_quantize_act(x, M, K, nullptr, nullptr, a.data());
  const int kb = K / 16;
#pragma omp parallel for
  for (int n = 0; n < N; ++n)
    for (int k = 0; k < K; ++k) {
      const uint8_t byte = wdata[(size_t(n) * K + k) / 2];
      const uint8_t nib = (k % 2 == 0) ? uint8_t(byte >> 4) : uint8_t(byte & 15);
      w[size_t(n) * K + k] = e2m1_to_f32(nib) * e4m3_to_f32(wscale[nvfp4_scale_slot(n, k / 16, kb)]);
    }
  std::vector<float> c(size_t(M) * N);
  orc_matmul_nt(a.data(), w.data(), M, N, K, c.data());
  for (size_t i = 0; i < c.size(); ++i) y[i] = f32_to_bf16(c[i] * global);
  if (bias) orc_add_bias_bf16(y, bias, 0, M, N);
  if (act == ORC_ACT_GELU_TANH) orc_gelu_tanh_bf16(y, size_t(M) * N);
}

// NVFP4 Linear with bf16 activations ("oracle A", the dequantize-then-GEMM
// path of src/cuda/linear.cu:227-248): y = bf16(x * bf16(W)^T), then bias.
ORC_API void orc_nvfp4_linear_dequant(const uint16_t* x, int M, const uint8_t* wdata, const uint8_t* wscale,
                                      float global, int N, int K, const float* bias, uint16_t* y) {
  std::vector<uint16_t> wb(size_t(N) * K);
  orc_nvfp4_dequant_bf16(wdata, wscale, global, N, K, wb.data());
  std::vector<float> a(size_t(M) * K), w(size_t(N) * K), c(size_t(M) * N);
  orc_bf16_to_f32_n(x, a.data(), a.size());
  orc_bf16_to_f32_n(wb.data(), w.data(), w.size());
  orc_matmul_nt(a.data(), w.data(), M, N, K, c.data());
  orc_f32_to_bf16_n(c.data(), y, c.size());
  if (bias) orc_add_bias_bf16(y, bias, 0, M, N);
}

// W4A8 / W6A8 Linear, the integer pipeline of src/cuda/linear.cu:188-206.
// bits = 4 or 6. Optional outputs expose every intermediate for parity checks.
ORC_API void orc_packed_int8_linear(const uint16_t* x, int M, const uint8_t* packed, const uint8_t* s_rel,
                                    const float* s_channel, const float* codebook, int bits, int group,
                                    int N, int K, const void* bias, int bias_is_bf16, int act,
                                    uint16_t* y, int8_t* w8_out, uint16_t* rot_out, int8_t* q_out,
                                    float* row_scale_out, int32_t* acc_out) {
  std::vector<int8_t> w8(size_t(N) * K), q(size_t(M) * K);
  std::vector<uint16_t> rot(size_t(M) * K);
  std::vector<float> rs(M);
  std::vector<int32_t> acc(size_t(M) * N);
  if (bits == 4)
    orc_w4a8_decode(packed, s_rel, codebook, N, K, group, w8.data());
  else
    orc_w6a8_decode(packed, s_rel, N, K, group, w8.data());
  orc_convrot_bf16(x, M, K, 256, rot.data());
  orc_quantize_int8_token(rot.data(), M, K, q.data(), rs.data());
  orc_int8_gemm(q.data(), w8.data(), M, N, K, acc.data());
  orc_w4a8_output_bf16(acc.data(), rs.data(), s_channel, M, N, y);
  if (bias) orc_add_bias_bf16(y, bias, bias_is_bf16, M, N);
  if (act == ORC_ACT_GELU_TANH) orc_gelu_tanh_bf16(y, size_t(M) * N);
  if (w8_out) std::memcpy(w8_out, w8.data(), w8.size());
  if (rot_out) std::memcpy(rot_out, rot.data(), rot.size() * 2);
  if (q_out) std::memcpy(q_out, q.data(), q.size());
  if (row_scale_out) std::memcpy(row_scale_out, rs.data(), rs.size() * 4);
  if (acc_out) std::memcpy(acc_out, acc.data(), acc.size() * 4);
}

// The timed host baseline: decode the packed weight to dense fp32
// (include/slopfab/dtype.h tables; W4/W6 per src/cuda/w4a8.cu:15-68) and
// multiply (tests/detail/nn_kernels_fixture.h:323-335, fp32 accumulate, all
// cores). format: 0 = NVFP4, 4 = W4A8, 6 = W6A8. Returns nothing useful; the
// caller times it.
ORC_API void orc_host_dequant_matmul(int format, const uint16_t* x, int M, const uint8_t* wdata,
                                     const uint8_t* wscale, const float* s_channel, const float* codebook,
                                     float global, int group, int N, int K, float* y) {
  std::vector<float> w(size_t(N) * K), a(size_t(M) * K);
  if (format == 0) {
    std::vector<uint16_t> wb(size_t(N) * K);
    orc_nvfp4_dequant_bf16(wdata, wscale, global, N, K, wb.data());
    orc_bf16_to_f32_n(wb.data(), w.data(), w.size());
    orc_bf16_to_f32_n(x, a.data(), a.size());
  } else {
    std::vector<int8_t> w8(size_t(N) * K);
    if (format == 4)
      orc_w4a8_decode(wdata, wscale, codebook, N, K, group, w8.data());
    else
      orc_w6a8_decode(wdata, wscale, N, K, group, w8.data());
#pragma omp parallel for
    for (int n = 0; n < N; ++n)
      for (int k = 0; k < K; ++k) w[size_t(n) * K + k] = float(w8[size_t(n) * K + k]) * s_channel[n];
    std::vector<uint16_t> rot(size_t(M) * K);
    orc_convrot_bf16(x, M, K, 256, rot.data());
    orc_bf16_to_f32_n(rot.data(), a.data(), a.size());
  }
  orc_matmul_nt_fast(a.data(), w.data(), M, N, K, y);
}

// Comparison metrics with the reference's definitions
// (include/slopfab/tensor_convert.h:25-91): max |r-a|, ||r-a||/||r||, and the
// mean-subtracted Pearson correlation. out[0..2].
ORC_API void orc_compare_bf16(const uint16_t* ref, const uint16_t* got, size_t n, double* out) {
  double max_abs = 0, num = 0, den = 0, sr = 0, sg = 0;
  for (size_t i = 0; i < n; ++i) {
    const double r = bf16_to_f32(ref[i]), g = bf16_to_f32(got[i]);
    max_abs = std::max(max_abs, std::fabs(r - g));
    num += (r - g) * (r - g);
    den += r * r;
    sr += r;
    sg += g;
  }
  const double mr = sr / double(n), mg = sg / double(n);
  double crr = 0, cgg = 0, crg = 0;
  for (size_t i = 0; i < n; ++i) {
    const double r = bf16_to_f32(ref[i]) - mr, g = bf16_to_f32(got[i]) - mg;
    crr += r * r;
    cgg += g * g;
    crg += r * g;
  }
  out[0] = max_abs;
  out[1] = den > 0 ? std::sqrt(num / den) : 0.0;
  out[2] = (crr > 0 && cgg > 0) ? crg / std::sqrt(crr * cgg) : 0.0;
}
