// Scalar codecs shared by host packers and device kernels: bf16 / fp16 / e4m3 /
// e2m1 and the NVFP4 scale-tile address map. Written from the formats; the
// results are compared with the reference's tables and encoders on every bit
// pattern by the test-suite.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#if defined(__CUDACC__)
#define SFQ_HD __host__ __device__ __forceinline__
#else
#define SFQ_HD inline
#endif

namespace sfq {

SFQ_HD uint32_t f32_bits(float f) {
#if defined(__CUDA_ARCH__)
  return __float_as_uint(f);
#else
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
#endif
}
SFQ_HD float bits_f32(uint32_t u) {
#if defined(__CUDA_ARCH__)
  return __uint_as_float(u);
#else
  float f;
  std::memcpy(&f, &u, 4);
  return f;
#endif
}

// E4M3 "fn" (bias 7, no infinities, S.1111.111 = NaN) -> fp32, exact.
// Same values as f8_e4m3_to_f32 (include/slopfab/dtype.h:123-151).
SFQ_HD float e4m3_decode(uint8_t v) {
  const uint32_t sign = uint32_t(v & 0x80u) << 24;
  const uint32_t e = (v >> 3) & 15u, m = v & 7u;
  if (e == 15u && m == 7u) return bits_f32(sign | 0x7FC00000u);
  if (e == 0u) {
    // m * 2^-9: build it from the position of the leading mantissa bit
    if (m == 0u) return bits_f32(sign);
    const uint32_t lead = m >= 4u ? 2u : (m >= 2u ? 1u : 0u);
    const uint32_t frac = (m << (3u - lead)) & 7u;
    return bits_f32(sign | ((lead + 118u) << 23) | (frac << 20));  // 2^(lead-9) * 1.frac
  }
  return bits_f32(sign | ((e + 120u) << 23) | (m << 20));
}

// fp32 -> E4M3, round to nearest even, saturate to 448, NaN -> 0x7F|sign.
// Equals cvt.rn.satfinite.e4m3x2 and f32_to_f8_e4m3_dev (src/cuda/linear_weights.cu:41-68).
SFQ_HD uint8_t e4m3_encode(float f) {
  const uint32_t u = f32_bits(f);
  const uint8_t sign = uint8_t((u >> 24) & 0x80u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a > 0x7F800000u) return uint8_t(sign | 0x7Fu);
  if (a >= 0x43E00000u) return uint8_t(sign | 0x7Eu);  // |f| >= 448
  const int e = int(a >> 23) - 127;
  if (e < -10) return sign;  // below half of the smallest subnormal 2^-9 (2^-10 itself ties to even = 0)
  // Keep 3 fraction bits for normals (e >= -6), fewer for the subnormal binade.
  const int drop = e >= -6 ? 20 : 20 + (-6 - e);
  const uint32_t sig = (a & 0x7FFFFFu) | 0x800000u;
  uint32_t q = sig >> drop;
  const uint32_t rem = sig & ((1u << drop) - 1u), half = 1u << (drop - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  if (e >= -6) {
    // q in [8,16]; 16 carries into the next exponent
    const uint32_t code = (uint32_t(e + 7) << 3) + (q - 8u);
    return uint8_t(sign | (code > 0x7Eu ? 0x7Eu : code));
  }
  return uint8_t(sign | q);  // q in [0,8]; 8 is the smallest normal
}

// E2M1 magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 (f4_e2m1_to_f32, include/slopfab/dtype.h:155-161).
SFQ_HD float e2m1_decode(uint32_t nib) {
  const uint32_t mag = nib & 7u;
  uint32_t bits = 0;
  if (mag == 1u)
    bits = 0x3F000000u;
  else if (mag > 1u)
    bits = ((126u + (mag >> 1)) << 23) | ((mag & 1u) << 22);
  return bits_f32(bits | ((nib & 8u) << 28));
}

// fp32 -> E2M1, nearest, ties to the even code, saturate at 6, the input's sign is
// kept even on a zero result (cvt.rn.satfinite.e2m1x2; host_e2m1,
// tests/detail/nn_weight_fixture.h:299-315).
SFQ_HD uint8_t e2m1_encode(float v) {
  const uint8_t sign = uint8_t((f32_bits(v) >> 28) & 8u);
  const float a = fabsf(v);
  uint8_t mag;
  if (!(a < 5.0f))
    mag = (a == 5.0f) ? 6 : 7;  // 5.0 ties between 4 (code 6) and 6 (code 7): even code 6; NaN saturates
  else if (a <= 0.25f)
    mag = 0;  // 0.25 ties to code 0
  else if (a < 0.75f)
    mag = 1;
  else if (a <= 1.25f)
    mag = 2;  // 0.75 and 1.25 tie to code 2
  else if (a < 1.75f)
    mag = 3;
  else if (a <= 2.5f)
    mag = 4;  // 1.75 and 2.5 tie to code 4
  else if (a < 3.5f)
    mag = 5;
  else
    mag = 6;  // 3.5 ties to code 6; (3.5, 5.0) is nearest 4
  return uint8_t(sign | mag);
}

// Byte offset of the scale of (row, 16-element block) in the 128x4-tiled layout
// (nvfp4_scale_offset, src/cuda/linear_weights.cu:111-115).
SFQ_HD size_t nvfp4_scale_offset(int row, int blk, int blocks_per_row) {
  const size_t tile = size_t(row >> 7) * size_t(blocks_per_row >> 2) + size_t(blk >> 2);
  return tile * 512 + size_t((row & 31) * 16 + ((row & 127) >> 5) * 4 + (blk & 3));
}

// Host-side bf16 / fp16 narrowing with round-to-nearest-even (include/slopfab/dtype.h:54-121).
inline uint16_t host_f32_to_bf16(float f) {
  const uint32_t u = f32_bits(f);
  return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
inline float host_bf16_to_f32(uint16_t v) { return bits_f32(uint32_t(v) << 16); }

}  // namespace sfq
