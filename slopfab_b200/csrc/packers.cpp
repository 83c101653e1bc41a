// Host weight packers: dense fp32 [out, in] -> the on-disk byte layouts the DiT loads.
//
// NVFP4 follows the reference's fixture packer byte for byte
// (tests/detail/nn_weight_fixture.h:333-360). The reference ships NO encoder for W4A8,
// W6A8 or INT8 weights -- its checkpoints come from a third-party quantizer -- so the
// encoding rules below are this library's own; what is fixed by the reference is the
// layout (docs/w4a8.md, docs/w6a8.md), the validity rules of
// validate_packed_int8_weight (src/core/w4a8.cpp:127-162) and the decode
// (src/cuda/w4a8.cu:15-68), and the tests hold the encoders to those.
#include "packers.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "codec.cuh"

namespace sfq {
namespace {

// y = H x per 256 (or `group`) elements, H = kron(h4,...)/sqrt(group), regular Hadamard, in double.
void rotate_row(const float* in, double* out, int n, int group) {
  std::vector<double> v(group);
  for (int g0 = 0; g0 < n; g0 += group) {
    for (int i = 0; i < group; ++i) v[i] = in[g0 + i];
    for (int stride = 1; stride < group; stride *= 4)
      for (int base = 0; base < group; base += 4 * stride)
        for (int i = 0; i < stride; ++i) {
          const int j = base + i;
          const double a = v[j], b = v[j + stride], c = v[j + 2 * stride], d = v[j + 3 * stride];
          v[j] = a + b + c - d;
          v[j + stride] = a + b - c + d;
          v[j + 2 * stride] = a - b + c + d;
          v[j + 3 * stride] = -a + b + c + d;
        }
    const double norm = 1.0 / std::sqrt(double(group));
    for (int i = 0; i < group; ++i) out[g0 + i] = v[i] * norm;
  }
}

inline int rint_clamp(float f, int lo, int hi) {
  const int q = int(std::nearbyint(f));
  return q < lo ? lo : (q > hi ? hi : q);
}

// Picks the E4M3 group scale (a non-negative, non-NaN byte) and the codes that minimise the squared
// error of the DECODED int8 values, clamp(rint(level * scale), -127, 127), against the targets.
// `level_of(code)` maps a code to its level; codes run over [0, n_codes).
template <class LevelOf>
uint8_t fit_group(const double* target, int n, int n_codes, double max_level, LevelOf level_of, uint8_t* codes) {
  double amax = 0.0;
  for (int i = 0; i < n; ++i) amax = std::max(amax, std::fabs(target[i]));
  if (amax == 0.0) {
    int zero_code = 0;
    for (int c = 0; c < n_codes; ++c)
      if (level_of(c) == 0.0f) zero_code = c;
    for (int i = 0; i < n; ++i) codes[i] = uint8_t(zero_code);
    return 0x38;  // 1.0: any scale decodes level 0 to 0
  }
  const uint8_t centre = e4m3_encode(float(amax / max_level));
  uint8_t best_scale = 0;
  double best_err = 1e300;
  std::vector<uint8_t> trial(n);
  for (int delta = -2; delta <= 2; ++delta) {
    const int sb = int(centre) + delta;
    if (sb < 1 || sb > 0x7E) continue;
    const float s = e4m3_decode(uint8_t(sb));
    double err = 0.0;
    for (int i = 0; i < n; ++i) {
      double e_best = 1e300;
      int c_best = 0;
      for (int c = 0; c < n_codes; ++c) {
        const double q = rint_clamp(level_of(c) * s, -127, 127);
        const double e = (q - target[i]) * (q - target[i]);
        if (e < e_best) e_best = e, c_best = c;
      }
      trial[i] = uint8_t(c_best);
      err += e_best;
    }
    if (err < best_err) {
      best_err = err;
      best_scale = uint8_t(sb);
      std::memcpy(codes, trial.data(), n);
    }
  }
  return best_scale;
}

}  // namespace

void pack_nvfp4(const float* w, int rows, int cols, float global, uint8_t* data, uint8_t* scale_tiled) {
  if (!w || !data || !scale_tiled) throw std::invalid_argument("pack_nvfp4: null buffer");
  if (rows <= 0 || cols <= 0 || rows % 128 != 0 || cols % 64 != 0)
    throw std::invalid_argument("pack_nvfp4: needs out_features % 128 == 0 and in_features % 64 == 0");
  if (!(global > 0.0f) || !std::isfinite(global)) throw std::invalid_argument("pack_nvfp4: global scale must be positive");
  const int kb = cols / 16;
  std::memset(data, 0, size_t(rows) * cols / 2);
#pragma omp parallel for
  for (int r = 0; r < rows; ++r)
    for (int b = 0; b < kb; ++b) {
      const float* blk = w + size_t(r) * cols + b * 16;
      float amax = 0.0f;
      for (int i = 0; i < 16; ++i) amax = std::max(amax, std::fabs(blk[i]));
      const uint8_t s8 = e4m3_encode(amax / 6.0f / global) & 0x7Fu;
      const float sd = e4m3_decode(s8) * global;
      const float inv = sd > 0.0f ? 1.0f / sd : 0.0f;
      scale_tiled[nvfp4_scale_offset(r, b, kb)] = s8;
      for (int i = 0; i < 16; i += 2) {
        const uint8_t even = e2m1_encode(blk[i] * inv), odd = e2m1_encode(blk[i + 1] * inv);
        data[(size_t(r) * cols + b * 16 + i) / 2] = uint8_t((even << 4) | odd);  // even element in the high nibble
      }
    }
}

void pack_w4a8(const float* w, int rows, int cols, int8_t* packed, uint8_t* group_scale, float* channel_scale,
               float* codebook16) {
  if (!w || !packed || !group_scale || !channel_scale || !codebook16) throw std::invalid_argument("pack_w4a8: null buffer");
  if (rows <= 0 || cols <= 0 || cols % 256 != 0) throw std::invalid_argument("pack_w4a8: in_features must be a positive multiple of 256");
  for (int i = 0; i < 16; ++i) codebook16[i] = float(i - 8);
#pragma omp parallel for
  for (int r = 0; r < rows; ++r) {
    std::vector<double> rot(cols);
    rotate_row(w + size_t(r) * cols, rot.data(), cols, 256);
    double amax = 0.0;
    for (int i = 0; i < cols; ++i) amax = std::max(amax, std::fabs(rot[i]));
    const float ch = amax > 0.0 ? float(amax / 127.0) : 1.0f;
    channel_scale[r] = ch;
    for (int i = 0; i < cols; ++i) rot[i] /= double(ch);
    uint8_t codes[16];
    for (int g = 0; g < cols / 16; ++g) {
      group_scale[size_t(r) * (cols / 16) + g] =
          fit_group(rot.data() + g * 16, 16, 16, 8.0, [](int c) { return float(c - 8); }, codes);
      for (int i = 0; i < 16; i += 2)
        packed[size_t(r) * (cols / 2) + g * 8 + i / 2] = int8_t(uint8_t(codes[i] | (codes[i + 1] << 4)));  // even element low
    }
  }
}

void pack_w6a8(const float* w, int rows, int cols, int group, int8_t* packed, uint8_t* group_scale, float* channel_scale) {
  if (!w || !packed || !group_scale || !channel_scale) throw std::invalid_argument("pack_w6a8: null buffer");
  if (rows <= 0 || cols <= 0 || cols % 256 != 0 || group < 16 || group % 16 != 0 || cols % group != 0)
    throw std::invalid_argument("pack_w6a8: in_features % 256 == 0, group a multiple of 16 dividing in_features");
  const size_t row_bytes = size_t(cols) * 3 / 4;
  std::memset(packed, 0, size_t(rows) * row_bytes);
#pragma omp parallel for
  for (int r = 0; r < rows; ++r) {
    std::vector<double> rot(cols);
    std::vector<uint8_t> codes(group);
    rotate_row(w + size_t(r) * cols, rot.data(), cols, 256);
    double amax = 0.0;
    for (int i = 0; i < cols; ++i) amax = std::max(amax, std::fabs(rot[i]));
    const float ch = amax > 0.0 ? float(amax / 127.0) : 1.0f;
    channel_scale[r] = ch;
    for (int i = 0; i < cols; ++i) rot[i] /= double(ch);
    uint8_t* row = reinterpret_cast<uint8_t*>(packed) + size_t(r) * row_bytes;
    for (int g = 0; g < cols / group; ++g) {
      group_scale[size_t(r) * (cols / group) + g] =
          fit_group(rot.data() + g * group, group, 64, 31.0, [](int c) { return float(c - 32); }, codes.data());
      for (int i = 0; i < group; ++i) {
        const int col = g * group + i;
        row[col / 2] |= uint8_t((codes[i] & 15) << ((col & 1) * 4));
        row[cols / 2 + col / 4] |= uint8_t((codes[i] >> 4) << ((col & 3) * 2));
      }
    }
  }
}

void pack_int8(const float* w, int rows, int cols, int convrot_group, int8_t* codes, float* scale) {
  if (!w || !codes || !scale) throw std::invalid_argument("pack_int8: null buffer");
  if (rows <= 0 || cols <= 0) throw std::invalid_argument("pack_int8: dimensions must be positive");
  if (convrot_group != 0 && convrot_group != 4 && convrot_group != 16 && convrot_group != 64 && convrot_group != 256)
    throw std::invalid_argument("pack_int8: ConvRot group must be 4, 16, 64 or 256");
  const int group = (convrot_group > 0 && cols % convrot_group == 0) ? convrot_group : 1;  // the quantizer skips ragged rows
#pragma omp parallel for
  for (int r = 0; r < rows; ++r) {
    std::vector<double> rot(cols);
    if (group > 1)
      rotate_row(w + size_t(r) * cols, rot.data(), cols, group);
    else
      for (int i = 0; i < cols; ++i) rot[i] = w[size_t(r) * cols + i];
    double amax = 0.0;
    for (int i = 0; i < cols; ++i) amax = std::max(amax, std::fabs(rot[i]));
    const float s = amax > 0.0 ? float(amax / 127.0) : 1.0f;
    scale[r] = s;
    for (int i = 0; i < cols; ++i) codes[size_t(r) * cols + i] = int8_t(rint_clamp(float(rot[i] / double(s)), -127, 127));
  }
}

}  // namespace sfq
