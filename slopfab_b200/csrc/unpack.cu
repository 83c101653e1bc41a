// Device unpackers: stored weight bytes -> bf16 / int8 / fp16, bit-exact with the
// reference's dequantisation kernels. All are streaming kernels bound by HBM;
// each thread handles one 16-element scale group with 128-bit stores.
#include "kernels.cuh"

#include <algorithm>
#include <stdexcept>
#include <string>

#include "codec.cuh"

namespace sfq {
namespace {

constexpr int kThreads = 256;

inline unsigned blocks_for(size_t n, int per_block) {
  return static_cast<unsigned>((n + per_block - 1) / per_block);
}

inline void check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// w = bf16( e2m1(nibble) * (e4m3(scale) * global) ), even element in the HIGH nibble,
// scales in the 128x4-tiled layout (dequant_nvfp4_kernel, src/cuda/linear_weights.cu:216-245).
__global__ void __launch_bounds__(kThreads)
unpack_nvfp4_kernel(const uint8_t* __restrict__ data, const uint8_t* __restrict__ scale, float global,
                    __nv_bfloat16* __restrict__ out, int rows, int blocks_per_row) {
  const size_t g = size_t(blockIdx.x) * kThreads + threadIdx.x;  // one 16-element block
  const size_t total = size_t(rows) * blocks_per_row;
  if (g >= total) return;
  const int row = int(g / blocks_per_row);
  const int blk = int(g - size_t(row) * blocks_per_row);
  const uint2 raw = __ldg(reinterpret_cast<const uint2*>(data) + g);
  const float s = e4m3_decode(__ldg(scale + nvfp4_scale_offset(row, blk, blocks_per_row))) * global;
  const uint32_t words[2] = {raw.x, raw.y};
  uint4 o[2];
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    const uint32_t byte = (words[b >> 2] >> (8 * (b & 3))) & 0xFFu;
    op[b] = __floats2bfloat162_rn(e2m1_decode(byte >> 4) * s, e2m1_decode(byte & 15u) * s);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + g * 16);
  dst[0] = o[0];
  dst[1] = o[1];
}

// q = clamp(rint(codebook[code] * e4m3(scale[row, col/16])), -127, 127), byte = even | odd << 4
// (dequant_weight_kernel, src/cuda/w4a8.cu:44-68).
//
// A group's 16 outputs depend only on its scale byte and its codes, and there are 256 scale bytes: every CTA first
// builds the table q[scale byte][code] (4 KB of shared memory, the reference's expression evaluated once per
// entry), then walks groups. For a group, one 16-byte shared load fetches the table row of its scale; four codes
// at a time are looked up with three byte permutes (the two 8-entry halves of the row, then a per-byte choice between them
// by bit 3 of each code), so a group costs ~20 instructions instead of ~170 and the kernel runs at memory speed.
__global__ void __launch_bounds__(kThreads)
unpack_w4a8_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ gscale,
                   const float* __restrict__ codebook, int8_t* __restrict__ out, size_t groups) {
  __shared__ __align__(16) uint8_t table[256 * 16];
  {
    // thread t builds the row of scale byte t (kThreads == 256): decode the scale once, sixteen products
    const float s = e4m3_decode(uint8_t(threadIdx.x));
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 c = __ldg(reinterpret_cast<const float4*>(codebook) + j);
      const float cc[4] = {c.x, c.y, c.z, c.w};
      uint32_t acc = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        // NaN scale bytes (0x7F, 0xFF) never occur in valid files; the integer conversion turns NaN into 0
        const int q = max(-127, min(127, __float2int_rn(cc[i] * s)));
        acc |= uint32_t(uint8_t(q)) << (8 * i);
      }
      w[j] = acc;
    }
    reinterpret_cast<uint4*>(table)[threadIdx.x] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  __syncthreads();
  const uint4* rows = reinterpret_cast<const uint4*>(table);
  auto expand = [&](const uint2 raw, const uint4 row, size_t g) {
    const uint32_t words[2] = {raw.x, raw.y};
    uint32_t o[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t codes = (words[w >> 1] >> (16 * (w & 1))) & 0xFFFFu;      // four nibbles = elements 4w .. 4w+3
      const uint32_t sel = codes & 0x7777u;                                   // index inside an 8-entry half
      const uint32_t lo = __byte_perm(row.x, row.y, sel), hi = __byte_perm(row.z, row.w, sel);
      // output byte i comes from `hi` when bit 3 of code i is set: a third permute whose selector is i + 4 * bit3(i)
      o[w] = __byte_perm(lo, hi, 0x3210u | ((codes & 0x8888u) >> 1));
    }
    reinterpret_cast<uint4*>(out)[g] = make_uint4(o[0], o[1], o[2], o[3]);
  };
  const size_t stride = size_t(gridDim.x) * kThreads;
  size_t g = size_t(blockIdx.x) * kThreads + threadIdx.x;
  for (; g + 3 * stride < groups; g += 4 * stride) {  // four groups per trip: eight independent loads in flight
    uint2 raw[4];
    uint8_t sc[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      raw[u] = __ldg(reinterpret_cast<const uint2*>(packed) + g + u * stride);  // 16 codes, element e in nibble e
      sc[u] = __ldg(gscale + g + u * stride);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) expand(raw[u], rows[sc[u]], g + u * stride);  // rows[s]: q for codes 0..15 at scale s
  }
  for (; g < groups; g += stride) expand(__ldg(reinterpret_cast<const uint2*>(packed) + g), rows[__ldg(gscale + g)], g);
}

// Row = K/2 low-nibble bytes then K/4 bytes of 2-bit highs (shifts 0,2,4,6);
// level = code - 32; q = clamp(rint(level * e4m3(scale[(row*K + col) / group])), -127, 127)
// (dequant_w6_kernel, src/cuda/w4a8.cu:15-29).
__global__ void __launch_bounds__(kThreads)
unpack_w6a8_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ gscale, int8_t* __restrict__ out,
                   int rows, int width, int group) {
  const int chunks_per_row = width / 16;
  const size_t c = size_t(blockIdx.x) * kThreads + threadIdx.x;  // 16 consecutive columns of one row
  if (c >= size_t(rows) * chunks_per_row) return;
  const int row = int(c / chunks_per_row);
  const int col0 = int(c - size_t(row) * chunks_per_row) * 16;
  const uint8_t* rowp = packed + size_t(row) * (size_t(width) * 3 / 4);
  const uint2 lo = __ldg(reinterpret_cast<const uint2*>(rowp + col0 / 2));
  const uint32_t hi = __ldg(reinterpret_cast<const uint32_t*>(rowp + width / 2 + col0 / 4));
  const float s = e4m3_decode(__ldg(gscale + (size_t(row) * width + col0) / group));
  const uint32_t words[2] = {lo.x, lo.y};
  uint32_t o[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    uint32_t acc = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int e = w * 4 + j;
      const uint32_t byte = (words[e >> 3] >> (8 * ((e >> 1) & 3))) & 0xFFu;
      const uint32_t low = (e & 1) ? (byte >> 4) : (byte & 15u);
      const uint32_t high = (hi >> (2 * e)) & 3u;  // byte e/4, shift (e&3)*2
      const int level = int(low | (high << 4)) - 32;
      const int q = max(-127, min(127, __float2int_rn(float(level) * s)));
      acc |= uint32_t(uint8_t(q)) << (8 * j);
    }
    o[w] = acc;
  }
  *reinterpret_cast<uint4*>(out + size_t(row) * width + col0) = make_uint4(o[0], o[1], o[2], o[3]);
}

// bf16(int8 * scale[row]) (dequant_i8_kernel, src/cuda/linear_weights.cu:177-192).
__global__ void __launch_bounds__(kThreads)
unpack_int8_bf16_kernel(const int8_t* __restrict__ src, const float* __restrict__ scale,
                        __nv_bfloat16* __restrict__ dst, int rows, int cols) {
  const size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x;
  const size_t total = size_t(rows) * cols;
  if (i >= total) return;
  dst[i] = __float2bfloat16(float(src[i]) * scale[i / cols]);
}
__global__ void __launch_bounds__(kThreads)
unpack_int8_bf16_vec_kernel(const int8_t* __restrict__ src, const float* __restrict__ scale,
                            __nv_bfloat16* __restrict__ dst, size_t packs, int packs_per_row) {
  const size_t p = size_t(blockIdx.x) * kThreads + threadIdx.x;  // 16 elements
  if (p >= packs) return;
  const float s = __ldg(scale + p / packs_per_row);
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(src) + p);
  const int8_t* b = reinterpret_cast<const int8_t*>(&raw);
  uint4 o[2];
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
  for (int j = 0; j < 8; ++j) op[j] = __floats2bfloat162_rn(float(b[2 * j]) * s, float(b[2 * j + 1]) * s);
  uint4* d = reinterpret_cast<uint4*>(dst + p * 16);
  d[0] = o[0];
  d[1] = o[1];
}

// INT8 ConvRot weight -> fp16 in ordinary coordinates: the regular-Hadamard butterfly on the
// int8 codes (left-to-right fp32 adds), times scale[row] / sqrt(group), rounded to fp16, with an
// optional flush of fp16 subnormals to signed zero (unpack_int8_weight, src/core/int8_weight.cpp:66-100;
// unpack_int8_kernel, src/cuda/nf4_weight.cu:20-51). One block of 64 threads per 256 columns.
__global__ void __launch_bounds__(64)
unpack_int8_f16_kernel(const int8_t* __restrict__ codes, const float* __restrict__ scales, __half* __restrict__ out,
                       int cols, int group, int stages, float norm, int flush) {
  __shared__ float v[256 + 64];
  const int row = blockIdx.x;
  const int c0 = blockIdx.y * 256;
  const int n = min(256, cols - c0);
  const size_t base = size_t(row) * cols + c0;
  const int t = threadIdx.x;
  for (int i = t; i < n; i += 64) v[i + (i >> 2)] = float(codes[base + i]);
  __syncthreads();
  int stride = 1;
  for (int s = 0; s < stages; ++s) {
    const int i = (t / stride) * 4 * stride + (t % stride);
    const bool live = i + 3 * stride < n;
    float a = 0, b = 0, c = 0, d = 0;
    const int i0 = i + (i >> 2), i1 = (i + stride) + ((i + stride) >> 2), i2 = (i + 2 * stride) + ((i + 2 * stride) >> 2),
              i3 = (i + 3 * stride) + ((i + 3 * stride) >> 2);
    if (live) a = v[i0], b = v[i1], c = v[i2], d = v[i3];
    __syncthreads();
    if (live) {
      v[i0] = ((a + b) + c) - d;
      v[i1] = ((a + b) - c) + d;
      v[i2] = ((a - b) + c) + d;
      v[i3] = ((-a + b) + c) + d;
    }
    __syncthreads();
    stride *= 4;
  }
  const float factor = scales[row] * norm;
  for (int i = t; i < n; i += 64) {
    __half h = __float2half_rn(v[i + (i >> 2)] * factor);
    unsigned short bits = __half_as_ushort(h);
    if (flush && (bits & 0x7C00u) == 0) bits &= 0x8000u;
    out[base + i] = __ushort_as_half(bits);
  }
}

// bf16(f8_e4m3(v) * scale), scale a device scalar (dequant_f8_kernel, src/cuda/linear_weights.cu:150-172).
__global__ void __launch_bounds__(kThreads)
unpack_f8_kernel(const uint8_t* __restrict__ src, const float* __restrict__ scale, __nv_bfloat16* __restrict__ dst, size_t n) {
  const size_t i = (size_t(blockIdx.x) * kThreads + threadIdx.x) * 8;
  if (i >= n) return;
  const float s = __ldg(scale);
  if (i + 8 <= n && (reinterpret_cast<uintptr_t>(src) & 7) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src + i));
    const uint32_t w[2] = {raw.x, raw.y};
    uint4 o;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t b0 = (w[j >> 1] >> (16 * (j & 1))) & 0xFFu, b1 = (w[j >> 1] >> (16 * (j & 1) + 8)) & 0xFFu;
      op[j] = __floats2bfloat162_rn(e4m3_decode(uint8_t(b0)) * s, e4m3_decode(uint8_t(b1)) * s);
    }
    *reinterpret_cast<uint4*>(dst + i) = o;
  } else {
    for (size_t j = i; j < n && j < i + 8; ++j) dst[j] = __float2bfloat16(e4m3_decode(src[j]) * s);
  }
}

// bitsandbytes NF4, double-quantized block scales, high nibble = even element
// (dequant_nf4_kernel / dequant_nf4_vec_kernel, src/cuda/linear_weights.cu:273-315):
// value = map[code] * (nested_map[absmax[block]] * nested_absmax[block / nested_block] + offset).
template <class T> __device__ __forceinline__ T narrow_to(float v);
template <> __device__ __forceinline__ __nv_bfloat16 narrow_to<__nv_bfloat16>(float v) { return __float2bfloat16(v); }
template <> __device__ __forceinline__ __half narrow_to<__half>(float v) { return __float2half_rn(v); }

template <class T>
__global__ void __launch_bounds__(kThreads)
unpack_nf4_kernel(const uint8_t* __restrict__ src, const uint8_t* __restrict__ absmax, const float* __restrict__ map,
                  const float* __restrict__ nested_map, const float* __restrict__ nested_absmax, int block,
                  int nested_block, float offset, T* __restrict__ dst, size_t n) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = map[threadIdx.x];
  __syncthreads();
  const size_t byte = size_t(blockIdx.x) * kThreads + threadIdx.x;
  const size_t even = byte * 2;
  if (even >= n) return;
  const size_t b = even / size_t(block);
  const float scale = __fmaf_rn(nested_map[absmax[b]], nested_absmax[b / size_t(nested_block)], offset);
  const uint8_t packed = src[byte];
  dst[even] = narrow_to<T>(lut[packed >> 4] * scale);
  if (even + 1 < n) {
    // an odd block size could put the odd element in the next block; recompute when it does
    const size_t b1 = (even + 1) / size_t(block);
    const float s1 = b1 == b ? scale : __fmaf_rn(nested_map[absmax[b1]], nested_absmax[b1 / size_t(nested_block)], offset);
    dst[even + 1] = narrow_to<T>(lut[packed & 15] * s1);
  }
}

template <class T> __global__ void __launch_bounds__(kThreads) to_bf16_kernel(const T* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
  const size_t i = size_t(blockIdx.x) * kThreads + threadIdx.x;
  if (i < n) dst[i] = __float2bfloat16(float(src[i]));
}

}  // namespace

void unpack_f8e4m3_bf16(const uint8_t* src, const float* scale, __nv_bfloat16* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return;
  if (!src || !scale || !dst) throw std::runtime_error("linear: fp8 weight without weight_scale");
  unpack_f8_kernel<<<blocks_for((n + 7) / 8, kThreads), kThreads, 0, stream>>>(src, scale, dst, n);
  check_launch("unpack_f8e4m3");
}

void unpack_nf4_bf16(const uint8_t* src, const uint8_t* absmax, const float* map, const float* nested_map,
                     const float* nested_absmax, int block, int nested_block, float offset, __nv_bfloat16* dst,
                     int out_features, int in_features, cudaStream_t stream) {
  if (out_features <= 0 || in_features <= 0) return;
  if (!src || !absmax || !map || !nested_map || !nested_absmax || !dst)
    throw std::runtime_error("linear: nf4 weight without complete double-quant state");
  if (block <= 0 || nested_block <= 0) throw std::invalid_argument("unpack_nf4: block sizes must be positive");
  const size_t n = size_t(out_features) * in_features;
  unpack_nf4_kernel<__nv_bfloat16><<<blocks_for((n + 1) / 2, kThreads), kThreads, 0, stream>>>(src, absmax, map, nested_map, nested_absmax,
                                                                                              block, nested_block, offset, dst, n);
  check_launch("unpack_nf4");
}

// The fp16 form over a flat element count (launch_dequant_nf4_f16, src/cuda/linear_weights.cu:317-335).
void unpack_nf4_f16(const uint8_t* src, const uint8_t* absmax, const float* map, const float* nested_map,
                    const float* nested_absmax, int block, int nested_block, float offset, __half* dst, size_t n,
                    cudaStream_t stream) {
  if (n == 0) return;
  if (!src || !absmax || !map || !nested_map || !nested_absmax || !dst)
    throw std::runtime_error("linear: nf4 weight without complete double-quant state");
  if (block <= 0 || nested_block <= 0) throw std::invalid_argument("unpack_nf4: block sizes must be positive");
  unpack_nf4_kernel<__half><<<blocks_for((n + 1) / 2, kThreads), kThreads, 0, stream>>>(src, absmax, map, nested_map, nested_absmax, block,
                                                                                       nested_block, offset, dst, n);
  check_launch("unpack_nf4_f16");
}

void convert_f16_bf16(const __half* src, __nv_bfloat16* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return;
  to_bf16_kernel<__half><<<blocks_for(n, kThreads), kThreads, 0, stream>>>(src, dst, n);
  check_launch("convert_f16_bf16");
}

void convert_f32_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return;
  to_bf16_kernel<float><<<blocks_for(n, kThreads), kThreads, 0, stream>>>(src, dst, n);
  check_launch("convert_f32_bf16");
}

void unpack_nvfp4_bf16(const uint8_t* data, const uint8_t* scale, float global, __nv_bfloat16* out, int out_features,
                       int in_features, cudaStream_t stream) {
  if (out_features <= 0 || in_features <= 0) return;
  if (!data || !out) throw std::invalid_argument("unpack_nvfp4: null buffer");
  if (!scale) throw std::runtime_error("unpack_nvfp4: block_scale is null");
  if (out_features % 128 != 0 || in_features % 64 != 0)
    throw std::runtime_error("unpack_nvfp4: " + std::to_string(out_features) + "x" + std::to_string(in_features) +
                             " does not tile the 128x4 block-scale layout (needs out % 128 == 0 and in % 64 == 0)");
  const size_t groups = size_t(out_features) * (in_features / 16);
  unpack_nvfp4_kernel<<<blocks_for(groups, kThreads), kThreads, 0, stream>>>(data, scale, global, out, out_features,
                                                                            in_features / 16);
  check_launch("unpack_nvfp4");
}

void unpack_w4a8_int8(const int8_t* packed, const uint8_t* gscale, const float* codebook, int8_t* out, int out_features,
                      int in_features, int group, cudaStream_t stream) {
  if (!packed || !gscale || !codebook || !out) throw std::invalid_argument("W4A8 weight decode: null buffer");
  if (out_features <= 0 || in_features <= 0 || group != 16 || in_features % 16 != 0)
    throw std::invalid_argument("W4A8 weight decode: needs positive dims, group 16 and in_features % 16 == 0");
  const size_t groups = size_t(out_features) * (in_features / 16);
  // every CTA first spends one table row per thread, so give each one many groups
  static_assert(kThreads == 256, "one table row per thread");
  if (reinterpret_cast<uintptr_t>(codebook) % 16 != 0) throw std::invalid_argument("W4A8 weight decode: codebook must be 16-byte aligned");
  const unsigned grid = unsigned(std::min<size_t>(blocks_for(groups, kThreads), size_t(148) * 4));
  unpack_w4a8_kernel<<<grid, kThreads, 0, stream>>>(reinterpret_cast<const uint8_t*>(packed), gscale, codebook, out, groups);
  check_launch("unpack_w4a8");
}

void unpack_w6a8_int8(const int8_t* packed, const uint8_t* gscale, int8_t* out, int out_features, int in_features,
                      int group, cudaStream_t stream) {
  if (!packed || !gscale || !out || out_features <= 0 || in_features <= 0 || in_features % 32 || group < 16 ||
      group % 16 || in_features % group)
    throw std::invalid_argument("W6A8 weight decode: invalid buffers or dimensions");
  const size_t chunks = size_t(out_features) * (in_features / 16);
  unpack_w6a8_kernel<<<blocks_for(chunks, kThreads), kThreads, 0, stream>>>(reinterpret_cast<const uint8_t*>(packed),
                                                                           gscale, out, out_features, in_features, group);
  check_launch("unpack_w6a8");
}

void unpack_int8_bf16(const int8_t* codes, const float* scale, __nv_bfloat16* out, int out_features, int in_features,
                      cudaStream_t stream) {
  if (out_features <= 0 || in_features <= 0) return;
  if (!codes || !scale || !out) throw std::invalid_argument("unpack_int8: null buffer");
  const size_t n = size_t(out_features) * in_features;
  if (in_features % 16 == 0 && reinterpret_cast<uintptr_t>(codes) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0)
    unpack_int8_bf16_vec_kernel<<<blocks_for(n / 16, kThreads), kThreads, 0, stream>>>(codes, scale, out, n / 16,
                                                                                     in_features / 16);
  else
    unpack_int8_bf16_kernel<<<blocks_for(n, kThreads), kThreads, 0, stream>>>(codes, scale, out, out_features, in_features);
  check_launch("unpack_int8");
}

void unpack_int8_f16(const int8_t* codes, const float* scale, __half* out, int out_features, int in_features,
                     int group, int flush, cudaStream_t stream) {
  if (out_features <= 0 || in_features <= 0) return;
  if (!codes || !scale || !out) throw std::invalid_argument("unpack_int8_f16: null buffer");
  int stages = 0, n = 1;
  while (n < group) n *= 4, ++stages;
  if (n != group || group > 256) throw std::invalid_argument("unpack_int8_f16: rotation group must be 1, 4, 16, 64 or 256");
  if (in_features % group != 0) throw std::invalid_argument("unpack_int8_f16: in_features must hold whole rotation groups");
  const dim3 grid(out_features, (in_features + 255) / 256);
  unpack_int8_f16_kernel<<<grid, 64, 0, stream>>>(codes, scale, out, in_features, group, stages,
                                                  1.0f / sqrtf(float(group)), flush);
  check_launch("unpack_int8_f16");
}

}  // namespace sfq
