// Stand-alone pointwise kernels of the block that sit next to the Linear:
// GELU-tanh, SwiGLU and the gated residual. The GEMM epilogue fuses GELU; these
// exist so that callers of the reference's launchers keep working unchanged.
#include "kernels.cuh"

#include <cuda_fp8.h>

#include <stdexcept>
#include <string>

namespace sfq {
namespace {

inline void check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// bf16(0.5 v (1 + tanh(k (v + 0.044715 v^3)))) in place (gelu_tanh_kernel, src/cuda/nn_pointwise.cu:74-81).
__global__ void gelu_tanh_kernel(__nv_bfloat16* x, size_t n) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) {
    const float v = __bfloat162float(x[i]);
    constexpr float k = 0.7978845608028654f;
    x[i] = __float2bfloat16(0.5f * v * (1.0f + tanhf(k * (v + 0.044715f * v * v * v))));
  }
}

// out = silu(fused[:, :inner]) * fused[:, inner:], gate first, fast exp (swiglu_kernel, src/cuda/nn_pointwise.cu:46-64).
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ fused, __nv_bfloat16* __restrict__ out, int inner) {
  const size_t row = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= inner) return;
  const float g = __bfloat162float(fused[row * 2 * size_t(inner) + i]);
  const float v = __bfloat162float(fused[row * 2 * size_t(inner) + inner + i]);
  out[row * size_t(inner) + i] = __float2bfloat16((g / (1.0f + __expf(-g))) * v);
}

// x = bf16(fma(gate[a[row]], branch, x)) (add_gated_kernel, src/cuda/nn_pointwise.cu:15-37).
__global__ void add_gated_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ branch,
                                 const float* __restrict__ gate, const int32_t* __restrict__ a, int dim) {
  const size_t row = blockIdx.x;
  const int i = blockIdx.y * blockDim.x + threadIdx.x;
  if (i >= dim) return;
  const float g = gate[size_t(a[row]) * dim + i];
  const size_t at = row * dim + i;
  x[at] = __float2bfloat16(fmaf(g, __bfloat162float(branch[at]), __bfloat162float(x[at])));
}

// Eight elements per thread, 128-bit accesses; same arithmetic as add_gated_kernel.
__global__ void add_gated_vec_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ branch,
                                     const float* __restrict__ gate, const int32_t* __restrict__ a, int packs) {
  const size_t row = blockIdx.x;
  const int p = blockIdx.y * blockDim.x + threadIdx.x;
  if (p >= packs) return;
  const size_t dim = size_t(packs) * 8;
  const float4* g = reinterpret_cast<const float4*>(gate + size_t(a[row]) * dim) + p * 2;
  uint4* xp = reinterpret_cast<uint4*>(x + row * dim) + p;
  const uint4 xv = *xp, bv = __ldg(reinterpret_cast<const uint4*>(branch + row * dim) + p);
  const float4 g0 = __ldg(g), g1 = __ldg(g + 1);
  const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
  const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
  const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bv);
  uint4 out;
  __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 xf = __bfloat1622float2(xh[i]), bf = __bfloat1622float2(bh[i]);
    oh[i] = __floats2bfloat162_rn(fmaf(gg[2 * i], bf.x, xf.x), fmaf(gg[2 * i + 1], bf.y, xf.y));
  }
  *xp = out;
}

// dst[r, i] = bf16(src[r, i] * scale[i]): the AWQ activation pre-scale (pre_quant_scale_kernel,
// src/cuda/linear_weights.cu:499-509).
__global__ void pre_quant_scale_kernel(const __nv_bfloat16* __restrict__ src, const __nv_bfloat16* __restrict__ scale,
                                       __nv_bfloat16* __restrict__ dst, int dim) {
  const int col = blockIdx.y * blockDim.x + threadIdx.x;
  if (col >= dim) return;
  const size_t i = size_t(blockIdx.x) * dim + col;
  dst[i] = __float2bfloat16(__bfloat162float(src[i]) * __bfloat162float(scale[col]));
}

}  // namespace

void pre_quant_scale(const __nv_bfloat16* src, const __nv_bfloat16* scale, __nv_bfloat16* dst, int rows, int dim,
                     cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) return;
  if (scale == nullptr) throw std::runtime_error("pre_quant_scale: null scale");
  if (!src || !dst) throw std::invalid_argument("pre_quant_scale: null buffer");
  pre_quant_scale_kernel<<<dim3(rows, (dim + 255) / 256), 256, 0, stream>>>(src, scale, dst, dim);
  check_launch("pre_quant_scale");
}

void gelu_tanh(__nv_bfloat16* x, size_t n, cudaStream_t stream) {
  if (n == 0) return;
  if (!x) throw std::invalid_argument("gelu_tanh: null buffer");
  gelu_tanh_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(x, n);
  check_launch("gelu_tanh");
}

void swiglu(const __nv_bfloat16* fused, __nv_bfloat16* out, int rows, int inner, cudaStream_t stream) {
  if (rows <= 0 || inner <= 0) throw std::invalid_argument("swiglu: rows and inner must be positive");
  if (!fused || !out) throw std::invalid_argument("swiglu: null buffer");
  swiglu_kernel<<<dim3(rows, (inner + 255) / 256), 256, 0, stream>>>(fused, out, inner);
  check_launch("swiglu");
}

void add_gated(__nv_bfloat16* x, const __nv_bfloat16* branch, const float* gate, const int32_t* index, int rows,
               int dim, cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) throw std::invalid_argument("add_gated: rows and dim must be positive");
  if (!x || !branch || !gate || !index) throw std::invalid_argument("add_gated: null buffer");
  const bool vec = dim % 8 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(branch) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(gate) % 16 == 0;
  if (vec)
    add_gated_vec_kernel<<<dim3(rows, (dim / 8 + 127) / 128), 128, 0, stream>>>(x, branch, gate, index, dim / 8);
  else
    add_gated_kernel<<<dim3(rows, (dim + 255) / 256), 256, 0, stream>>>(x, branch, gate, index, dim);
  check_launch("add_gated");
}

// ---- small launchers of the reference's linear headers that the runner itself does not need -----------------
namespace {
// ConvRot over fp32 (convrot_kernel<float>, src/cuda/linear_weights.cu:422-471): H = kron^stages(h4) / sqrt(group) as
// `stages` radix-4 butterfly passes at strides 1, 4, 16, ... over one group, each output a left-to-right sum of the
// four inputs with the signs of the regular Hadamard h4, one multiplication by 1 / sqrt(group) at the end. One warp per
// group, the group in shared memory, a butterfly read and written by the same lane.
__global__ void __launch_bounds__(256) convrot_f32_kernel(const float* __restrict__ in, float* __restrict__ out, int group, int stages,
                                                          float norm, size_t total_groups) {
  extern __shared__ float rot_buf[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t g = size_t(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (g >= total_groups) return;  // whole warps leave; only __syncwarp below
  float* buf = rot_buf + size_t(warp) * group;
  const float* src = in + g * group;
  for (int i = lane; i < group; i += 32) buf[i] = src[i];
  __syncwarp();
  int stride = 1;
  for (int s = 0; s < stages; ++s, stride *= 4) {
    for (int b = lane; b < group / 4; b += 32) {
      const int i = (b / stride) * 4 * stride + (b % stride);
      const float a = buf[i], bb = buf[i + stride], c = buf[i + 2 * stride], d = buf[i + 3 * stride];
      buf[i] = __fsub_rn(__fadd_rn(__fadd_rn(a, bb), c), d);
      buf[i + stride] = __fadd_rn(__fsub_rn(__fadd_rn(a, bb), c), d);
      buf[i + 2 * stride] = __fadd_rn(__fadd_rn(__fsub_rn(a, bb), c), d);
      buf[i + 3 * stride] = __fadd_rn(__fadd_rn(__fadd_rn(-a, bb), c), d);
    }
    __syncwarp();
  }
  float* dst = out + g * group;
  for (int i = lane; i < group; i += 32) dst[i] = buf[i] * norm;
}

// dst[r, i] = src[r, i] * scale[i] in fp32 (pre_quant_scale_kernel<float>, src/cuda/linear_weights.cu:499-509).
__global__ void pre_quant_scale_f32_kernel(const float* __restrict__ src, const __nv_bfloat16* __restrict__ scale, float* __restrict__ dst,
                                           int dim) {
  const int col = blockIdx.y * blockDim.x + threadIdx.x;
  if (col >= dim) return;
  const size_t i = size_t(blockIdx.x) * dim + col;
  dst[i] = src[i] * __bfloat162float(scale[col]);
}

// bf16((float(acc) * row) * channel) (output_bf16, src/cuda/w4a8.cu:218-223), and the fp32 form written over the
// accumulator itself (dequant_output_kernel, src/cuda/w4a8.cu:126-136).
__global__ void int8_output_bf16_kernel(const int32_t* __restrict__ acc, const float* __restrict__ rows, const float* __restrict__ channels,
                                        __nv_bfloat16* __restrict__ out, int cols) {
  const int col = blockIdx.y * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  const size_t i = size_t(blockIdx.x) * cols + col;
  out[i] = __float2bfloat16(__fmul_rn(__fmul_rn(float(acc[i]), rows[blockIdx.x]), channels[col]));
}
__global__ void int8_output_f32_kernel(int32_t* io, const float* __restrict__ rows, const float* __restrict__ channels, int cols) {
  const int col = blockIdx.y * blockDim.x + threadIdx.x;
  if (col >= cols) return;
  const size_t i = size_t(blockIdx.x) * cols + col;
  const float v = __fmul_rn(__fmul_rn(float(io[i]), rows[blockIdx.x]), channels[col]);
  reinterpret_cast<float*>(io)[i] = v;
}

// e4m3(bf16 * (1 / input_scale)), round to nearest even, saturating at 448 (quantize_f8_kernel,
// src/cuda/linear_weights.cu:337-343 with the encoder of :41-68).
__global__ void quantize_f8_kernel(const __nv_bfloat16* __restrict__ src, float inv_scale, uint8_t* __restrict__ dst, size_t n) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = uint8_t(__nv_cvt_float_to_fp8(__bfloat162float(src[i]) * inv_scale, __NV_SATFINITE, __NV_E4M3));
}
__global__ void widen_kernel(const __nv_bfloat16* __restrict__ src, float* __restrict__ dst, size_t n) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __bfloat162float(src[i]);
}
__global__ void narrow_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
  const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = __float2bfloat16(src[i]);
}

// Quantized fp4 activations from the reference's layout (low nibble = even element, scales row-major [rows, dim/16];
// launch_quantize_nvfp4_activations, include/slopfab/cuda/nvfp4_gemm.cuh:77-82) into the layout the tcgen05 GEMM
// reads: nibbles of every byte exchanged, scales in 128-row x 4-block tiles of 512 bytes with the rows padded to a
// multiple of 128 (pad rows zero). One thread per 16-element block of a padded row.
__global__ void nvfp4_act_to_feed_kernel(const uint8_t* __restrict__ xq, const uint8_t* __restrict__ xs, uint8_t* __restrict__ oq,
                                         uint8_t* __restrict__ os, int rows, int blocks_per_row) {
  const int kb = blockIdx.y * blockDim.x + threadIdx.x;
  if (kb >= blocks_per_row) return;
  const int r = blockIdx.x;
  uint8_t scale = 0;
  if (r < rows) {
    const size_t b = size_t(r) * blocks_per_row + kb;
    const uint64_t v = reinterpret_cast<const uint64_t*>(xq)[b];
    reinterpret_cast<uint64_t*>(oq)[b] = ((v >> 4) & 0x0F0F0F0F0F0F0F0Full) | ((v & 0x0F0F0F0F0F0F0F0Full) << 4);
    scale = xs[b];
  }
  const size_t tile = size_t(r / 128) * (blocks_per_row / 4) + kb / 4;
  os[tile * 512 + (r % 32) * 16 + ((r % 128) / 32) * 4 + kb % 4] = scale;
}
}  // namespace

void convrot_f32(const float* in, float* out, int rows, int dim, int group, cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) return;
  if (group <= 0 || dim % group != 0)
    throw std::runtime_error("convrot: dim " + std::to_string(dim) + " is not a multiple of group " + std::to_string(group));
  int stages = 0, n = 1;
  while (n < group) n *= 4, ++stages;
  if (n != group) throw std::runtime_error("convrot: group size must be a power of four, got " + std::to_string(group));
  if (group > 4096) throw std::runtime_error("convrot: group " + std::to_string(group) + " needs more than 1024 threads per block");
  if (!in || !out) throw std::invalid_argument("convrot_f32: null buffer");
  const size_t groups = size_t(rows) * (dim / group);
  const float norm = 1.0f / sqrtf(float(group));  // a power of two: exact
  const int warps = group > 1024 ? 2 : 8;
  convrot_f32_kernel<<<unsigned((groups + warps - 1) / warps), warps * 32, size_t(warps) * group * sizeof(float), stream>>>(in, out, group, stages,
                                                                                                                       norm, groups);
  check_launch("convrot_f32");
}

void pre_quant_scale_f32(const float* src, const __nv_bfloat16* scale, float* dst, int rows, int dim, cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) return;
  if (scale == nullptr) throw std::runtime_error("pre_quant_scale: null scale");
  if (!src || !dst) throw std::invalid_argument("pre_quant_scale: null buffer");
  pre_quant_scale_f32_kernel<<<dim3(rows, (dim + 255) / 256), 256, 0, stream>>>(src, scale, dst, dim);
  check_launch("pre_quant_scale_f32");
}

void int8_output_bf16(const int32_t* acc, const float* row_scale, const float* channel_scale, __nv_bfloat16* out, int rows, int cols,
                      cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return;
  if (!acc || !row_scale || !channel_scale || !out) throw std::invalid_argument("W4A8 output scaling received a null buffer");
  int8_output_bf16_kernel<<<dim3(rows, (cols + 255) / 256), 256, 0, stream>>>(acc, row_scale, channel_scale, out, cols);
  check_launch("int8_output_bf16");
}

void int8_output_f32_inplace(int32_t* io, const float* row_scale, const float* channel_scale, int rows, int cols, cudaStream_t stream) {
  if (!io || !row_scale || !channel_scale) throw std::invalid_argument("W4A8 output dequantization received a null buffer");
  if (rows <= 0 || cols <= 0) throw std::invalid_argument("W4A8 output dequantization received an invalid shape");
  int8_output_f32_kernel<<<dim3(rows, (cols + 255) / 256), 256, 0, stream>>>(io, row_scale, channel_scale, cols);
  check_launch("int8_output_f32");
}

void quantize_f8e4m3(const __nv_bfloat16* src, float input_scale, uint8_t* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return;
  if (input_scale == 0.0f)
    throw std::runtime_error("launch_quantize_f8e4m3: input_scale is zero, which marks a layer that has no activation scale");
  if (!src || !dst) throw std::invalid_argument("quantize_f8e4m3: null buffer");
  quantize_f8_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(src, 1.0f / input_scale, dst, n);
  check_launch("quantize_f8e4m3");
}

void widen_bf16(const __nv_bfloat16* src, float* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return;
  widen_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(src, dst, n);
  check_launch("widen_bf16");
}

void narrow_to_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t stream) {
  if (n == 0) return;
  narrow_kernel<<<unsigned((n + 255) / 256), 256, 0, stream>>>(src, dst, n);
  check_launch("narrow_to_bf16");
}

void nvfp4_act_to_feed(const uint8_t* xq, const uint8_t* xs, uint8_t* feed_q, uint8_t* feed_scale_tiled, int rows, int dim,
                       cudaStream_t stream) {
  if (rows <= 0) return;
  if (dim <= 0 || dim % 64 != 0) throw std::invalid_argument("nvfp4_act_to_feed: dim must be a multiple of 64");
  if (!xq || !xs || !feed_q || !feed_scale_tiled) throw std::invalid_argument("nvfp4_act_to_feed: null buffer");
  if (reinterpret_cast<uintptr_t>(xq) % 8 != 0 || reinterpret_cast<uintptr_t>(feed_q) % 8 != 0)
    throw std::invalid_argument("nvfp4_act_to_feed: packed activations must be 8-byte aligned");
  const int blocks = dim / 16, padded = (rows + 127) / 128 * 128;
  nvfp4_act_to_feed_kernel<<<dim3(padded, (blocks + 127) / 128), 128, 0, stream>>>(xq, xs, feed_q, feed_scale_tiled, rows, blocks);
  check_launch("nvfp4_act_to_feed");
}

// ---- fp32 Linear (the reference's fp32-compute arm, src/cuda/linear.cu:251-285: fp32 GEMM + add_bias) ----
// y[m, n] = sum_k x[m, k] * w[n, k] (+ bias[n], added to the finished sum as add_bias_kernel does). CUDA cores: the
// DiT calls this arm only for the handful of timestep rows that make the adaLN tables. 64 x 64 outputs per block,
// 4 x 4 per thread, K in slices of 16 through shared memory.
namespace {
template <typename WT> __device__ __forceinline__ float widen(WT v);
template <> __device__ __forceinline__ float widen<float>(float v) { return v; }
template <> __device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename WT>
__global__ void __launch_bounds__(256) linear_f32_kernel(const float* __restrict__ x, const WT* __restrict__ w, const void* __restrict__ bias,
                                                         int bias_is_bf16, float* __restrict__ y, int rows, int out_features, int in_features) {
  __shared__ float xs[16][65], ws[16][65];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < in_features; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int r = i >> 4, k = i & 15;
      const bool k_ok = k0 + k < in_features;
      xs[k][r] = (k_ok && m0 + r < rows) ? x[size_t(m0 + r) * in_features + k0 + k] : 0.0f;
      ws[k][r] = (k_ok && n0 + r < out_features) ? widen<WT>(w[size_t(n0 + r) * in_features + k0 + k]) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i], b[i] = ws[k][tx * 4 + i];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < rows && n < out_features) {
        float v = acc[i][j];
        if (bias != nullptr)
          v += bias_is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]) : static_cast<const float*>(bias)[n];
        y[size_t(m) * out_features + n] = v;
      }
    }
}

// adaLN table expansion (adaln_expand_kernel, src/cuda/dit_kernels.cu:61-90): one fp32 fma chain per output feature
// and timestep, started from the bias, k ascending; the result lands at [param][timestep][modality][channel].
__global__ void adaln_expand_kernel(const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ code,
                                    float* __restrict__ out, int num_t, int num_modality, int num_param, int channels, int rank,
                                    int out_features) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= out_features) return;
  const int ti = blockIdx.y;
  const float* c = code + size_t(ti) * rank;
  const float* row = w + size_t(p) * rank;
  float acc = bias[p];
  for (int k = 0; k < rank; ++k) acc = fmaf(row[k], c[k], acc);
  const int channel = p % channels, rest = p / channels;
  const int param = rest % num_param, modality = rest / num_param;
  out[(size_t(param) * num_t * num_modality + size_t(ti) * num_modality + modality) * channels + channel] = acc;
}
}  // namespace

void linear_f32(const float* x, const void* w, bool w_is_bf16, const void* bias, bool bias_is_bf16, float* y, int rows, int out_features,
                int in_features, cudaStream_t stream) {
  if (rows <= 0 || out_features <= 0) return;
  if (in_features <= 0 || !x || !w || !y) throw std::invalid_argument("linear_f32: bad arguments");
  const dim3 grid((out_features + 63) / 64, (rows + 63) / 64);
  if (grid.y > 65535) throw std::invalid_argument("linear_f32: too many rows for one launch");
  if (w_is_bf16)
    linear_f32_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(x, static_cast<const __nv_bfloat16*>(w), bias, bias_is_bf16 ? 1 : 0, y, rows,
                                                                out_features, in_features);
  else
    linear_f32_kernel<float><<<grid, 256, 0, stream>>>(x, static_cast<const float*>(w), bias, bias_is_bf16 ? 1 : 0, y, rows, out_features,
                                                       in_features);
  check_launch("linear_f32");
}

void adaln_expand(const float* w, const float* bias, const float* code, float* out, int num_t, int num_modality, int num_param,
                  int channels, int rank, cudaStream_t stream) {
  // the checks of launch_adaln_expand (src/cuda/dit_kernels.cu:108-127), same messages
  if (num_t <= 0 || num_modality <= 0 || num_param <= 0 || channels <= 0 || rank <= 0)
    throw std::runtime_error("launch_adaln_expand: every extent must be positive");
  const size_t features = size_t(num_modality) * num_param * channels;
  if (features > 0x7FFFFFFFull)
    throw std::runtime_error("launch_adaln_expand: " + std::to_string(features) + " output features overflows the kernel's index type");
  if (num_t > 65535) throw std::runtime_error("launch_adaln_expand: " + std::to_string(num_t) + " timesteps exceeds the gridDim.y limit");
  if (!w || !bias || !code || !out) throw std::invalid_argument("adaln_expand: null operand");
  const dim3 grid(unsigned((features + 255) / 256), unsigned(num_t));
  adaln_expand_kernel<<<grid, 256, 0, stream>>>(w, bias, code, out, num_t, num_modality, num_param, channels, rank, int(features));
  check_launch("adaln_expand");
}

}  // namespace sfq
