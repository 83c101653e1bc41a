// Stand-alone pointwise kernels of the block that sit next to the Linear:
// GELU-tanh, SwiGLU and the gated residual. The GEMM epilogue fuses GELU; these
// exist so that callers of the reference's launchers keep working unchanged.
#include "kernels.cuh"

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

}  // namespace sfq
