// Fused activation front end of the quantized Linear, one pass over HBM:
//
//   [RMSNorm | RMSNorm + adaLN modulate]  ->  [ConvRot-256 -> per-token int8]  |  [per-16-block fp4]
//
// Replaces, with identical bits, the separate launches of the reference:
// rmsnorm_modulate_bf16_kernel (src/cuda/nn_kernels.cu:153-198), convrot_kernel
// (src/cuda/linear_weights.cu:422-471), quantize_bf16 (src/cuda/w4a8.cu:193-216)
// and quantize_act_kernel (src/cuda/nvfp4_gemm.cu:107-158). The activation is read
// once (2 bytes/element, 128-bit loads) and only the quantized form is written.
//
// Work split: one CTA per token row, one thread per 16 consecutive elements (one
// fp4 scale block; 16 threads = one 256-wide rotation group, always inside one
// warp). The rotation runs two radix-4 stages in registers, transposes the group
// through a padded, conflict-free shared-memory tile, and runs the other two.
//
// Bit-exactness notes. The sum of squares is accumulated in the order of the
// reference's 256-thread block kernel (thread v owns packs v, v+256, ... with a
// fused multiply-add chain, then the shfl_down tree); 1/sqrt is the reference's
// integer Newton iteration; the butterfly adds associate left to right; bf16
// roundings sit where the reference stores bf16 between its kernels.
#include "kernels.cuh"
#include "runtime.h"

#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include <algorithm>
#include <stdexcept>
#include <string>

#include "codec.cuh"
#include "ptx.cuh"

namespace sfq {
namespace {

enum Mode { kModeInt8 = 0, kModeFp4Ref = 1, kModeFp4Feed = 2, kModeNormOnly = 3, kModeRotOnly = 4 };

struct FusedArgs {
  const __nv_bfloat16* x;
  const __nv_bfloat16* norm_w;
  const float* mod_scale;
  const float* mod_shift;
  const int32_t* mod_index;
  float eps;
  int rows, dim;
  int apply_convrot;
  int8_t* q;
  float* row_scale;
  uint8_t* packed;
  uint8_t* scales;
  __nv_bfloat16* bf16_out;  // normed activation (optional) or the rotated one (rot-only mode)
};

// ---- integer-exact norm reciprocal (include/slopfab/cuda/deterministic_math.cuh:26-197) ----
__device__ __forceinline__ uint64_t shift_rne(uint64_t v, unsigned s) {
  const uint64_t q = v >> s;
  const uint64_t rem = v & ((uint64_t(1) << s) - 1);
  const uint64_t half = uint64_t(1) << (s - 1);
  return q + ((rem > half || (rem == half && (q & 1))) ? 1 : 0);
}
// 1/sqrt(v) for a positive normal v: Newton in unsigned Q30 with round-half-even shifts, six
// steps from a seed chosen by the exponent's parity, then rounded to 24 bits.
__device__ float rsqrt_q30(float value) {
  const uint32_t mag = __float_as_uint(value) & 0x7FFFFFFFu;
  if (mag == 0u) return __uint_as_float(0x7F800000u);
  if ((__float_as_uint(value) & 0x80000000u) || mag > 0x7F800000u) return __uint_as_float(0x7FC00000u);
  if (mag == 0x7F800000u) return 0.0f;
  uint32_t sig = mag & 0x007FFFFFu;
  int expo;
  if (mag < 0x00800000u) {
    const int t = 31 - __clz(sig);
    expo = t - 149;
    sig <<= unsigned(23 - t);
  } else {
    expo = int(mag >> 23) - 127;
    sig |= 0x00800000u;
  }
  const int odd = expo & 1;
  const uint64_t m = uint64_t(sig) << (7 + odd);
  const int out_scale = -(expo - odd) / 2;
  uint64_t y = odd ? 637534208ull : 872415232ull;
#pragma unroll 1
  for (int it = 0; it < 6; ++it) {
    const uint64_t y2 = shift_rne(y * y, 30);
    const uint64_t my2 = shift_rne(m * y2, 30);
    y = shift_rne(y * (3ull * (1ull << 30) - my2), 31);
  }
  int t = 63 - __clzll((long long)y);
  uint64_t r = shift_rne(y, unsigned(t - 23));
  if (r == (1ull << 24)) {
    r >>= 1;
    ++t;
  }
  return __uint_as_float((uint32_t(t - 30 + out_scale + 127) << 23) | (uint32_t(r) & 0x007FFFFFu));
}
// rsqrt(RNE(sum / dim) + eps); IEEE division and addition are the reference's integer forms.
__device__ float norm_rsqrt(float sum, int dim, float eps) {
  const float mean = sum == 0.0f ? 0.0f : __fdiv_rn(sum, float(dim));
  return rsqrt_q30(__fadd_rn(mean, eps));
}

// One radix-4 stage of the regular Hadamard on (a,b,c,d) -> rows of h4, each a left-to-right
// sum as in convrot_kernel (src/cuda/linear_weights.cu:458-461). a-b is exactly -(b-a), so the
// four outputs cost ten additions instead of twelve.
__device__ __forceinline__ void h4(float& a, float& b, float& c, float& d) {
  const float s = __fadd_rn(a, b);
  const float u = __fsub_rn(a, b);
  const float r0 = __fsub_rn(__fadd_rn(s, c), d);
  const float r1 = __fadd_rn(__fsub_rn(s, c), d);
  const float r2 = __fadd_rn(__fadd_rn(u, c), d);
  const float r3 = __fadd_rn(__fadd_rn(-u, c), d);
  a = r0, b = r1, c = r2, d = r3;
}
// Two stages (strides 1 and 4) over 16 values held by one thread.
__device__ __forceinline__ void two_stages(float (&v)[16]) {
#pragma unroll
  for (int b = 0; b < 4; ++b) h4(v[4 * b], v[4 * b + 1], v[4 * b + 2], v[4 * b + 3]);
#pragma unroll
  for (int i = 0; i < 4; ++i) h4(v[i], v[i + 4], v[i + 8], v[i + 12]);
}

__device__ __forceinline__ float round_bf16(float f) { return __bfloat162float(__float2bfloat16(f)); }

// One token row. `r0`, `r1` are this thread's 16 bf16 elements, already loaded (zero for an inactive thread).
// A thread may return early only where no block-wide barrier follows in this function.
template <int MODE>
__device__ __forceinline__ void process_row(const FusedArgs& a, const int row, uint4 r0, uint4 r1, uint8_t* smem) {
  // [tile: 17 floats per thread][partials: 256 + 8 + 8 floats][raw row: dim bf16 when the norm is on]
  float* tile = reinterpret_cast<float*>(smem);
  float* partial = tile + size_t(blockDim.x) * 17;
  float* warp_tot = partial + 256;
  float* bcast = warp_tot + 8;
  uint4* raw = reinterpret_cast<uint4*>(bcast + 8);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int chunks = a.dim >> 4;
  const bool active = tid < chunks;

  if constexpr (MODE == kModeFp4Feed) {
    if (row >= a.rows) {  // padding rows of the last 128-row scale tile: zero scales
      if (active) a.scales[nvfp4_scale_offset(row, tid, chunks)] = 0;
      return;
    }
  }

  float v[16];
  {
    const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&r0);
    const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f0 = __bfloat1622float2(h0[i]), f1 = __bfloat1622float2(h1[i]);
      v[2 * i] = f0.x, v[2 * i + 1] = f0.y, v[8 + 2 * i] = f1.x, v[8 + 2 * i + 1] = f1.y;
    }
    if (a.norm_w != nullptr && active) {
      raw[tid * 2] = r0;
      raw[tid * 2 + 1] = r1;
    }
  }

  // ---------------------------------------------------------------- RMSNorm [+ modulate]
  if (a.norm_w != nullptr) {
    __syncthreads();
    const int packs = a.dim >> 3;
    for (int vt = tid; vt < 256; vt += blockDim.x) {  // virtual thread vt of the 256-thread block kernel
      float s = 0.0f;
      for (int p = vt; p < packs; p += 256) {
        const uint4 pk = raw[p];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&pk);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          s = __fmaf_rn(f.x, f.x, s);
          s = __fmaf_rn(f.y, f.y, s);
        }
      }
      partial[vt] = s;
    }
    __syncthreads();
    if (tid < 32) {
      for (int w = 0; w < 8; ++w) {  // shfl_down tree of each virtual warp
        float s = partial[w * 32 + lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s = __fadd_rn(s, __shfl_down_sync(0xFFFFFFFFu, s, off));
        if (lane == 0) warp_tot[w] = s;
      }
      __syncwarp();
      float s = lane < 8 ? warp_tot[lane] : 0.0f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) s = __fadd_rn(s, __shfl_down_sync(0xFFFFFFFFu, s, off));
      if (lane == 0) bcast[0] = norm_rsqrt(s, a.dim, a.eps);
    }
    __syncthreads();
    const float inv = bcast[0];
    if (active) {
      const uint4* wp = reinterpret_cast<const uint4*>(a.norm_w) + tid * 2;
      const uint4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
      const __nv_bfloat162* wh0 = reinterpret_cast<const __nv_bfloat162*>(&w0);
      const __nv_bfloat162* wh1 = reinterpret_cast<const __nv_bfloat162*>(&w1);
      float w[16];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f0 = __bfloat1622float2(wh0[i]), f1 = __bfloat1622float2(wh1[i]);
        w[2 * i] = f0.x, w[2 * i + 1] = f0.y, w[8 + 2 * i] = f1.x, w[8 + 2 * i + 1] = f1.y;
      }
      if (a.mod_scale != nullptr) {
        const size_t mod = size_t(a.mod_index[row]) * a.dim + size_t(tid) * 16;
        const float4* sc = reinterpret_cast<const float4*>(a.mod_scale + mod);
        const float4* sh = reinterpret_cast<const float4*>(a.mod_shift + mod);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 s4 = __ldg(sc + j), h4v = __ldg(sh + j);
          const float ss[4] = {s4.x, s4.y, s4.z, s4.w}, hh[4] = {h4v.x, h4v.y, h4v.z, h4v.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float n = __fmul_rn(__fmul_rn(v[4 * j + i], inv), w[4 * j + i]);
            v[4 * j + i] = round_bf16(__fmaf_rn(n, __fadd_rn(1.0f, ss[i]), hh[i]));
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = round_bf16(__fmul_rn(__fmul_rn(v[i], inv), w[i]));
      }
    }
    if (a.bf16_out != nullptr && MODE != kModeRotOnly && active) {
      uint4 o[2];
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
      for (int i = 0; i < 8; ++i) op[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      uint4* dst = reinterpret_cast<uint4*>(a.bf16_out + size_t(row) * a.dim) + tid * 2;
      dst[0] = o[0];
      dst[1] = o[1];
    }
  }
  if constexpr (MODE == kModeNormOnly) return;

  if constexpr (MODE == kModeInt8 || MODE == kModeRotOnly) {
    // ------------------------------------------------------------ ConvRot-256
    if (a.apply_convrot) {
      // Element i = 16*T + e of the group sits at word 17*T + e of the group's tile: a thread's own 16
      // words are consecutive, and the 16 threads' words for a fixed e fall in 16 distinct banks.
      float* grp = tile + (tid >> 4) * 272;
      const int T = tid & 15;
      two_stages(v);  // strides 1 and 4
#pragma unroll
      for (int e = 0; e < 16; ++e) grp[17 * T + e] = v[e];
      __syncwarp();
#pragma unroll
      for (int t = 0; t < 16; ++t) v[t] = grp[17 * t + T];  // now v[t] = element 16*t + T
      two_stages(v);  // strides 16 and 64
      __syncwarp();
#pragma unroll
      for (int t = 0; t < 16; ++t) grp[17 * t + T] = round_bf16(v[t] * 0.0625f);  // 1/16, then the bf16 store
      __syncwarp();
#pragma unroll
      for (int e = 0; e < 16; ++e) v[e] = grp[17 * T + e];
    }
    if constexpr (MODE == kModeRotOnly) {
      if (active) {
        uint4 o[2];
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(o);
#pragma unroll
        for (int i = 0; i < 8; ++i) op[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        uint4* dst = reinterpret_cast<uint4*>(a.bf16_out + size_t(row) * a.dim) + tid * 2;
        dst[0] = o[0];
        dst[1] = o[1];
      }
      return;
    }
    // ------------------------------------------------------------ per-token int8 (src/cuda/w4a8.cu:193-216)
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    __syncthreads();  // `partial` may still be read by slow warps of the norm phase
    if (lane == 0) partial[tid >> 5] = amax;
    __syncthreads();
    if (tid < 32) {
      float m = tid < int(blockDim.x >> 5) ? partial[tid] : 0.0f;
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, off));
      if (tid == 0) {
        const float scale = fmaxf(__fdiv_rn(m, 127.0f), 1e-30f);
        bcast[1] = scale;
        a.row_scale[row] = scale;
      }
    }
    __syncthreads();
    const float divisor = round_bf16(bcast[1]);
    // x / divisor, correctly rounded, without a division per element: with r = RN(1/d) exactly rounded,
    // q0 = RN(x r), e = x - d q0 (exact in one fused multiply-add) and q = RN(q0 + e r) is the IEEE quotient.
    const float rcp = __frcp_rn(divisor);
    if (active) {
      uint32_t o[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        int q[4];
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
          const float x0 = v[4 * w + j], x1 = v[4 * w + j + 1];
          const float a0 = __fmul_rn(x0, rcp), a1 = __fmul_rn(x1, rcp);
          const float q0 = __fmaf_rn(__fmaf_rn(-a0, divisor, x0), rcp, a0);
          const float q1 = __fmaf_rn(__fmaf_rn(-a1, divisor, x1), rcp, a1);
          const float2 f = __bfloat1622float2(__floats2bfloat162_rn(q0, q1));  // the quotient is rounded to bf16 first
          q[j] = __float2int_rn(f.x);
          q[j + 1] = __float2int_rn(f.y);
        }
        // saturating pack to int8 = clamp to [-128, 127]
        uint32_t hi, all;
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(q[3]), "r"(q[2]), "r"(0));
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(all) : "r"(q[1]), "r"(q[0]), "r"(hi));
        o[w] = all;
      }
      reinterpret_cast<uint4*>(a.q + size_t(row) * a.dim)[tid] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  } else {
    // ------------------------------------------------------------ per-16 fp4 (src/cuda/nvfp4_gemm.cu:107-158)
    if (!active) return;
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const uint8_t s8 = __nv_cvt_float_to_fp8(amax * (1.0f / 6.0f), __NV_SATFINITE, __NV_E4M3);
    const float decoded = e4m3_decode(s8);
    const float inv = decoded > 0.0f ? __fdiv_rn(1.0f, decoded) : 0.0f;
    uint32_t words[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float even = v[2 * i] * inv, odd = v[2 * i + 1] * inv;
      // The conversion puts its first component in the low nibble. The reference layout wants the even
      // element there; the GEMM feed wants it in the high nibble, like the weight files.
      const __nv_fp4x2_storage_t b = MODE == kModeFp4Ref
                                         ? __nv_cvt_float2_to_fp4x2(make_float2(even, odd), __NV_E2M1, cudaRoundNearest)
                                         : __nv_cvt_float2_to_fp4x2(make_float2(odd, even), __NV_E2M1, cudaRoundNearest);
      words[i >> 2] |= uint32_t(b) << (8 * (i & 3));
    }
    reinterpret_cast<uint2*>(a.packed + size_t(row) * (a.dim >> 1))[tid] = make_uint2(words[0], words[1]);
    if constexpr (MODE == kModeFp4Ref)
      a.scales[size_t(row) * chunks + tid] = s8;
    else
      a.scales[nvfp4_scale_offset(row, tid, chunks)] = s8;
  }
}

// The kernel: a CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ... and loads the NEXT row's 32 bytes per
// thread before working on the current one, so every resident warp always has a load in flight (one row per
// CTA without prefetch keeps too few bytes in flight to cover HBM latency).
template <int MODE>
__global__ void __launch_bounds__(1024, 1) fused_act_kernel(FusedArgs a) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int chunks = a.dim >> 4;
  const bool active = int(threadIdx.x) < chunks;
  const int total_rows = MODE == kModeFp4Feed ? (a.rows + 127) / 128 * 128 : a.rows;
  auto load = [&](int row, uint4& r0, uint4& r1) {
    r0 = make_uint4(0, 0, 0, 0);
    r1 = r0;
    if (active && row < a.rows) {
      const uint4* src = reinterpret_cast<const uint4*>(a.x + size_t(row) * a.dim) + threadIdx.x * 2;
      r0 = __ldg(src);
      r1 = __ldg(src + 1);
    }
  };
  uint4 r0, r1, n0, n1;
  int row = blockIdx.x;
  load(row, r0, r1);
  for (; row < total_rows; row += gridDim.x) {
    load(row + gridDim.x, n0, n1);
    process_row<MODE>(a, row, r0, r1, smem);
    __syncthreads();  // shared memory is reused by the next row
    r0 = n0;
    r1 = n1;
  }
}

// Generic rotation for the other power-of-four groups (4, 16, 64): not on the hot path (the INT8
// weight-only format of the text encoder); one block of 64 threads per 256 columns.
__global__ void __launch_bounds__(64)
convrot_small_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int dim, int stages,
                     float norm) {
  __shared__ float v[256 + 64];
  const int row = blockIdx.x, c0 = blockIdx.y * 256, t = threadIdx.x;
  const int n = min(256, dim - c0);
  const size_t base = size_t(row) * dim + c0;
  for (int i = t; i < n; i += 64) v[i + (i >> 2)] = __bfloat162float(in[base + i]);
  __syncthreads();
  int stride = 1;
  for (int s = 0; s < stages; ++s) {
    const int i = (t / stride) * 4 * stride + (t % stride);
    const bool live = i + 3 * stride < n;
    const int j0 = i, j1 = i + stride, j2 = i + 2 * stride, j3 = i + 3 * stride;
    float a = 0, b = 0, c = 0, d = 0;
    if (live) a = v[j0 + (j0 >> 2)], b = v[j1 + (j1 >> 2)], c = v[j2 + (j2 >> 2)], d = v[j3 + (j3 >> 2)];
    __syncthreads();
    if (live) {
      h4(a, b, c, d);
      v[j0 + (j0 >> 2)] = a, v[j1 + (j1 >> 2)] = b, v[j2 + (j2 >> 2)] = c, v[j3 + (j3 >> 2)] = d;
    }
    __syncthreads();
    stride *= 4;
  }
  for (int i = t; i < n; i += 64) out[base + i] = __float2bfloat16(v[i + (i >> 2)] * norm);
}

inline void check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <int MODE> void launch_fused(const FusedArgs& a, int grid_rows, cudaStream_t stream, const char* what) {
  if (a.dim % 16 != 0 || a.dim > 16384)
    throw std::invalid_argument(std::string(what) + ": dim must be a multiple of 16 and at most 16384");
  if (reinterpret_cast<uintptr_t>(a.x) % 16 != 0)
    throw std::invalid_argument(std::string(what) + ": activation pointer must be 16-byte aligned");
  if (a.norm_w != nullptr && a.mod_scale != nullptr && (a.mod_shift == nullptr || a.mod_index == nullptr))
    throw std::invalid_argument(std::string(what) + ": modulation needs scale, shift and the row index");
  const int threads = ((a.dim / 16 + 31) / 32) * 32;
  const size_t smem = size_t(threads) * 17 * 4 + (256 + 16) * 4 + (a.norm_w ? size_t(a.dim) * 2 : 0);
  reserve_dynamic_smem(reinterpret_cast<const void*>(&fused_act_kernel<MODE>), smem, what);
  // As many CTAs as stay resident at once; each walks rows with a stride of the grid size.
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fused_act_kernel<MODE>, threads, smem) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const int grid = std::min(grid_rows, per_sm * device_sm_count());
  fused_act_kernel<MODE><<<grid, threads, smem, stream>>>(a);
  check_launch(what);
}

FusedArgs base_args(const __nv_bfloat16* x, const NormArgs& n, int rows, int dim) {
  FusedArgs a{};
  a.x = x;
  a.norm_w = n.weight;
  a.mod_scale = n.weight ? n.scale : nullptr;
  a.mod_shift = n.weight ? n.shift : nullptr;
  a.mod_index = n.weight ? n.index : nullptr;
  a.eps = n.eps;
  a.rows = rows;
  a.dim = dim;
  return a;
}

}  // namespace

void rmsnorm(const __nv_bfloat16* x, const NormArgs& norm, __nv_bfloat16* out, int rows, int dim, cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) throw std::invalid_argument("rmsnorm: rows and dim must be positive");
  if (!x || !out || !norm.weight) throw std::invalid_argument("rmsnorm: null buffer");
  FusedArgs a = base_args(x, norm, rows, dim);
  a.bf16_out = out;
  launch_fused<kModeNormOnly>(a, rows, stream, "rmsnorm");
}

void convrot(const __nv_bfloat16* x, __nv_bfloat16* out, int rows, int dim, int group, cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) return;
  if (!x || !out) throw std::invalid_argument("convrot: null buffer");
  int stages = 0, n = 1;
  while (n < group) n *= 4, ++stages;
  if (n != group) throw std::runtime_error("convrot: group size must be a power of four, got " + std::to_string(group));
  if (dim % group != 0) throw std::runtime_error("convrot: dim must be a multiple of the group size");
  if (group == 256 && dim <= 16384) {
    FusedArgs a = base_args(x, NormArgs{}, rows, dim);
    a.apply_convrot = 1;
    a.bf16_out = out;
    launch_fused<kModeRotOnly>(a, rows, stream, "convrot");
    return;
  }
  if (group > 256) throw std::runtime_error("convrot: groups above 256 are not supported");
  convrot_small_kernel<<<dim3(rows, (dim + 255) / 256), 64, 0, stream>>>(x, out, dim, stages, 1.0f / float(1 << stages));
  check_launch("convrot");
}

void quantize_int8_token(const __nv_bfloat16* x, const NormArgs& norm, int8_t* q, float* row_scale,
                         __nv_bfloat16* normed_out, int rows, int dim, bool apply_convrot, cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) throw std::invalid_argument("W4A8 activation shape");
  if (!x || !q || !row_scale) throw std::invalid_argument("quantize_int8_token: null buffer");
  if (apply_convrot && dim % 256 != 0) throw std::invalid_argument("W4A8 activation requires K divisible by 256");
  if (reinterpret_cast<uintptr_t>(q) % 16 != 0) throw std::invalid_argument("quantize_int8_token: output must be 16-byte aligned");
  // The Linear's own case (rotation on, nothing fused in front, K <= 6144) has a two-rows-per-step kernel.
  if (apply_convrot && norm.weight == nullptr && quantize_int8_rot_pairs(x, q, row_scale, rows, dim, stream)) return;
  FusedArgs a = base_args(x, norm, rows, dim);
  a.q = q;
  a.row_scale = row_scale;
  a.apply_convrot = apply_convrot ? 1 : 0;
  a.bf16_out = norm.weight ? normed_out : nullptr;
  launch_fused<kModeInt8>(a, rows, stream, "quantize_int8_token");
}

size_t nvfp4_act_scale_bytes(int rows, int dim) {
  if (rows <= 0 || dim <= 0) return 0;
  return size_t((rows + 127) / 128) * 128 * size_t(dim / 16);
}

// ---- per-16-block fp4 quantizer without a norm in front (the Linear's own case) --------------------------------------
// The same arithmetic as the fp4 branch of process_row (quantize_act_kernel, src/cuda/nvfp4_gemm.cu:107-158): per 16
// elements s8 = e4m3_rn_sat(amax / 6), inv = 1 / decode(s8) (0 for an all-zero block), code = e2m1_rn_sat(x * inv). A
// block's scale depends on that block alone, so there is nothing to exchange between threads: the activation is walked as
// a flat array of 16-element blocks, two per thread in flight, with no barrier and no shared memory, the maximum on
// bf16x2 words and the products on packed fp32 pairs. FEED: high nibble = even element, scales in the 128x4-tiled layout
// with the rows padded to a multiple of 128 (the pad rows' scales are written as zero).
namespace {
__device__ __forceinline__ uint32_t habs2(uint32_t a) {
  uint32_t d;
  asm("abs.bf16x2 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t hmax2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <bool FEED>
__device__ __forceinline__ void quantize_block16(const uint4 r0, const uint4 r1, uint2& codes, uint8_t& s8) {
  const uint32_t w[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};  // element 2i in the low half of word i
  uint32_t m = hmax2(hmax2(hmax2(habs2(w[0]), habs2(w[1])), hmax2(habs2(w[2]), habs2(w[3]))),
                     hmax2(hmax2(habs2(w[4]), habs2(w[5])), hmax2(habs2(w[6]), habs2(w[7]))));
  m = hmax2(m, m >> 16);
  const float amax = __uint_as_float(m << 16);
  s8 = uint8_t(__nv_cvt_float_to_fp8(amax * (1.0f / 6.0f), __NV_SATFINITE, __NV_E4M3));
  const float decoded = __half2float(__half(__nv_cvt_fp8_to_halfraw(s8, __NV_E4M3)));
  const float inv = decoded > 0.0f ? __frcp_rn(decoded) : 0.0f;  // the correctly rounded reciprocal, as 1.0f / decoded
  const ptx::f32x2 inv2 = ptx::pack2(inv, inv);
  uint32_t out[2] = {0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float even, odd;
    ptx::unpack2(ptx::mul2(ptx::pack2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u)), inv2), even, odd);
    // The conversion puts its first component in the low nibble. The reference layout wants the even element there; the
    // GEMM feed wants it in the high nibble, like the weight files.
    const __nv_fp4x2_storage_t b = FEED ? __nv_cvt_float2_to_fp4x2(make_float2(odd, even), __NV_E2M1, cudaRoundNearest)
                                        : __nv_cvt_float2_to_fp4x2(make_float2(even, odd), __NV_E2M1, cudaRoundNearest);
    out[i >> 2] |= uint32_t(b) << (8 * (i & 3));
  }
  codes = make_uint2(out[0], out[1]);
}

template <bool FEED>
__global__ void __launch_bounds__(256) quantize_nvfp4_flat_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ packed,
                                                                  uint8_t* __restrict__ scales, int rows, int padded_rows, int chunks) {
  // item g = (row, chunk): advance by the grid's stride without a division per item
  const uint32_t stride = gridDim.x * blockDim.x;
  const uint32_t first = blockIdx.x * blockDim.x + threadIdx.x;
  int row = int(first / uint32_t(chunks)), c = int(first % uint32_t(chunks));
  const int drow = int(stride / uint32_t(chunks)), dc = int(stride % uint32_t(chunks));
  auto load = [&](int r, int cc, uint4& a, uint4& b) {
    a = make_uint4(0, 0, 0, 0);
    b = a;
    if (r < rows) {
      const uint4* src = reinterpret_cast<const uint4*>(x) + (size_t(r) * chunks + cc) * 2;
      a = __ldg(src);
      b = __ldg(src + 1);
    }
  };
  auto emit = [&](int r, int cc, const uint4& a, const uint4& b) {
    if (r >= padded_rows) return;
    uint2 codes;
    uint8_t s8 = 0;
    if (r < rows) {
      quantize_block16<FEED>(a, b, codes, s8);
      reinterpret_cast<uint2*>(packed)[size_t(r) * chunks + cc] = codes;
    }
    scales[FEED ? nvfp4_scale_offset(r, cc, chunks) : size_t(r) * chunks + cc] = s8;
  };
  while (row < padded_rows) {
    int row2 = row + drow, c2 = c + dc;
    if (c2 >= chunks) c2 -= chunks, ++row2;
    uint4 a0, b0, a1, b1;
    load(row, c, a0, b0);
    load(row2, c2, a1, b1);
    emit(row, c, a0, b0);
    emit(row2, c2, a1, b1);
    row = row2 + drow, c = c2 + dc;
    if (c >= chunks) c -= chunks, ++row;
  }
}

template <bool FEED>
void launch_nvfp4_flat(const __nv_bfloat16* x, uint8_t* packed, uint8_t* scales, int rows, int dim, cudaStream_t stream) {
  const int chunks = dim / 16;
  const int padded = FEED ? (rows + 127) / 128 * 128 : rows;
  const size_t items = size_t(padded) * chunks;
  if (items >= (size_t(1) << 31)) throw std::invalid_argument("quantize_nvfp4_block: too many 16-element blocks for one launch");
  const int ctas = int(std::min<size_t>((items + 511) / 512, size_t(device_sm_count()) * 8));  // two items per thread and trip
  quantize_nvfp4_flat_kernel<FEED><<<ctas, 256, 0, stream>>>(x, packed, scales, rows, padded, chunks);
  check_launch("quantize_nvfp4_block");
}
}  // namespace

void quantize_nvfp4_block(const __nv_bfloat16* x, const NormArgs& norm, uint8_t* packed, uint8_t* scales,
                          __nv_bfloat16* normed_out, int rows, int dim, int layout, cudaStream_t stream) {
  if (rows <= 0 || dim <= 0) return;
  if (!x || !packed || !scales) throw std::invalid_argument("quantize_nvfp4_block: null buffer");
  if (dim % 16 != 0)
    throw std::runtime_error("nvfp4: activation dim must be a multiple of 16, got " + std::to_string(dim));
  if (reinterpret_cast<uintptr_t>(packed) % 8 != 0) throw std::invalid_argument("quantize_nvfp4_block: output must be 8-byte aligned");
  if (layout != SFQ_NVFP4_ACT_REFERENCE && layout != SFQ_NVFP4_ACT_GEMM_FEED) throw std::invalid_argument("quantize_nvfp4_block: unknown layout");
  if (layout == SFQ_NVFP4_ACT_GEMM_FEED && dim % 64 != 0)
    throw std::invalid_argument("quantize_nvfp4_block: the tiled scale layout needs dim % 64 == 0");
  if (norm.weight == nullptr) {  // no norm in front: the barrier-free kernel
    if (reinterpret_cast<uintptr_t>(x) % 16 != 0) throw std::invalid_argument("quantize_nvfp4_block: activation pointer must be 16-byte aligned");
    if (layout == SFQ_NVFP4_ACT_REFERENCE)
      launch_nvfp4_flat<false>(x, packed, scales, rows, dim, stream);
    else
      launch_nvfp4_flat<true>(x, packed, scales, rows, dim, stream);
    return;
  }
  FusedArgs a = base_args(x, norm, rows, dim);
  a.packed = packed;
  a.scales = scales;
  a.bf16_out = norm.weight ? normed_out : nullptr;
  if (layout == SFQ_NVFP4_ACT_REFERENCE) {
    launch_fused<kModeFp4Ref>(a, rows, stream, "quantize_nvfp4_block");
  } else if (layout == SFQ_NVFP4_ACT_GEMM_FEED) {
    if (dim % 64 != 0) throw std::invalid_argument("quantize_nvfp4_block: the tiled scale layout needs dim % 64 == 0");
    launch_fused<kModeFp4Feed>(a, (rows + 127) / 128 * 128, stream, "quantize_nvfp4_block");
  } else {
    throw std::invalid_argument("quantize_nvfp4_block: unknown layout");
  }
}

// ---- head-wise q/k RMSNorm and MM-RoPE, the two steps between the fused projection and attention ----
// launch_head_rmsnorm (src/cuda/nn_kernels.cu:296-305 -> rmsnorm_warp_kernel, :100-136) followed by launch_rope_h3
// (src/cuda/nn_position.cu:15-68,111-123), in place, one warp per (row, head), head_dim 128, on a row pitch so that
// the q and k thirds of the fused projection are processed where they lie. Bit-exact: 16 lanes hold 8 channels each;
// the sum of squares is the reference's per-lane chain and xor butterfly; the normalised value is rounded to bf16
// before the rotation (the reference stores it between its two kernels); the rotation pairs channel j with j + 48
// over the first 96 channels with the reference's subnormal canonicalisation at every step.
namespace {
__device__ __forceinline__ float rope_bf16_value(unsigned short bits) {
  return (bits & 0x7fffu) < 0x0080u ? __uint_as_float(unsigned(bits & 0x8000u) << 16) : __uint_as_float(unsigned(bits) << 16);
}
__device__ __forceinline__ float rope_float_value(float value) {
  const unsigned bits = __float_as_uint(value);
  return (bits & 0x7fffffffu) < 0x00800000u ? __uint_as_float(bits & 0x80000000u) : value;
}
__device__ __forceinline__ unsigned short rope_bf16_result(float value) {
  const unsigned short bits = __bfloat16_as_ushort(__float2bfloat16(value));
  return (bits & 0x7fffu) < 0x0080u ? (unsigned short)(bits & 0x8000u) : bits;
}
__device__ __forceinline__ float rope_fma_product(float a, float b, float base) {
  const float product = __fmul_rn(a, b);
  const unsigned magnitude = __float_as_uint(product) & 0x7fffffffu;
  if (magnitude < 0x00800000u && (__float_as_uint(a) & 0x7fffffffu) != 0u && (__float_as_uint(b) & 0x7fffffffu) != 0u) return base;
  return fmaf(a, b, base);
}

__global__ void __launch_bounds__(256) head_norm_rope_kernel(__nv_bfloat16* __restrict__ x, int ld, const __nv_bfloat16* __restrict__ w,
                                                             const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                                                             int rows, int heads, float eps) {
  const int lane = threadIdx.x & 31;
  const long long unit = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);  // (row, head)
  if (unit >= (long long)rows * heads) return;
  const int row = int(unit / heads), head = int(unit % heads);
  __nv_bfloat16* v = x + size_t(row) * ld + head * 128;
  const bool active = lane < 16;
  uint4 raw = make_uint4(0, 0, 0, 0);
  if (active) raw = *reinterpret_cast<const uint4*>(v + lane * 8);
  unsigned short h[8];
  {
    const unsigned u[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) h[2 * i] = (unsigned short)(u[i] & 0xFFFFu), h[2 * i + 1] = (unsigned short)(u[i] >> 16);
  }
  if (w != nullptr) {
    float buf[8];
    float sum_sq = 0.0f;
    if (active) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        buf[i] = __uint_as_float(unsigned(h[i]) << 16);
        sum_sq = fmaf(buf[i], buf[i], sum_sq);
      }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) sum_sq = __fadd_rn(sum_sq, __shfl_xor_sync(0xFFFFFFFFu, sum_sq, offset));
    float inv = lane == 0 ? norm_rsqrt(sum_sq, 128, eps) : 0.0f;
    inv = __shfl_sync(0xFFFFFFFFu, inv, 0);
    if (active) {
      const uint4 wr = *reinterpret_cast<const uint4*>(w + lane * 8);
      const unsigned wu[4] = {wr.x, wr.y, wr.z, wr.w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float wf = __uint_as_float(((wu[i >> 1] >> (16 * (i & 1))) & 0xFFFFu) << 16);
        h[i] = __bfloat16_as_ushort(__float2bfloat16(__fmul_rn(__fmul_rn(buf[i], inv), wf)));
      }
    }
  }
  if (cos_tab != nullptr) {
    // lanes 0-5 hold channels j = 8*lane .. (the low halves), lanes 6-11 their partners j + 48, lanes 12-15 pass through
    const bool low = lane < 6, high = lane >= 6 && lane < 12;
    const int partner = low ? lane + 6 : lane - 6;
    unsigned short other[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const unsigned mine = unsigned(h[2 * i]) | (unsigned(h[2 * i + 1]) << 16);
      const unsigned got = __shfl_sync(0xFFFFFFFFu, mine, partner & 31);
      other[2 * i] = (unsigned short)(got & 0xFFFFu), other[2 * i + 1] = (unsigned short)(got >> 16);
    }
    if (low || high) {
      const int j0 = (low ? lane : lane - 6) * 8;
      const float* cr = cos_tab + size_t(row) * 96 + j0;
      const float* sr = sin_tab + size_t(row) * 96 + j0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float c = rope_float_value(cr[i]), s = rope_float_value(sr[i]);
        const float lo = rope_bf16_value(low ? h[i] : other[i]);
        const float hi = rope_bf16_value(low ? other[i] : h[i]);
        if (low) {
          const float left = rope_float_value(__fmul_rn(lo, c)), right = rope_float_value(__fmul_rn(hi, s));
          h[i] = rope_bf16_result(__fsub_rn(left, right));
        } else {
          const float base = rope_float_value(__fmul_rn(hi, c));
          h[i] = rope_bf16_result(rope_fma_product(lo, s, base));
        }
      }
    }
  }
  if (active) {
    uint4 o;
    o.x = unsigned(h[0]) | (unsigned(h[1]) << 16), o.y = unsigned(h[2]) | (unsigned(h[3]) << 16);
    o.z = unsigned(h[4]) | (unsigned(h[5]) << 16), o.w = unsigned(h[6]) | (unsigned(h[7]) << 16);
    *reinterpret_cast<uint4*>(v + lane * 8) = o;
  }
}
}  // namespace

void head_norm_rope(__nv_bfloat16* x, int ld, const __nv_bfloat16* norm_weight, const float* cos_tab, const float* sin_tab, int rows,
                    int heads, int head_dim, float eps, cudaStream_t stream) {
  if (rows <= 0 || heads <= 0) throw std::runtime_error("head_norm_rope: rows and heads must be positive");
  if (head_dim != 128) throw std::runtime_error("head_norm_rope: built for head_dim 128 (96 rotary channels + 32 passed through)");
  if (x == nullptr || (norm_weight == nullptr && cos_tab == nullptr)) throw std::invalid_argument("head_norm_rope: nothing to do");
  if ((cos_tab == nullptr) != (sin_tab == nullptr)) throw std::invalid_argument("head_norm_rope: cos and sin come together");
  if (ld < heads * 128 || ld % 8 != 0 || reinterpret_cast<uintptr_t>(x) % 16 != 0 ||
      (norm_weight != nullptr && reinterpret_cast<uintptr_t>(norm_weight) % 16 != 0))
    throw std::invalid_argument("head_norm_rope: the row pitch must cover heads * 128 and keep 16-byte alignment");
  const long long units = (long long)rows * heads;
  head_norm_rope_kernel<<<unsigned((units + 7) / 8), 256, 0, stream>>>(x, ld, norm_weight, cos_tab, sin_tab, rows, heads, eps);
  check_launch("head_norm_rope");
}

}  // namespace sfq
