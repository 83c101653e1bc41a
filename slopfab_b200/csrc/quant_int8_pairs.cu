// ConvRot-256 + per-token int8 quantizer, two token rows per step with packed fp32x2 arithmetic.
//
// Same bits as the fused kernel of act_quant.cu (and so as the reference's convrot_kernel followed by
// quantize_bf16, src/cuda/linear_weights.cu:422-471 and src/cuda/w4a8.cu:193-216), for the case the W4A8 / W6A8
// Linear runs in its chunk loop: no norm in front, rotation on (K up to 6144 with one 16-element chunk per thread,
// wider rows with two to four). That kernel is bound by instruction
// issue, not by HBM, so this one halves the instruction count per row:
//   * a thread holds its 16 elements of TWO rows as 16 fp32x2 pairs (row r in the low half, row r+1 in the high
//     half); every butterfly add, the 1/16 scale and the quotient are one add/mul.rn.f32x2 for both;
//   * the in-group transposes move 64-bit pairs (half the shared-memory instructions);
//   * the absolute maximum runs on bf16x2 words (both rows per max.bf16x2);
//   * the rotated values are quantized in the transposed layout; the int8 bytes of both rows go to shared memory as
//     one 16-bit store per element and come back as two 16-byte rows, so the second float transpose disappears;
//   * one block-wide barrier per row pair: every thread folds the per-warp maxima itself. (A split-phase form of that
//     barrier -- an mbarrier a warp arrives on when its maximum is written and waits on only after it has rotated the
//     NEXT row pair, 92 registers, two CTAs per SM -- was built and measured: 3.04 TB/s against 3.2 for this form at
//     32768 x 5120, same bits. The kernel is bound by its instruction count, not by warps idling at the barrier.)
#include "kernels.cuh"
#include "runtime.h"

#include <algorithm>
#include <stdexcept>
#include <string>

namespace sfq {
namespace {

using f2 = unsigned long long;  // two fp32 in one 64-bit register: .x = row r, .y = row r + 1

__device__ __forceinline__ f2 pk(float lo, float hi) {
  f2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ f2 pku(uint32_t lo, uint32_t hi) {
  f2 d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}
__device__ __forceinline__ void upk(f2 v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ f2 add2(f2 a, f2 b) {
  f2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f2 sub2(f2 a, f2 b) {
  f2 d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f2 mul2(f2 a, f2 b) {
  f2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// bf16x2 word: low half = round(lo), high half = round(hi)
__device__ __forceinline__ uint32_t to_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ uint32_t max_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("max.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// One radix-4 stage on four pairs; each output is a left-to-right sum as in convrot_kernel
// (src/cuda/linear_weights.cu:458-461). a-b is exactly -(b-a) and (-u)+c is exactly c-u, so ten operations.
__device__ __forceinline__ void h4(f2& a, f2& b, f2& c, f2& d) {
  const f2 s = add2(a, b);
  const f2 u = sub2(a, b);
  const f2 r0 = sub2(add2(s, c), d);
  const f2 r1 = add2(sub2(s, c), d);
  const f2 r2 = add2(add2(u, c), d);
  const f2 r3 = add2(sub2(c, u), d);
  a = r0, b = r1, c = r2, d = r3;
}
__device__ __forceinline__ void two_stages(f2 (&v)[16]) {
#pragma unroll
  for (int b = 0; b < 4; ++b) h4(v[4 * b], v[4 * b + 1], v[4 * b + 2], v[4 * b + 3]);
#pragma unroll
  for (int i = 0; i < 4; ++i) h4(v[i], v[i + 4], v[i + 8], v[i + 12]);
}

constexpr int kGroupTile = 16 * 17;       // 64-bit words per rotation group (16 threads x 16 pairs, padded)
constexpr int kGroupBytesOut = 512 + 32;  // int8 pairs of a group (256 elements x 2 rows), padded against bank overlap

// x / 127 correctly rounded (r = RN(1/127); exact for every bf16 numerator, as an exhaustive host check shows).
__device__ __forceinline__ float div127(float m) {
  const float r = 1.0f / 127.0f;
  const float q0 = __fmul_rn(m, r);
  return __fmaf_rn(__fmaf_rn(-q0, 127.0f, m), r, q0);
}

// MAXT / MINB: 320 threads (K <= 5120) fit three CTAs per SM in 64 registers; up to 384 threads (K <= 6144) two; up to 1024
// threads (K <= 16384, whole warps) one.
template <int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB)
quantize_int8_pairs_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ row_scale,
                           int rows, int dim) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  const int chunks = dim >> 4;
  const bool active = tid < chunks;
  f2* tile = reinterpret_cast<f2*>(smem) + (tid >> 4) * kGroupTile;  // this thread's group
  uint8_t* bytes = smem + size_t(blockDim.x >> 4) * kGroupTile * 8 + (tid >> 4) * kGroupBytesOut;
  uint32_t* partial = reinterpret_cast<uint32_t*>(smem + size_t(blockDim.x >> 4) * (kGroupTile * 8 + kGroupBytesOut));  // [2][32]
  const int T = tid & 15;
  const int pairs = (rows + 1) >> 1;

  auto load = [&](int pair, uint4 (&r)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) r[i] = make_uint4(0, 0, 0, 0);
    if (active && pair < pairs) {
      const int r0 = 2 * pair;
      const uint4* s0 = reinterpret_cast<const uint4*>(x + size_t(r0) * dim) + tid * 2;
      r[0] = __ldg(s0);
      r[1] = __ldg(s0 + 1);
      if (r0 + 1 < rows) {
        const uint4* s1 = reinterpret_cast<const uint4*>(x + size_t(r0 + 1) * dim) + tid * 2;
        r[2] = __ldg(s1);
        r[3] = __ldg(s1 + 1);
      }
    }
  };

  uint4 cur[4], nxt[4];
  int pair = blockIdx.x;
  load(pair, cur);
  for (int iter = 0; pair < pairs; pair += gridDim.x, ++iter) {
    load(pair + gridDim.x, nxt);
    // bf16 -> fp32 pairs: v[e] = (row r element e, row r+1 element e)
    f2 v[16];
    {
      const uint32_t a[8] = {cur[0].x, cur[0].y, cur[0].z, cur[0].w, cur[1].x, cur[1].y, cur[1].z, cur[1].w};
      const uint32_t b[8] = {cur[2].x, cur[2].y, cur[2].z, cur[2].w, cur[3].x, cur[3].y, cur[3].z, cur[3].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[2 * i] = pku(a[i] << 16, b[i] << 16);
        v[2 * i + 1] = pku(a[i] & 0xFFFF0000u, b[i] & 0xFFFF0000u);
      }
    }
    // ---- ConvRot-256: two stages in registers, transpose inside the 16-thread group, two more stages
    two_stages(v);
#pragma unroll
    for (int e = 0; e < 16; ++e) tile[17 * T + e] = v[e];
    __syncwarp();
#pragma unroll
    for (int t = 0; t < 16; ++t) v[t] = tile[17 * t + T];  // v[t] = element 16 t + T of the group
    two_stages(v);
    // ---- 1/16, the bf16 store of the rotation, and the row maxima on bf16x2 words
    const f2 sixteenth = pk(0.0625f, 0.0625f);
    uint32_t w[16];
    uint32_t amax = 0;
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      float lo, hi;
      upk(mul2(v[t], sixteenth), lo, hi);
      w[t] = to_bf16x2(lo, hi);
      amax = max_bf16x2(amax, w[t] & 0x7FFF7FFFu);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = max_bf16x2(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    uint32_t* part = partial + (iter & 1) * 32;  // two buffers: a fast warp may already be one row pair ahead
    if (lane == 0) part[warp] = amax;
    __syncthreads();
    uint32_t m = 0;
    for (int i = 0; i < nwarps; ++i) m = max_bf16x2(m, part[i]);
    const float m0 = __uint_as_float(m << 16), m1 = __uint_as_float(m & 0xFFFF0000u);
    const float scale0 = fmaxf(div127(m0), 1e-30f), scale1 = fmaxf(div127(m1), 1e-30f);
    const int r0 = 2 * pair;
    if (tid == 0) {
      row_scale[r0] = scale0;
      if (r0 + 1 < rows) row_scale[r0 + 1] = scale1;
    }
    // The divisor is the scale rounded to bf16, and the quotient x / d is rounded to bf16 before the integer rounding.
    // x and d are both bf16 values, so x / d is a ratio of two 8-bit integers times a power of two: it is never a bf16
    // rounding tie and never closer than 7.6e-6 (relative) to one, while x * RN(1/d) is within 1.2e-7 of it. The
    // product therefore rounds to the same bf16 value as the correctly rounded quotient (checked for every pair of
    // mantissas on the host); no refinement step is needed.
    const float d0 = __bfloat162float(__float2bfloat16(scale0)), d1 = __bfloat162float(__float2bfloat16(scale1));
    const f2 rcp = pk(__frcp_rn(d0), __frcp_rn(d1));
#pragma unroll
    for (int t = 0; t < 16; ++t) {
      const f2 xv = pku(w[t] << 16, w[t] & 0xFFFF0000u);
      const f2 qv = mul2(xv, rcp);
      float lo, hi;
      upk(qv, lo, hi);
      const uint32_t qb = to_bf16x2(lo, hi);  // the quotient is rounded to bf16 before the integer rounding
      const int i0 = __float2int_rn(__uint_as_float(qb << 16));
      const int i1 = __float2int_rn(__uint_as_float(qb & 0xFFFF0000u));
      uint32_t two;  // byte 0 = row r, byte 1 = row r+1, both saturated to int8
      asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(two) : "r"(i1), "r"(i0), "r"(0));
      reinterpret_cast<uint16_t*>(bytes)[16 * t + T] = uint16_t(two);
    }
    __syncwarp();
    if (active) {
      // this thread's 16 consecutive elements of both rows, interleaved by row: split them apart
      const uint4 p0 = reinterpret_cast<const uint4*>(bytes)[2 * T], p1 = reinterpret_cast<const uint4*>(bytes)[2 * T + 1];
      uint4 o0, o1;
      o0.x = __byte_perm(p0.x, p0.y, 0x6420), o1.x = __byte_perm(p0.x, p0.y, 0x7531);
      o0.y = __byte_perm(p0.z, p0.w, 0x6420), o1.y = __byte_perm(p0.z, p0.w, 0x7531);
      o0.z = __byte_perm(p1.x, p1.y, 0x6420), o1.z = __byte_perm(p1.x, p1.y, 0x7531);
      o0.w = __byte_perm(p1.z, p1.w, 0x6420), o1.w = __byte_perm(p1.z, p1.w, 0x7531);
      reinterpret_cast<uint4*>(q + size_t(r0) * dim)[tid] = o0;
      if (r0 + 1 < rows) reinterpret_cast<uint4*>(q + size_t(r0 + 1) * dim)[tid] = o1;
    }
    __syncwarp();  // the group's tile and byte block are rewritten by the next row pair
#pragma unroll
    for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
  }
}

// Wide rows (6144 < K <= 16384) whose chunk count is not a whole number of warps: the same arithmetic with NC chunks of 16
// elements per thread. A thread rotates its
// chunks one after the other, keeps the rotated bf16 pairs of all of them (16 words per chunk), and quantizes them
// after the single block-wide maximum. Chunk k of thread t is chunk k * blockDim.x + t of the row, so a rotation
// group is still 16 neighbouring threads.
constexpr int wide_max_threads(int nc) { return nc == 2 ? 384 : (nc == 3 ? 320 : 256); }  // two CTAs per SM each

template <int NC>
__global__ void __launch_bounds__(wide_max_threads(NC), 2)
quantize_int8_pairs_wide_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q, float* __restrict__ row_scale,
                                int rows, int dim) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nwarps = blockDim.x >> 5;
  f2* tile = reinterpret_cast<f2*>(smem) + (tid >> 4) * kGroupTile;
  uint8_t* bytes = smem + size_t(blockDim.x >> 4) * kGroupTile * 8 + (tid >> 4) * kGroupBytesOut;
  uint32_t* partial = reinterpret_cast<uint32_t*>(smem + size_t(blockDim.x >> 4) * (kGroupTile * 8 + kGroupBytesOut));
  const int T = tid & 15;
  const int pairs = (rows + 1) >> 1;
  const f2 sixteenth = pk(0.0625f, 0.0625f);

  for (int pair = blockIdx.x, iter = 0; pair < pairs; pair += gridDim.x, ++iter) {
    const int r0 = 2 * pair;
    const bool two = r0 + 1 < rows;
    const uint4* s0 = reinterpret_cast<const uint4*>(x + size_t(r0) * dim);
    const uint4* s1 = reinterpret_cast<const uint4*>(x + size_t(two ? r0 + 1 : r0) * dim);
    auto load = [&](int k, uint4 (&r)[4]) {
      const int c = k * blockDim.x + tid;
      r[0] = __ldg(s0 + 2 * c);
      r[1] = __ldg(s0 + 2 * c + 1);
      r[2] = two ? __ldg(s1 + 2 * c) : make_uint4(0, 0, 0, 0);
      r[3] = two ? __ldg(s1 + 2 * c + 1) : make_uint4(0, 0, 0, 0);
    };
    uint4 raw[2][4];  // this chunk's 64 bytes and the next chunk's, already in flight
    load(0, raw[0]);
    uint32_t w[NC][16];
    uint32_t amax = 0;
#pragma unroll
    for (int k = 0; k < NC; ++k) {
      if (k + 1 < NC) load(k + 1, raw[(k + 1) & 1]);
      f2 v[16];
      const uint4(&rk)[4] = raw[k & 1];
      const uint32_t a[8] = {rk[0].x, rk[0].y, rk[0].z, rk[0].w, rk[1].x, rk[1].y, rk[1].z, rk[1].w};
      const uint32_t b[8] = {rk[2].x, rk[2].y, rk[2].z, rk[2].w, rk[3].x, rk[3].y, rk[3].z, rk[3].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[2 * i] = pku(a[i] << 16, b[i] << 16);
        v[2 * i + 1] = pku(a[i] & 0xFFFF0000u, b[i] & 0xFFFF0000u);
      }
      two_stages(v);
#pragma unroll
      for (int e = 0; e < 16; ++e) tile[17 * T + e] = v[e];
      __syncwarp();
#pragma unroll
      for (int t = 0; t < 16; ++t) v[t] = tile[17 * t + T];
      __syncwarp();  // the tile is rewritten by the next chunk
      two_stages(v);
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        float lo, hi;
        upk(mul2(v[t], sixteenth), lo, hi);
        w[k][t] = to_bf16x2(lo, hi);
        amax = max_bf16x2(amax, w[k][t] & 0x7FFF7FFFu);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = max_bf16x2(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    uint32_t* part = partial + (iter & 1) * 32;
    if (lane == 0) part[warp] = amax;
    __syncthreads();
    uint32_t m = 0;
    for (int i = 0; i < nwarps; ++i) m = max_bf16x2(m, part[i]);
    const float scale0 = fmaxf(div127(__uint_as_float(m << 16)), 1e-30f);
    const float scale1 = fmaxf(div127(__uint_as_float(m & 0xFFFF0000u)), 1e-30f);
    if (tid == 0) {
      row_scale[r0] = scale0;
      if (two) row_scale[r0 + 1] = scale1;
    }
    const float d0 = __bfloat162float(__float2bfloat16(scale0)), d1 = __bfloat162float(__float2bfloat16(scale1));
    const f2 rcp = pk(__frcp_rn(d0), __frcp_rn(d1));
#pragma unroll
    for (int k = 0; k < NC; ++k) {
#pragma unroll
      for (int t = 0; t < 16; ++t) {
        const f2 xv = pku(w[k][t] << 16, w[k][t] & 0xFFFF0000u);
        const f2 qv = mul2(xv, rcp);
        float lo, hi;
        upk(qv, lo, hi);
        const uint32_t qb = to_bf16x2(lo, hi);
        const int i0 = __float2int_rn(__uint_as_float(qb << 16));
        const int i1 = __float2int_rn(__uint_as_float(qb & 0xFFFF0000u));
        uint32_t both;
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(both) : "r"(i1), "r"(i0), "r"(0));
        reinterpret_cast<uint16_t*>(bytes)[16 * t + T] = uint16_t(both);
      }
      __syncwarp();
      const uint4 p0 = reinterpret_cast<const uint4*>(bytes)[2 * T], p1 = reinterpret_cast<const uint4*>(bytes)[2 * T + 1];
      __syncwarp();  // the byte block is rewritten by the next chunk
      uint4 o0, o1;
      o0.x = __byte_perm(p0.x, p0.y, 0x6420), o1.x = __byte_perm(p0.x, p0.y, 0x7531);
      o0.y = __byte_perm(p0.z, p0.w, 0x6420), o1.y = __byte_perm(p0.z, p0.w, 0x7531);
      o0.z = __byte_perm(p1.x, p1.y, 0x6420), o1.z = __byte_perm(p1.x, p1.y, 0x7531);
      o0.w = __byte_perm(p1.z, p1.w, 0x6420), o1.w = __byte_perm(p1.z, p1.w, 0x7531);
      const int c = k * blockDim.x + tid;
      reinterpret_cast<uint4*>(q + size_t(r0) * dim)[c] = o0;
      if (two) reinterpret_cast<uint4*>(q + size_t(r0 + 1) * dim)[c] = o1;
    }
  }
}

template <int NC>
void launch_pairs_wide(const __nv_bfloat16* x, int8_t* q, float* row_scale, int rows, int dim, int threads, cudaStream_t stream) {
  const size_t smem = size_t(threads / 16) * (kGroupTile * 8 + kGroupBytesOut) + 2 * 32 * sizeof(uint32_t);
  reserve_dynamic_smem(reinterpret_cast<const void*>(&quantize_int8_pairs_wide_kernel<NC>), smem, "quantize_int8_token");
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_int8_pairs_wide_kernel<NC>, threads, smem) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const int grid = std::min((rows + 1) / 2, per_sm * device_sm_count());
  quantize_int8_pairs_wide_kernel<NC><<<grid, threads, smem, stream>>>(x, q, row_scale, rows, dim);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("quantize_int8_token: ") + cudaGetErrorString(e));
}

template <int MAXT, int MINB>
void launch_pairs(const __nv_bfloat16* x, int8_t* q, float* row_scale, int rows, int dim, int threads, cudaStream_t stream) {
  const size_t smem = size_t(threads / 16) * (kGroupTile * 8 + kGroupBytesOut) + 2 * 32 * sizeof(uint32_t);
  reserve_dynamic_smem(reinterpret_cast<const void*>(&quantize_int8_pairs_kernel<MAXT, MINB>), smem, "quantize_int8_token");
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, quantize_int8_pairs_kernel<MAXT, MINB>, threads, smem) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  const int grid = std::min((rows + 1) / 2, per_sm * device_sm_count());
  quantize_int8_pairs_kernel<MAXT, MINB><<<grid, threads, smem, stream>>>(x, q, row_scale, rows, dim);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) throw std::runtime_error(std::string("quantize_int8_token: ") + cudaGetErrorString(e));
}

}  // namespace

bool quantize_int8_rot_pairs(const __nv_bfloat16* x, int8_t* q, float* row_scale, int rows, int dim, cudaStream_t stream) {
  if (dim % 256 != 0 || rows <= 0) return false;
  if (reinterpret_cast<uintptr_t>(x) % 16 != 0 || reinterpret_cast<uintptr_t>(q) % 16 != 0) return false;
  if (dim > 6144 && dim / 16 <= 1024 && (dim / 16) % 32 == 0) {
    // One chunk per thread in ONE large CTA per SM (864 threads at K = 13824): 3.2 TB/s against 2.9 for the form below with
    // three chunks per thread in two CTAs of 288, whose rotated values of all chunks stay in registers across the barrier.
    launch_pairs<1024, 1>(x, q, row_scale, rows, dim, dim / 16, stream);
    return true;
  }
  if (dim > 6144) {
    // NC chunks per thread; every thread must own whole chunks and a warp whole rotation groups
    const int chunks = dim / 16;
    for (int nc = 2; nc <= 4; ++nc) {
      if (chunks % nc != 0 || (chunks / nc) % 32 != 0 || chunks / nc > wide_max_threads(nc)) continue;
      if (nc == 2) launch_pairs_wide<2>(x, q, row_scale, rows, dim, chunks / nc, stream);
      if (nc == 3) launch_pairs_wide<3>(x, q, row_scale, rows, dim, chunks / nc, stream);
      if (nc == 4) launch_pairs_wide<4>(x, q, row_scale, rows, dim, chunks / nc, stream);
      return true;
    }
    return false;  // the one-row kernel takes it
  }
  const int threads = ((dim / 16 + 31) / 32) * 32;
  if (threads <= 320)
    launch_pairs<320, 3>(x, q, row_scale, rows, dim, threads, stream);
  else
    launch_pairs<384, 2>(x, q, row_scale, rows, dim, threads, stream);
  return true;
}

}  // namespace sfq
