// Pieces shared by the one-CTA (gemm_tc.cu) and CTA-pair (gemm_tc2.cu) tcgen05 GEMM kernels: tile constants,
// the barrier block in shared memory, bounded waits, the epilogue arithmetic and store path, and the host-side
// tensor-map encoding. Everything here has internal linkage; each kernel file includes it once.
#pragma once

#include <cuda_bf16.h>

#include <mutex>
#include <stdexcept>
#include <string>

#include "gemm_tc.cuh"
#include "ptx.cuh"
#include "runtime.h"

namespace sfq {
namespace {

using namespace ptx;

constexpr int kBM = 128;             // rows of a tile = TMEM lanes
constexpr int kSlabBytes = 128;      // bytes of K per row per stage (one swizzle atom)
constexpr int kMmaKBytes = 32;       // bytes of K one tcgen05.mma consumes, every kind
constexpr int kThreads = 512;        // warpgroups: {producer, MMA, 2 idle}, 2 x epilogue, scale copies (nvfp4)
constexpr int kRegsLean = 56;        // per-thread registers of the single-lane warpgroups after setmaxnreg.dec
constexpr int kRegsEpilogue = 200;   // 2*128*56 + 256*200 = 65536 = the CTA's allocation at 128 registers x 512
constexpr long long kWaitCycles = 2000000000ll;  // ~1 s: far above any legitimate wait

enum Kind { kI8 = 0, kNvfp4 = 1, kBf16 = 2 };

struct Shared {  // lives after the stage ring
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t sf_full[8];   // one-CTA nvfp4: the scale factors of stage s are in TMEM slot s; pair kernel with W4 expansion: the int8 rows of stage s are written
  uint64_t w4_full[8];   // pair kernel with W4 expansion: this CTA's nibbles of stage s have landed
  uint32_t tmem_base;
  volatile int abort;
  long long wait_cycles;  // limit of every bounded wait of this launch
  alignas(16) float col_scale[2][256];  // per-column epilogue operands of the tile being drained
  alignas(16) float bias[2][256];
};

// Bounded wait. Returns false when the CTA is aborting.
__device__ __forceinline__ bool wait_barrier(uint32_t bar, uint32_t parity, Shared* sh, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock_now();
  for (;;) {
    for (int i = 0; i < 64; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (sh->abort) return false;
    if (clock_now() - start > sh->wait_cycles) {
      atomicCAS(status, 0, code);
      sh->abort = 1;
      return false;
    }
  }
}

// The same for a converged warp: every lane polls, the verdict is made uniform by a vote.
__device__ __forceinline__ bool wait_barrier_warp(uint32_t bar, uint32_t parity, Shared* sh, int* status, int code) {
  return __all_sync(0xffffffffu, wait_barrier(bar, parity, sh, status, code));
}

__device__ __forceinline__ float gelu_tanh_ref(float v) {
  // 0.5 v (1 + tanh(k (v + 0.044715 v^3))), evaluated in the association order of
  // gelu_tanh_kernel (src/cuda/nn_pointwise.cu:74-81) so the bits agree.
  constexpr float k = 0.7978845608028654f;
  return 0.5f * v * (1.0f + tanhf(k * (v + 0.044715f * v * v * v)));
}

// out = silu(gate) * up on bf16 inputs, fast exponential and IEEE division as in swiglu_kernel
// (src/cuda/nn_pointwise.cu:44-64): 32 columns of one row, gate and up already rounded like a stored GEMM output.
__device__ __forceinline__ void swiglu_chunk(const uint4 (&gate)[4], const uint4 (&up)[4], uint4 (&out)[4]) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gate[v]);
    const __nv_bfloat162* up2 = reinterpret_cast<const __nv_bfloat162*>(&up[v]);
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&out[v]);
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      const float2 g = __bfloat1622float2(gp[h]), u = __bfloat1622float2(up2[h]);
      op[h] = __floats2bfloat162_rn((g.x / (1.0f + __expf(-g.x))) * u.x, (g.y / (1.0f + __expf(-g.y))) * u.y);
    }
  }
}

// Rounding points of the epilogue, as in the reference: the GEMM result is rounded to bf16 (output_bf16 /
// the GEMM's own store), the bias is added to that bf16 value and re-rounded (add_bias_kernel,
// src/cuda/linear_weights.cu:483-491), and GELU runs in place on the bf16 result.

// Epilogue arithmetic for 32 consecutive columns of one row (a thread owns a ROW in TMEM): scale, round to
// bf16, [add bias, re-round], [GELU, re-round]; the result stays in registers as four 16-byte units.
// `cs`/`bs` point at this chunk's column operands in shared memory (broadcast reads). The rounding points
// are those of `finish`.
template <int KIND, bool BIAS, bool GELU>
__device__ __forceinline__ void pack_chunk(const uint32_t (&r)[32], float rs, const float* cs, const float* bs,
                                           uint4 (&out)[4]) {
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const float4 c0 = *reinterpret_cast<const float4*>(cs + v * 8), c1 = *reinterpret_cast<const float4*>(cs + v * 8 + 4);
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    float b[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if constexpr (BIAS) {
      const float4 b0 = *reinterpret_cast<const float4*>(bs + v * 8), b1 = *reinterpret_cast<const float4*>(bs + v * 8 + 4);
      b[0] = b0.x, b[1] = b0.y, b[2] = b0.z, b[3] = b0.w, b[4] = b1.x, b[5] = b1.y, b[6] = b1.z, b[7] = b1.w;
    }
    __nv_bfloat162* pp = reinterpret_cast<__nv_bfloat162*>(&out[v]);
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      float lo, hi;
      if constexpr (KIND == kI8) {
        lo = (float(int32_t(r[v * 8 + 2 * h])) * rs) * c[2 * h];
        hi = (float(int32_t(r[v * 8 + 2 * h + 1])) * rs) * c[2 * h + 1];
      } else if constexpr (KIND == kNvfp4) {
        lo = __uint_as_float(r[v * 8 + 2 * h]) * c[2 * h];
        hi = __uint_as_float(r[v * 8 + 2 * h + 1]) * c[2 * h + 1];
      } else {
        lo = __uint_as_float(r[v * 8 + 2 * h]);
        hi = __uint_as_float(r[v * 8 + 2 * h + 1]);
      }
      __nv_bfloat162 o = __floats2bfloat162_rn(lo, hi);  // the GEMM's own bf16 store
      if constexpr (BIAS) {
        const float2 f = __bfloat1622float2(o);
        o = __floats2bfloat162_rn(f.x + b[2 * h], f.y + b[2 * h + 1]);  // add_bias re-rounds
      }
      if constexpr (GELU) {
        const float2 f = __bfloat1622float2(o);
        o = __floats2bfloat162_rn(gelu_tanh_ref(f.x), gelu_tanh_ref(f.y));
      }
      pp[h] = o;
    }
  }
}

// Writes one warp's 32 rows x 32 bf16 columns. Storing straight from registers would scatter every store
// instruction over 32 rows, so the block goes through a 2 KB shared-memory transpose (16-byte units
// XOR-swizzled with the row, both phases bank-conflict free) and each instruction then writes 64 contiguous
// bytes of 8 rows. `dst` = global address of (first row of the warp, first column of the chunk).
__device__ __forceinline__ void flush_chunk(const uint4 (&packed)[4], uint4* stage, __nv_bfloat16* dst, size_t ldy,
                                            int rows_ok, int lane, const float* gate = nullptr, size_t gate_ld = 0,
                                            const int (&gate_idx)[4] = {0, 0, 0, 0}) {
#pragma unroll
  for (int v = 0; v < 4; ++v) stage[lane * 4 + (v ^ ((lane >> 1) & 3))] = packed[v];
  __syncwarp();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = 8 * i + (lane >> 2), unit = lane & 3;
    uint4 val = stage[row * 4 + (unit ^ ((row >> 1) & 3))];
    if (row < rows_ok) {
      uint4* out = reinterpret_cast<uint4*>(dst + size_t(row) * ldy + unit * 8);
      if (gate != nullptr) {  // `gate` already points at this chunk's first column
        // gated residual, y = bf16(fma(gate, branch, y)) with the branch rounded to bf16 first: the arithmetic of
        // add_gated_kernel (src/cuda/nn_pointwise.cu:16-37) on the value this GEMM would have stored
        const uint4 cur = *out;
        const float4* gp = reinterpret_cast<const float4*>(gate + size_t(gate_idx[i]) * gate_ld + unit * 8);
        const float4 g0 = __ldg(gp), g1 = __ldg(gp + 1);
        const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        const __nv_bfloat162* bp = reinterpret_cast<const __nv_bfloat162*>(&val);
        const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&cur);
        uint4 res;
        __nv_bfloat162* rp = reinterpret_cast<__nv_bfloat162*>(&res);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          const float2 b = __bfloat1622float2(bp[h]), x = __bfloat1622float2(xp[h]);
          rp[h] = __floats2bfloat162_rn(__fmaf_rn(gg[2 * h], b.x, x.x), __fmaf_rn(gg[2 * h + 1], b.y, x.y));
        }
        val = res;
        *out = val;
      } else {
        // A plain output tile is written once and not read again by this kernel: store it with the streaming (evict-first)
        // policy, so that the gigabytes of y that pass through L2 do not push out the weight and activation slabs the
        // other tiles are about to re-read (measured at 27900 x 5120 -> 13824: 618 MB of DRAM reads for 120 MB of operands).
        __stcs(out, val);
      }
    }
  }
  __syncwarp();  // the block is reused by the next chunk
}

// The gate-table rows of the four output rows a lane meets in flush_chunk (rows 8 i + lane / 4 of its warp's 32).
__device__ __forceinline__ void gate_rows_for(const GemmArgs& g, int warp_row0, int lane, int (&idx)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = warp_row0 + 8 * i + (lane >> 2);
    idx[i] = (g.gate != nullptr && r < g.M) ? __ldg(g.gate_index + r) : 0;
  }
}

// ------------------------------------------------------------------ host side

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr)
      throw std::runtime_error("sfq: cuTensorMapEncodeTiled is not available from this driver");
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

// A [rows, row_bytes] byte matrix, boxes of {128 bytes, box_rows}, 128-byte swizzle, zero fill outside.
CUtensorMap make_map(const void* base, size_t rows, size_t row_bytes, int box_rows) {
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0 || row_bytes % 16 != 0)
    throw std::invalid_argument("sfq gemm: operand base and row pitch must be 16-byte aligned for TMA");
  CUtensorMap m;
  const cuuint64_t dims[2] = {row_bytes, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {kSlabBytes, cuuint32_t(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("sfq gemm: cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return m;
}

int sm_count() { return device_sm_count(); }

}  // namespace
}  // namespace sfq
