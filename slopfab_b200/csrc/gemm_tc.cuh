// Host interface of the tcgen05 GEMM kernels (gemm_tc.cu).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/sfq.h"

namespace sfq {

struct GemmArgs {
  int M = 0, N = 0, K = 0;        // y[M,N] = A[M,K] * W[N,K]^T, K in elements
  __nv_bfloat16* y = nullptr;     // row-major, leading dimension ldy (elements)
  int ldy = 0;
  // epilogue
  const float* row_scale = nullptr;  // int8: per-token activation scale [M]
  const float* col_scale = nullptr;  // int8: per-output-channel weight scale [N]
  float global_scale = 1.0f;         // nvfp4: second-level weight scale
  const void* bias = nullptr;        // [N] fp32 or bf16, optional
  int bias_is_bf16 = 0;
  int act = SFQ_ACT_NONE;
  // optional gated residual: y[r, c] = bf16(fma(gate[gate_index[r], c], branch[r, c], y[r, c])), branch = what the
  // epilogue would otherwise have stored (launch_add_gated, include/slopfab/cuda/nn_kernels.cuh:64-69)
  const float* gate = nullptr;          // fp32 [*, N]
  const int32_t* gate_index = nullptr;  // int32 [M]
  // nvfp4 block scales, both in the 128x4-tiled layout (512-byte tiles, row tile major)
  const uint8_t* a_scale_tiled = nullptr;
  const uint8_t* w_scale_tiled = nullptr;
  // W4A8 weight expanded inside the CTA-pair int8 kernel (gemm_pair_w4a8): group scales [N, K/16] e4m3 and the codebook
  const uint8_t* w4_gscale = nullptr;
  const float* w4_codebook = nullptr;  // 16 floats, 16-byte aligned
  // bookkeeping
  int* status = nullptr;  // device word; a kernel that gives up waiting stores a non-zero code
  int band_m = 0;         // row tiles per raster band (0 = default)
  int max_ctas = 0;       // 0 = one CTA per SM
  int tile_n = 0;         // 128 or 256 select the one-CTA kernel with that tile width; 0 = default (CTA pairs, 256 x 256)
  int tail_split = -1;    // CTA-pair kernel: trailing tiles cut into two 128-column halves (-1 = let the launcher choose)
  // test hooks (see runtime.h); never set on a runner's path
  int test_drop_iteration = -1;  // the producer skips the loads of this pipeline iteration (bytes still announced)
  long long wait_cycles = 0;     // limit of every bounded wait in clocks; 0 = the default (about a second)
};

// All three throw std::invalid_argument / std::runtime_error before launching on a contract violation.
void gemm_int8(const int8_t* a, const int8_t* w, const GemmArgs& g, cudaStream_t stream);
void gemm_nvfp4(const uint8_t* a_packed, const uint8_t* w_packed, const GemmArgs& g, cudaStream_t stream);
void gemm_bf16(const __nv_bfloat16* a, const __nv_bfloat16* w, const GemmArgs& g, cudaStream_t stream);

// CTA-pair kernels (gemm_tc2.cu), called by the three entry points above when the shape allows. They return false
// without launching when the device cannot co-schedule clusters of two.
bool gemm_pair_int8(const int8_t* a, const int8_t* w, const GemmArgs& g, cudaStream_t stream);
bool gemm_pair_nvfp4(const uint8_t* a_packed, const uint8_t* w_packed, const GemmArgs& g, cudaStream_t stream);
bool gemm_pair_bf16(const __nv_bfloat16* a, const __nv_bfloat16* w, const GemmArgs& g, cudaStream_t stream);
// y = epilogue(int32(q * W^T)) with W given as W4A8 nibbles [N, K/2] + e4m3 group scales [N, K/16] (g.w4_gscale) + codebook
// (g.w4_codebook): the int8 rows are produced in shared memory inside the kernel, stage by stage, instead of by
// unpack_w4a8_int8 into a dense [N, K] copy. Same int32 accumulators, hence the same output bits. Needs K % 128 == 0 and the
// plain epilogue (bias / GELU allowed, no gate, no SwiGLU); returns false without launching when that or the device does not fit.
bool gemm_pair_w4a8(const int8_t* a, const uint8_t* w_packed, const GemmArgs& g, cudaStream_t stream);

}  // namespace sfq
