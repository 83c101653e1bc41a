// Host launchers of the non-GEMM kernels (unpack.cu, act_quant.cu, pointwise.cu).
// Every launcher validates before launching and throws std::invalid_argument /
// std::runtime_error on a contract violation, like the reference's launchers.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "../../include/sfq.h"

namespace sfq {

// ---- unpack.cu
void unpack_nvfp4_bf16(const uint8_t* data, const uint8_t* scale_tiled, float global, __nv_bfloat16* out,
                       int out_features, int in_features, cudaStream_t stream);
void unpack_w4a8_int8(const int8_t* packed, const uint8_t* group_scale, const float* codebook, int8_t* out,
                      int out_features, int in_features, int group, cudaStream_t stream);
void unpack_w6a8_int8(const int8_t* packed, const uint8_t* group_scale, int8_t* out, int out_features,
                      int in_features, int group, cudaStream_t stream);
void unpack_int8_bf16(const int8_t* codes, const float* scale, __nv_bfloat16* out, int out_features, int in_features,
                      cudaStream_t stream);
void unpack_int8_f16(const int8_t* codes, const float* scale, __half* out, int out_features, int in_features,
                     int rotation_group, int canonicalize_subnormals, cudaStream_t stream);

void unpack_f8e4m3_bf16(const uint8_t* src, const float* scale, __nv_bfloat16* dst, size_t n, cudaStream_t stream);
void unpack_nf4_bf16(const uint8_t* src, const uint8_t* absmax, const float* map, const float* nested_map,
                     const float* nested_absmax, int block, int nested_block, float offset, __nv_bfloat16* dst,
                     int out_features, int in_features, cudaStream_t stream);
void unpack_nf4_f16(const uint8_t* src, const uint8_t* absmax, const float* map, const float* nested_map,
                    const float* nested_absmax, int block, int nested_block, float offset, __half* dst, size_t n,
                    cudaStream_t stream);
void convert_f16_bf16(const __half* src, __nv_bfloat16* dst, size_t n, cudaStream_t stream);
void convert_f32_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t stream);

// ---- act_quant.cu
struct NormArgs {  // null weight = stage disabled
  const __nv_bfloat16* weight = nullptr;
  const float* scale = nullptr;  // adaLN tables, fp32 [*, dim]; null = plain RMSNorm
  const float* shift = nullptr;
  const int32_t* index = nullptr;  // a[r]
  float eps = 1e-5f;
};
void rmsnorm(const __nv_bfloat16* x, const NormArgs& norm, __nv_bfloat16* out, int rows, int dim, cudaStream_t stream);
void convrot(const __nv_bfloat16* x, __nv_bfloat16* out, int rows, int dim, int group, cudaStream_t stream);
void quantize_int8_token(const __nv_bfloat16* x, const NormArgs& norm, int8_t* q, float* row_scale,
                         __nv_bfloat16* normed_out, int rows, int dim, bool apply_convrot, cudaStream_t stream);
void quantize_nvfp4_block(const __nv_bfloat16* x, const NormArgs& norm, uint8_t* packed, uint8_t* scales,
                          __nv_bfloat16* normed_out, int rows, int dim, int layout, cudaStream_t stream);
size_t nvfp4_act_scale_bytes(int rows, int dim);

// ---- pointwise.cu
void gelu_tanh(__nv_bfloat16* x, size_t n, cudaStream_t stream);
void swiglu(const __nv_bfloat16* fused, __nv_bfloat16* out, int rows, int inner, cudaStream_t stream);
void pre_quant_scale(const __nv_bfloat16* src, const __nv_bfloat16* scale, __nv_bfloat16* dst, int rows, int dim,
                     cudaStream_t stream);
// The reference's remaining linear-header launchers (thin kernels, off the runner's own path).
void convrot_f32(const float* in, float* out, int rows, int dim, int group, cudaStream_t stream);
void pre_quant_scale_f32(const float* src, const __nv_bfloat16* scale, float* dst, int rows, int dim, cudaStream_t stream);
void int8_output_bf16(const int32_t* acc, const float* row_scale, const float* channel_scale, __nv_bfloat16* out, int rows, int cols,
                      cudaStream_t stream);
void int8_output_f32_inplace(int32_t* io, const float* row_scale, const float* channel_scale, int rows, int cols, cudaStream_t stream);
void quantize_f8e4m3(const __nv_bfloat16* src, float input_scale, uint8_t* dst, size_t n, cudaStream_t stream);
void widen_bf16(const __nv_bfloat16* src, float* dst, size_t n, cudaStream_t stream);
void narrow_to_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t stream);
// fp4 activations from the reference's layout into the GEMM_FEED layout (nibbles exchanged, scales tiled and padded).
void nvfp4_act_to_feed(const uint8_t* xq, const uint8_t* xs, uint8_t* feed_q, uint8_t* feed_scale_tiled, int rows, int dim,
                       cudaStream_t stream);
// quant_int8_pairs.cu: ConvRot-256 + per-token int8 without a norm in front; false when the shape is not covered.
bool quantize_int8_rot_pairs(const __nv_bfloat16* x, int8_t* q, float* row_scale, int rows, int dim, cudaStream_t stream);
void add_gated(__nv_bfloat16* x, const __nv_bfloat16* branch, const float* gate, const int32_t* index, int rows,
               int dim, cudaStream_t stream);

// fp32 Linear on CUDA cores: y[rows,out] = x[rows,in] W^T (+ bias), W fp32 or bf16, bias fp32 or bf16 or null.
void linear_f32(const float* x, const void* w, bool w_is_bf16, const void* bias, bool bias_is_bf16, float* y, int rows, int out_features,
                int in_features, cudaStream_t stream);
// adaLN table expansion, launch_adaln_expand (src/cuda/dit_kernels.cu:108-134): out[param][t][modality][channel].
void adaln_expand(const float* w, const float* bias, const float* code, float* out, int num_t, int num_modality, int num_param,
                  int channels, int rank, cudaStream_t stream);

// Full self-attention, head_dim 128 (attention.cu). q: [seq_q, heads*128] with row pitch ld_q; k, v: [seq_kv, kv_heads*128]
// with row pitch ld_kv; out: [seq_q, heads*128] with row pitch ld_out. scale <= 0 selects 1/sqrt(head_dim). The workspace
// holds V^T (attention_workspace_bytes).
size_t attention_workspace_bytes(int seq_kv, int kv_heads, int head_dim);
void attention_forward(const __nv_bfloat16* q, int ld_q, const __nv_bfloat16* k, const __nv_bfloat16* v, int ld_kv, __nv_bfloat16* out, int ld_out,
                       int seq_q, int seq_kv, int heads, int kv_heads, int head_dim, float scale, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream);

// Head-wise RMSNorm (norm_weight [128], may be null) and MM-RoPE (cos / sin fp32 [rows, 96], may be null) in place on
// x [rows, heads, 128] with a row pitch of ld elements.
void head_norm_rope(__nv_bfloat16* x, int ld, const __nv_bfloat16* norm_weight, const float* cos_tab, const float* sin_tab, int rows,
                    int heads, int head_dim, float eps, cudaStream_t stream);

}  // namespace sfq
