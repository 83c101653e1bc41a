/* sfq -- C ABI of the B200 quantized-Linear library (libsfq.so).
 *
 * Drop-in boundary for the quantized Linear of slopfab's DiT: weight packing and
 * unpacking (NVFP4, W4A8, W6A8, INT8), the fused norm + activation quantizer, the
 * tcgen05 GEMMs with their fused epilogue, and the LinearRunner dispatch above
 * them. Each entry point names the reference interface it replaces (paths are
 * relative to the reference project root).
 *
 * Conventions (modelled on include/slopfab/capi.h:172-200 and
 * src/capi/internal.h:54-130 of the reference):
 *   - every function returns an int status: SFQ_OK, or a negative code; the text
 *     of the failure is available from sfq_last_error() on the calling thread;
 *     no C++ exception crosses this boundary;
 *   - pointers named d_* are device pointers, h_* are host pointers; nothing is
 *     owned by the library except an opaque runner handle;
 *   - `stream` is a cudaStream_t passed as void*; every device entry point only
 *     enqueues work on it and never synchronises;
 *   - weights are [out_features, in_features] row-major, contraction over the
 *     second axis, never transposed (include/slopfab/cuda/linear.cuh:18-20).
 *
 * There is no CPU fallback: without a CUDA device every device entry point fails
 * with SFQ_ERR_RUNTIME.
 */
#ifndef SFQ_H_
#define SFQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define SFQ_API __declspec(dllexport)
#else
#define SFQ_API __attribute__((visibility("default")))
#endif

enum {
  SFQ_OK = 0,
  SFQ_ERR_INVALID_ARGUMENT = -1, /* std::invalid_argument in the reference */
  SFQ_ERR_RUNTIME = -2,          /* std::runtime_error / cuda::Error in the reference */
  SFQ_ERR_OUT_OF_MEMORY = -3,    /* workspace exhausted or cudaErrorMemoryAllocation */
  SFQ_ERR_DEVICE_TIMEOUT = -4    /* a kernel gave up a bounded wait; see sfq_device_status */
};

/* QuantFormat, include/slopfab/cuda/linear.cuh:49-59 (same order, same values). */
typedef enum {
  SFQ_F32 = 0, SFQ_F16 = 1, SFQ_BF16 = 2, SFQ_F8E4M3 = 3, SFQ_I8 = 4,
  SFQ_NVFP4 = 5, SFQ_NF4 = 6, SFQ_W4A8 = 7, SFQ_W6A8 = 8
} sfq_format;

/* ComputeType, include/slopfab/cuda/linear.cuh:73-76. */
typedef enum { SFQ_COMPUTE_BF16 = 0, SFQ_COMPUTE_F32 = 1 } sfq_compute;

/* Fused activation of the GEMM epilogue. GELU-tanh is the arithmetic of
 * launch_gelu_tanh (src/cuda/nn_pointwise.cu:74-81) applied to the bf16 result. */
/* SFQ_ACT_SWIGLU: the weight's N rows are [gate (N/2) | up (N/2)] as in the reference's fused mlp.fc1, and the output has
 * N/2 columns: y[r, i] = bf16(silu(g) * u) with g, u the bf16 values a plain epilogue would have stored at columns i and
 * N/2 + i (launch_swiglu, include/slopfab/cuda/nn_kernels.cuh; swiglu_kernel, src/cuda/nn_pointwise.cu:44-64). Needs
 * N % 256 == 0; not combined with the gated residual. */
typedef enum { SFQ_ACT_NONE = 0, SFQ_ACT_GELU_TANH = 1, SFQ_ACT_SWIGLU = 2 } sfq_activation;

/* Layout of quantized NVFP4 activations.
 * REFERENCE: low nibble = even element, scales row-major [rows, dim/16]
 *   (launch_quantize_nvfp4_activations, include/slopfab/cuda/nvfp4_gemm.cuh:77-82).
 * GEMM_FEED: high nibble = even element (the weight file's convention, so no nibble
 *   swap is needed on either operand) and scales in the 128x4-tiled layout of the
 *   weight scales, rows padded to a multiple of 128. */
typedef enum { SFQ_NVFP4_ACT_REFERENCE = 0, SFQ_NVFP4_ACT_GEMM_FEED = 1 } sfq_nvfp4_act_layout;

/* QuantWeight, include/slopfab/cuda/linear.cuh:80-152: same fields, same defaults
 * (use sfq_quant_weight_init). Owns nothing. */
typedef struct sfq_quant_weight {
  int32_t format;              /* sfq_format */
  const void* data;            /* device */
  int32_t out_features;
  int32_t in_features;
  const float* weight_scale;   /* device; 1 element, or out_features when per_channel_scale */
  int32_t per_channel_scale;
  float input_scale;
  int32_t full_precision;
  const uint8_t* block_scale;  /* device; NVFP4: 128x4-tiled e4m3; W4A8/W6A8: row-major e4m3 groups */
  uint32_t packed_group_size;  /* W4A8: 16; W6A8: multiple of 16 */
  const float* w4_codebook;    /* device, 16 entries, W4A8 only */
  float global_scale;          /* NVFP4 .weight_scale_2 */
  const void* pre_quant_scale; /* device bf16 [in_features], AWQ; must be null on the native paths */
  const uint8_t* nf4_absmax;
  const float* nf4_quant_map;
  const float* nf4_nested_quant_map;
  const float* nf4_nested_absmax;
  int32_t nf4_block_size;
  int32_t nf4_nested_block_size;
  float nf4_nested_offset;
  int32_t convrot;
  int32_t convrot_group;
  const void* bias;            /* device, out_features elements, optional */
  int32_t bias_format;         /* SFQ_F32 or SFQ_BF16 */
} sfq_quant_weight;

/* Epilogue of the stand-alone GEMM entry points. */
typedef struct sfq_epilogue {
  const float* d_row_scale;    /* int8: per-token activation scale [M] */
  const float* d_col_scale;    /* int8: per-output-channel weight scale [N] */
  float global_scale;          /* nvfp4: multiplies the accumulator once */
  const void* d_bias;          /* optional [N] */
  int32_t bias_format;         /* SFQ_F32 or SFQ_BF16 */
  int32_t activation;          /* sfq_activation */
  /* Optional gated residual (launch_add_gated, include/slopfab/cuda/nn_kernels.cuh:64-69) fused behind bias and
   * activation: when d_gate is non-null the output buffer is read-modify-written,
   * y[r, c] = bf16(fma(d_gate[d_gate_index[r] * N + c], branch[r, c], y[r, c])), branch = the bf16 value the
   * epilogue would have stored. Both null: plain store. */
  const float* d_gate;         /* fp32 [*, N] */
  const int32_t* d_gate_index; /* int32 [M] */
} sfq_epilogue;

/* Optional RMSNorm / adaLN-modulate stage fused in front of a quantizer.
 * out = (x * rsqrt(mean(x^2) + eps)) * w, then fma(out, 1 + scale[a[r]], shift[a[r]])
 * when d_scale is non-null (launch_rmsnorm / launch_rmsnorm_modulate,
 * include/slopfab/cuda/nn_kernels.cuh:28-57; tables are fp32 [*, dim], a[r] int32).
 * A null d_norm_weight disables the stage. */
typedef struct sfq_norm {
  const void* d_norm_weight;   /* bf16 [dim] */
  const float* d_scale;
  const float* d_shift;
  const int32_t* d_adaln_index;
  float eps;
} sfq_norm;

typedef struct sfq_runner sfq_runner;

SFQ_API const char* sfq_last_error(void);
SFQ_API int sfq_version(void);
SFQ_API void sfq_quant_weight_init(sfq_quant_weight* w);

/* Reads and clears the device status word of the current device: 0, or the code a
 * kernel stored when it abandoned a bounded wait. Synchronises the device. */
SFQ_API int sfq_device_status(int* h_code);

/* ---- host packers -------------------------------------------------------- */

/* fp32 [out,in] -> NVFP4 storage: data u8 [out,in/2] (even element in the high
 * nibble), scale u8 [out*in/16] in the 128x4-tiled layout, with the caller's
 * global scale. Byte-identical to the reference's fixture packer pack_nvfp4
 * (tests/detail/nn_weight_fixture.h:333-360). Needs out % 128 == 0, in % 64 == 0. */
SFQ_API int sfq_pack_nvfp4(const float* h_w, int out_features, int in_features, float global_scale,
                           uint8_t* h_data, uint8_t* h_scale_tiled);

/* fp32 [out,in] -> W4A8 storage of docs/w4a8.md: ConvRot-256 along in_features,
 * int4 codes low-nibble-first [out,in/2], E4M3 group scales [out,in/16] row-major,
 * fp32 channel scales [out], and the 16-entry codebook (i - 8). The reference
 * ships no encoder for this format (its files come from a third-party tool), so the
 * rule is this library's; the bytes satisfy validate_packed_int8_weight
 * (src/core/w4a8.cpp:127-162) and decode through launch_dequant_w4a8_weight. */
SFQ_API int sfq_pack_w4a8(const float* h_w, int out_features, int in_features, int8_t* h_packed,
                          uint8_t* h_group_scale, float* h_channel_scale, float* h_codebook16);

/* fp32 [out,in] -> W6A8 storage of docs/w6a8.md: per row in/2 low-nibble bytes then
 * in/4 bytes of 2-bit highs, levels code-32, E4M3 group scales [out,in/group]. */
SFQ_API int sfq_pack_w6a8(const float* h_w, int out_features, int in_features, int group,
                          int8_t* h_packed, uint8_t* h_group_scale, float* h_channel_scale);

/* fp32 [out,in] -> INT8 weight-only ("int8_tensorwise" with per-row scales,
 * src/core/int8_weight.cpp:11-64): optional ConvRot with group in {4,16,64,256}
 * (0 = none; skipped when in % group != 0), codes [out,in], scales [out]. */
SFQ_API int sfq_pack_int8(const float* h_w, int out_features, int in_features, int convrot_group,
                          int8_t* h_codes, float* h_scale);

/* ---- device unpackers ---------------------------------------------------- */

/* launch_dequant_nvfp4, include/slopfab/cuda/linear.cuh:289-291 (bit-exact). */
SFQ_API int sfq_unpack_nvfp4_bf16(const uint8_t* d_data, const uint8_t* d_scale_tiled, float global_scale,
                                  void* d_out_bf16, int out_features, int in_features, void* stream);
/* launch_dequant_w4a8_weight, include/slopfab/cuda/w4a8.cuh:18-20 (bit-exact). */
SFQ_API int sfq_unpack_w4a8_int8(const int8_t* d_packed, const uint8_t* d_group_scale, const float* d_codebook,
                                 int8_t* d_out, int out_features, int in_features, int group, void* stream);
/* launch_dequant_w6a8_weight, include/slopfab/cuda/w4a8.cuh:12-14 (bit-exact). */
SFQ_API int sfq_unpack_w6a8_int8(const int8_t* d_packed, const uint8_t* d_group_scale, int8_t* d_out,
                                 int out_features, int in_features, int group, void* stream);
/* launch_dequant_i8_per_channel, include/slopfab/cuda/linear.cuh:264-265 (bit-exact). */
SFQ_API int sfq_unpack_int8_bf16(const int8_t* d_codes, const float* d_scale, void* d_out_bf16,
                                 int out_features, int in_features, void* stream);
/* launch_dequant_f8e4m3, include/slopfab/cuda/linear.cuh:259-260: bf16(e4m3(v) * *d_scale), one device
 * scalar scale (bit-exact). */
SFQ_API int sfq_unpack_f8e4m3_bf16(const uint8_t* d_codes, const float* d_scale, void* d_out_bf16, size_t n,
                                   void* stream);
/* launch_dequant_nf4, include/slopfab/cuda/linear.cuh:293-296: bitsandbytes NF4 with double-quantized
 * block scales, high nibble = even element (bit-exact). */
SFQ_API int sfq_unpack_nf4_bf16(const uint8_t* d_packed, const uint8_t* d_absmax, const float* d_quant_map,
                                const float* d_nested_quant_map, const float* d_nested_absmax, int block_size,
                                int nested_block_size, float nested_offset, void* d_out_bf16, int out_features,
                                int in_features, void* stream);
/* launch_dequant_nf4_f16, include/slopfab/cuda/linear.cuh:298-301: the same decode into fp16 over a flat element
 * count (bit-exact). */
SFQ_API int sfq_unpack_nf4_f16(const uint8_t* d_packed, const uint8_t* d_absmax, const float* d_quant_map,
                               const float* d_nested_quant_map, const float* d_nested_absmax, int block_size,
                               int nested_block_size, float nested_offset, void* d_out_f16, size_t n, void* stream);
/* launch_pre_quant_scale, include/slopfab/cuda/linear.cuh:305-306: the AWQ activation pre-scale
 * dst[r, i] = bf16(src[r, i] * scale[i]) (bit-exact). */
SFQ_API int sfq_pre_quant_scale(const void* d_src_bf16, const void* d_scale_bf16, void* d_dst_bf16, int rows, int dim,
                                void* stream);
/* F16Weight::materialize for INT8 ConvRot weights (src/cuda/nf4_weight.cu:20-51; host twin
 * unpack_int8_weight, src/core/int8_weight.cpp:66-100): inverse rotation into fp16 (bit-exact). */
SFQ_API int sfq_unpack_int8_f16(const int8_t* d_codes, const float* d_scale, void* d_out_f16, int out_features,
                                int in_features, int rotation_group, int canonicalize_subnormals, void* stream);

/* ---- activation side ------------------------------------------------------ */

/* launch_rmsnorm / launch_rmsnorm_modulate, include/slopfab/cuda/nn_kernels.cuh:28-57 (bit-exact for dim % 8 == 0). */
SFQ_API int sfq_rmsnorm(const void* d_x_bf16, const sfq_norm* norm, void* d_out_bf16, int rows, int dim, void* stream);
/* launch_convrot, include/slopfab/cuda/linear.cuh:251-252 (bit-exact). */
SFQ_API int sfq_convrot(const void* d_x_bf16, void* d_out_bf16, int rows, int dim, int group, void* stream);

/* launch_convrot_f32, include/slopfab/cuda/linear.cuh:253-254: the same rotation over fp32 rows (bit-exact). */
SFQ_API int sfq_convrot_f32(const float* d_x, float* d_out, int rows, int dim, int group, void* stream);
/* launch_w4a8_output_bf16 and launch_dequant_w4a8_output, include/slopfab/cuda/w4a8.cuh:30-36: an int32 accumulator
 * [rows, cols] scaled by row and channel scales into bf16, or into fp32 over the accumulator itself (bit-exact). The
 * runner never uses them: sfq_gemm_int8 applies the same arithmetic in its epilogue. */
SFQ_API int sfq_int8_output_bf16(const int32_t* d_acc, const float* d_row_scale, const float* d_channel_scale,
                                 void* d_y_bf16, int rows, int cols, void* stream);
SFQ_API int sfq_int8_output_f32(int32_t* d_acc_inout, const float* d_row_scale, const float* d_channel_scale, int rows,
                                int cols, void* stream);
/* launch_quantize_f8e4m3, include/slopfab/cuda/linear.cuh:308-310: e4m3(x / input_scale), saturating (bit-exact). */
SFQ_API int sfq_quantize_f8e4m3(const void* d_x_bf16, float input_scale, uint8_t* d_out, size_t n, void* stream);

/* One pass: [RMSNorm / modulate] -> ConvRot-256 -> per-token int8. Replaces
 * launch_rmsnorm_modulate + launch_convrot + launch_quantize_w4a8_bf16
 * (src/dit/transformer_execution.cpp:260; src/cuda/linear.cu:199-200) with identical
 * bits: q int8 [rows,dim], row scales fp32 [rows]. dim % 256 == 0. `norm` may be null.
 * `d_normed_out_bf16`, when non-null, also receives the normed activation. */
SFQ_API int sfq_quantize_int8_token(const void* d_x_bf16, const sfq_norm* norm, int8_t* d_q, float* d_row_scale,
                                    void* d_normed_out_bf16, int rows, int dim, int apply_convrot, void* stream);

/* One pass: [RMSNorm / modulate] -> per-16-block fp4. The REFERENCE layout is
 * launch_quantize_nvfp4_activations (src/cuda/nvfp4_gemm.cu:107-158, byte-exact);
 * GEMM_FEED is what sfq_gemm_nvfp4 consumes. dim % 16 == 0 (GEMM_FEED: dim % 64 == 0).
 * GEMM_FEED scale buffer size: sfq_nvfp4_act_scale_bytes(rows, dim). */
SFQ_API int sfq_quantize_nvfp4_block(const void* d_x_bf16, const sfq_norm* norm, uint8_t* d_packed, uint8_t* d_scales,
                                     void* d_normed_out_bf16, int rows, int dim, int layout, void* stream);
SFQ_API size_t sfq_nvfp4_act_scale_bytes(int rows, int dim);

/* launch_gelu_tanh / launch_swiglu / launch_add_gated, include/slopfab/cuda/nn_kernels.cuh:68-88. */
SFQ_API int sfq_gelu_tanh(void* d_x_bf16, size_t n, void* stream);
SFQ_API int sfq_swiglu(const void* d_fused_bf16, void* d_out_bf16, int rows, int inner, void* stream);
SFQ_API int sfq_add_gated(void* d_x_bf16, const void* d_branch_bf16, const float* d_gate, const int32_t* d_adaln_index,
                          int rows, int dim, void* stream);

/* ---- GEMMs ---------------------------------------------------------------- */

/* y[M,N] bf16 = epilogue(int32(q[M,K] * w8[N,K]^T)). Replaces the cuBLAS int8 GemmEx,
 * launch_w4a8_output_bf16 and add_bias of src/cuda/linear.cu:202-206; the int32
 * accumulators and therefore the bf16 output are bit-exact. K % 16 == 0. */
SFQ_API int sfq_gemm_int8(const int8_t* d_q, const int8_t* d_w8, const sfq_epilogue* ep, void* d_y_bf16,
                          int M, int N, int K, void* stream);
/* The same product with the weight still in its W4A8 storage form: nibbles [N, K/2] (element e of a group in nibble e),
 * e4m3 group scales [N, K/16] and the 16-entry codebook. The int8 weight rows are produced in shared memory inside the
 * GEMM, K-slab by K-slab (dequant_weight_kernel's arithmetic, src/cuda/w4a8.cu:44-68), instead of by sfq_unpack_w4a8_int8 into a
 * dense [N, K] copy; accumulators and output bits are those of sfq_unpack_w4a8_int8 + sfq_gemm_int8. No counterpart in the
 * reference, which always materialises the int8 weight. K % 128 == 0; bias and GELU allowed, no gate, no SwiGLU; nibbles and
 * codebook 16-byte aligned, group scales 8-byte aligned. Returns an error (and launches nothing) where that does not hold. */
SFQ_API int sfq_gemm_w4a8_fused(const int8_t* d_q, const uint8_t* d_w_packed, const uint8_t* d_group_scale,
                                const float* d_codebook, const sfq_epilogue* ep, void* d_y_bf16, int M, int N, int K,
                                void* stream);
/* y = epilogue(global * sum(a_fp4 * w_fp4 * block scales)). Replaces nvfp4_gemm_forward_q
 * (include/slopfab/cuda/nvfp4_gemm.cuh:101-113). Activations in the GEMM_FEED layout. */
SFQ_API int sfq_gemm_nvfp4(const uint8_t* d_a_packed, const uint8_t* d_a_scale_tiled, const uint8_t* d_w_packed,
                           const uint8_t* d_w_scale_tiled, const sfq_epilogue* ep, void* d_y_bf16,
                           int M, int N, int K, void* stream);
/* nvfp4_gemm_forward_q with its own operand convention (include/slopfab/cuda/nvfp4_gemm.cuh:101-113): activations as
 * launch_quantize_nvfp4_activations / sfq_quantize_nvfp4_block(REFERENCE) wrote them (low nibble = even element, scales
 * row-major), no bias, no activation. They are converted into the GEMM_FEED layout in stream-ordered scratch that the
 * call allocates and frees on `stream` (the reference signature has no workspace); sfq_gemm_nvfp4 is the form without
 * that conversion. Refused like the reference when the device or the shape has no native path. */
SFQ_API int sfq_gemm_nvfp4_reference_layout(const uint8_t* d_xq, const uint8_t* d_xs, const uint8_t* d_w_packed,
                                            const uint8_t* d_w_scale_tiled, float global_scale, void* d_y_bf16, int rows,
                                            int out_features, int in_features, void* stream);
/* y = epilogue(x[M,K] * w[N,K]^T), bf16 operands, fp32 accumulate: the cuBLAS bf16 GemmEx of
 * src/cuda/linear.cu:243-246. K % 8 == 0. */
SFQ_API int sfq_gemm_bf16(const void* d_x_bf16, const void* d_w_bf16, const sfq_epilogue* ep, void* d_y_bf16,
                          int M, int N, int K, void* stream);
/* Test hooks. Both are thread-local, apply only to the three stand-alone sfq_gemm_* entry points above when called from
 * the same thread (a runner, the LoRA branch and the static entry point never read them), and are switched off again by
 * passing zeros / -1. No counterpart in the reference.
 *   variant: tile_n 128 or 256 selects the one-CTA kernel with that tile width (0 = the default CTA-pair kernel),
 *     band_m the row tiles per raster band (0 = default), max_ctas the grid size (0 = one CTA per SM).
 *   lost load: the producer warp leaves out the loads of pipeline iteration `iteration` (>= 0) while still announcing
 *     their bytes, and every bounded wait gives up after `wait_cycles` clocks instead of about a second. The launch then
 *     ends by the kernels' own abort path -- status code in sfq_device_status, loads drained, TMEM freed -- which is
 *     what the test of that path checks; the output of such a launch is unspecified. */
SFQ_API void sfq_test_gemm_variant(int tile_n, int band_m, int max_ctas);
SFQ_API void sfq_test_gemm_lost_load(int iteration, long long wait_cycles);

/* ---- LinearRunner (include/slopfab/cuda/linear.cuh:182-242) ---------------- */

SFQ_API int sfq_runner_create(void* stream, sfq_runner** out);
SFQ_API void sfq_runner_destroy(sfq_runner* r);
SFQ_API int sfq_runner_set_native(sfq_runner* r, int enable); /* LinearRunner::set_native */
SFQ_API int sfq_runner_native(const sfq_runner* r);
/* Fused epilogue activation applied by forward/forward_prepared (default none). Not part of
 * the reference runner, which runs launch_gelu_tanh as a separate launch. */
SFQ_API int sfq_runner_set_activation(sfq_runner* r, int activation);

/* linear_workspace_bytes / linear_dense_weight_bytes / linear_activation_workspace_bytes,
 * include/slopfab/cuda/linear.cuh:156,179-180. Sizes are for THIS library's kernels
 * (smaller than the reference's: no int32 [M,N] buffer, no rotated bf16 copy). */
SFQ_API int sfq_linear_workspace_bytes(const sfq_quant_weight* w, int rows, int compute, size_t* out);
SFQ_API int sfq_linear_dense_weight_bytes(const sfq_quant_weight* w, size_t* out);
SFQ_API int sfq_linear_activation_workspace_bytes(const sfq_quant_weight* w, int rows, int compute, size_t* out);

/* LinearRunner::forward: y[rows,out] = x[rows,in] W^T + b. The workspace is a caller-owned
 * device arena (256-byte aligned carving, rewound at return; Workspace of
 * include/slopfab/cuda/workspace.cuh:21-76). rows <= 0 is a no-op. */
SFQ_API int sfq_linear_forward(sfq_runner* r, const sfq_quant_weight* w, const void* d_x_bf16, int rows,
                               void* d_y_bf16, void* d_workspace, size_t workspace_bytes);
/* LinearRunner::prepare: carves what stays constant across a row-chunk loop out of the
 * front of the workspace and reports how many bytes it consumed; *d_prepared is null exactly
 * when the weight has no dense bf16 form (native NVFP4), as in the reference. For W4A8/W6A8 the
 * expanded int8 weight is kept in the consumed prefix so that chunks do not re-expand it. */
SFQ_API int sfq_linear_prepare(sfq_runner* r, const sfq_quant_weight* w, void* d_workspace, size_t workspace_bytes,
                               const void** d_prepared, size_t* consumed_bytes);
/* LinearRunner::forward_prepared. `d_prepared` is what sfq_linear_prepare returned for `w`;
 * the workspace passed here must start after the consumed prefix. */
SFQ_API int sfq_linear_forward_prepared(sfq_runner* r, const sfq_quant_weight* w, const void* d_prepared,
                                        const void* d_x_bf16, int rows, void* d_y_bf16, void* d_workspace,
                                        size_t workspace_bytes);

/* ---- caller side: the checkpoint boundary ------------------------------------------ */

/* Element types of safetensors entries (the reference's DType, include/slopfab/dtype.h:16-30). */
typedef enum {
  SFQ_DT_UNKNOWN = 0, SFQ_DT_BOOL, SFQ_DT_U8, SFQ_DT_I8, SFQ_DT_I16, SFQ_DT_I32, SFQ_DT_I64, SFQ_DT_F8E4M3, SFQ_DT_F8E5M2,
  SFQ_DT_F16, SFQ_DT_BF16, SFQ_DT_F32, SFQ_DT_F64
} sfq_dtype;

typedef struct sfq_checkpoint sfq_checkpoint;

/* Maps a .safetensors file and parses its header (SafeTensors, include/slopfab/safetensors.h). The handle owns the
 * mapping and every device buffer sfq_checkpoint_linear uploads; close it after the last use of those weights. */
SFQ_API int sfq_checkpoint_open(const char* path, sfq_checkpoint** out);
SFQ_API void sfq_checkpoint_close(sfq_checkpoint* c);
SFQ_API int sfq_checkpoint_count(const sfq_checkpoint* c);
/* One entry by name: dtype (sfq_dtype), rank and up to 8 dimensions, host pointer into the mapping, byte count.
 * Any output may be null. SFQ_ERR_RUNTIME when the tensor does not exist. */
SFQ_API int sfq_checkpoint_tensor(const sfq_checkpoint* c, const char* name, int32_t* dtype, int32_t* rank, int64_t* shape8,
                                  const void** h_data, size_t* nbytes);
/* One string of the header's __metadata__ table, NUL-terminated into `buffer` (truncated to capacity); *length is
 * the full length. */
SFQ_API int sfq_checkpoint_metadata(const sfq_checkpoint* c, const char* key, char* buffer, size_t capacity, size_t* length);
/* quant() of the reference's loader (src/dit/transformer_load.cpp:585-659): decides the layer's format from the file
 * (<name>.comfy_quant or the header's _quantization_metadata for W4A8 / W6A8 / ConvRot tags, the bitsandbytes NF4
 * state tensor, the U8 weight + e4m3 [*, in/16] scale pair for NVFP4, else the weight's dtype), checks the tensor
 * sizes the layer needs, uploads them (each tensor once per handle; channel scales, codebooks and NF4 tables as fp32)
 * and fills `out` with DEVICE pointers. Same refusals as the reference: nvfp4 without weight_scale_2, fp8 / int8
 * without weight_scale, unknown quant formats, incompatible ConvRot metadata, W4 group != 16, ConvRot != 256. */
SFQ_API int sfq_checkpoint_linear(sfq_checkpoint* c, const char* name, int out_features, int in_features,
                                  sfq_quant_weight* out);
/* The same rule without a device: every pointer of `out` is a HOST pointer (into the mapping, or into fp32 copies the
 * handle keeps). For inspection and for hosts that stage uploads themselves. */
SFQ_API int sfq_checkpoint_linear_host(sfq_checkpoint* c, const char* name, int out_features, int in_features,
                                       sfq_quant_weight* out);

/* ---- caller side: views over a row-fused weight ----------------------------------- */

/* The index-th of `parts` equal row blocks of a fused weight, e.g. Wq / Wk / Wv of the canonical [Wq; Wk; Wv] upload:
 * build_block's view slicing (src/dit/transformer_load.cpp:660-737). Every row-indexed array moves with the view (packed
 * data, group / block scales, per-channel scales, bias). Refused with SFQ_ERR_INVALID_ARGUMENT where a block is not a
 * whole number of storage units: NVFP4 needs rows-per-block % 128 == 0 (128-row scale tiles), NF4 whole absmax and
 * nested blocks. Pointers are not dereferenced (host or device). Host only. */
SFQ_API int sfq_weight_row_block(const sfq_quant_weight* fused, int parts, int index, sfq_quant_weight* out);

/* ---- caller side: token packing -> adaLN table index --------------------------- */

/* SequenceLayout (include/slopfab/dit/packing.h:37-73) reduced to the extents the row order depends on. Rows are
 * packed [text | condition video | condition audio | audio | video]. */
typedef struct sfq_sequence_layout {
  int32_t num_text;
  int32_t num_condition_video;
  int32_t num_condition_audio;
  int32_t condition_audio_is_explicit; /* 0: the legacy convention, num_condition_video is also the audio prefix */
  int32_t num_audio_rows;
  int32_t num_video_rows;
} sfq_sequence_layout;

/* build_indices (src/dit/packing.cpp:213-248): h_text [num_text], h_audio [num_audio_rows], h_video [conditions +
 * num_video_rows] (every condition row, then the targets), h_tags [total] (video 0, text 1, audio 2). Any output may
 * be null. Host only. */
SFQ_API int sfq_build_indices(const sfq_sequence_layout* layout, int32_t* h_text, int32_t* h_audio, int32_t* h_video,
                              int32_t* h_tags);
/* build_row_timesteps, the two-timestep form (src/dit/packing.cpp:407-489): h_indices [total] (position of the row's
 * timestep in the ascending set of those that occur), h_adaln [total] = index * 3 + max(tag, 0) -- the d_adaln_index
 * of sfq_norm -- and up to unique_capacity entries of the set. h_tags: the caller's tags (padding rows carry -1), or
 * null for the layout's own. h_indices, h_unique, h_num_unique may be null. Host only. */
SFQ_API int sfq_build_row_timesteps(const sfq_sequence_layout* layout, const int32_t* h_tags, float video_t, float audio_t,
                                    int32_t* h_indices, int32_t* h_adaln, float* h_unique, int unique_capacity,
                                    int* h_num_unique);
/* The four-timestep form for reference-conditioned requests (src/dit/packing.cpp:491-523): the first
 * num_condition_video entries of the video list carry condition_video_t, the first num_condition_audio entries of the
 * audio list condition_audio_t, the rest of the audio list audio_t, everything else video_t. Up to four unique values. */
SFQ_API int sfq_build_row_timesteps4(const sfq_sequence_layout* layout, const int32_t* h_tags, float video_t, float audio_t,
                                     float condition_video_t, float condition_audio_t, int32_t* h_indices,
                                     int32_t* h_adaln, float* h_unique, int unique_capacity, int* h_num_unique);
/* sfq_build_indices + sfq_build_row_timesteps in one call with the layout spelled out (the layout's own tags, at most
 * two unique values). Any output except h_adaln may be null. Host only. */
SFQ_API int sfq_build_adaln_index(int num_text, int num_condition_video, int num_condition_audio,
                                  int condition_audio_is_explicit, int num_audio_rows, int num_video_rows,
                                  float video_t, float audio_t, int32_t* h_tags, int32_t* h_indices,
                                  int32_t* h_adaln, float* h_unique2, int* h_num_unique);

/* ---- for callers that cannot allocate ------------------------------------------ */

/* LinearRunner::forward_f32 (include/slopfab/cuda/linear.cuh:229-232, src/cuda/linear.cu:251-285): fp32 activations
 * and fp32 output; the weight as stored when fp32, else its dense bf16 form; fp32 accumulation on CUDA cores; the
 * bias added to the finished sum. The DiT uses this arm for the few timestep rows of the adaLN tables
 * (src/dit/transformer_execution.cpp:55,63). AWQ pre-scale and ConvRot are applied to the fp32 activation first, as in
 * the reference; W4A8/W6A8 weights are refused (they need bf16 activations). */
SFQ_API int sfq_linear_forward_f32(sfq_runner* r, const sfq_quant_weight* w, const float* d_x_f32, int rows, float* d_y_f32,
                                   void* d_workspace, size_t workspace_bytes);

/* launch_adaln_expand (src/dit/transformer_support.h:58, src/cuda/dit_kernels.cu:61-134): the per-timestep
 * modulation tables out[param][t][modality][channel] = bias[p] + sum_k w[p,k] code[t,k] as one fp32 fma chain
 * started from the bias, p = (modality * num_param + param) * channels + channel. Bit-exact. */
SFQ_API int sfq_adaln_expand(const float* d_w, const float* d_bias, const float* d_code, float* d_out, int num_t,
                             int num_modality, int num_param, int channels, int rank, void* stream);

/* launch_head_rmsnorm (include/slopfab/cuda/nn_kernels.cuh:129-134) and launch_rope_h3 (:95-112) as ONE in-place
 * pass over x[rows, heads, 128] with a row pitch of `ld` elements, so that the q and k thirds of the fused projection
 * are normalised and rotated where they lie (src/dit/transformer_execution.cpp:277-289: QK-norm first, then RoPE; v is
 * left alone). d_norm_weight: bf16 [128] or null (no norm); d_cos / d_sin: fp32 [rows, 96] or both null (no rotation);
 * the rotation pairs channel j with j + 48 over the first 96 channels and passes 96..127 through. Bit-exact. */
SFQ_API int sfq_head_norm_rope(void* d_x_bf16, int ld, const void* d_norm_weight_bf16, const float* d_cos, const float* d_sin,
                               int rows, int heads, int head_dim, float eps, void* stream);

/* ---- full self-attention, head_dim 128 ---------------------------------------------------------------
 * attention_forward / attention_forward_query_chunk / attention_forward_gqa of
 * include/slopfab/cuda/attention.cuh:176-203: out[seq_q, heads*128] = softmax(q k^T * scale) v per head, no mask,
 * no causality. q and out may be a compact chunk of the sequence's rows (seq_q <= seq_kv is not required); k and v
 * are the whole sequence, [seq_kv, kv_heads*128]; query head h reads key/value head h / (heads / kv_heads). The
 * three leading dimensions are in elements, so the thirds of a fused QKV projection are passed as they lie
 * (ld = 3 * heads * 128). scale <= 0 selects 1/sqrt(128). The workspace (sfq_attention_workspace_bytes) holds V
 * transposed. out may not alias the inputs. Parity: the reference's own bound against a dense fp64 softmax,
 * |err| <= 1e-3 + 1e-2 |want| (tests/test_nn_kernels_attention_synthetic.cu:40). */
SFQ_API int sfq_attention_workspace_bytes(int seq_kv, int kv_heads, int head_dim, size_t* out);
SFQ_API int sfq_attention_forward(const void* d_q_bf16, int ld_q, const void* d_k_bf16, const void* d_v_bf16, int ld_kv,
                                  void* d_out_bf16, int ld_out, int seq_q, int seq_kv, int heads, int kv_heads,
                                  int head_dim, float scale, void* d_workspace, size_t workspace_bytes, void* stream);

/* ---- LoRA side branch: y[rows,out] += (x[rows,in] A^T) B^T -------------------------------------------
 * LoraRunner of include/slopfab/cuda/lora.cuh:14-37 (src/cuda/lora.cu:16-93). Factors arrive as fp32 host
 * arrays in model coordinates (LoraFactors, include/slopfab/lora.h:18-23: a[rank,in], b[out_total,rank], the
 * adapter's scale already folded into b) and are rounded to bf16 on upload. `row_offset`/`out` select the rows
 * of b that belong to one view of a fused projection (q, k or v). Several attach calls under one key add
 * several factor pairs; apply runs all of them; an unknown key is a no-op. Both products run on the tcgen05
 * bf16 GEMM (fp32 accumulation), hidden and product rounded to bf16 like the reference's, the addition fused
 * into the second GEMM's epilogue. */
typedef struct sfq_lora sfq_lora;
SFQ_API int sfq_lora_create(sfq_lora** out);
SFQ_API void sfq_lora_destroy(sfq_lora* l);
SFQ_API int sfq_lora_attach(sfq_lora* l, const void* key, const float* a, const float* b, int rank, int in_features,
                            int out_total, int row_offset, int out);
/* The same with the bf16 factor bytes written to host staging memory at *staged_offset (advanced in 256-byte
 * steps) instead of being uploaded; apply reads them at the same offset of `staged_device` (the caller copies). */
SFQ_API int sfq_lora_attach_staged(sfq_lora* l, const void* key, const float* a, const float* b, int rank,
                                   int in_features, int out_total, int row_offset, int out, uint8_t* staged_host,
                                   uint8_t* staged_device, size_t* staged_offset);
SFQ_API int sfq_lora_apply(sfq_lora* l, const void* key, const void* d_x_bf16, int rows, void* d_y_bf16, void* stream);
SFQ_API int sfq_lora_bytes(const sfq_lora* l, size_t* weight_bytes, size_t* scratch_bytes);

/* Bytes of scratch built into the library image for sfq_linear_nvfp4_forward_static (16 MiB, plus a
 * 256-byte status area). Every GPU that loads libsfq.so holds this much until the process exits. */
#define SFQ_STATIC_SCRATCH_BYTES (16u * 1024u * 1024u)

/* The native NVFP4 Linear, y[rows,out] = epilogue(x[rows,in] W^T), without any allocation and without a
 * caller workspace. (No counterpart in the reference: its runner always carves scratch from a
 * Workspace arena.) It is meant for hosts that may not allocate when they call us -- an embedder that has
 * handed out all device memory up front, a plugin invoked inside a frame or audio callback, a serving loop
 * that freezes its allocator after start-up -- and for whom even passing a workspace is not possible
 * because they own no spare device buffer. The quantized activation lives in a fixed array inside the
 * library instead; inputs and outputs are still the caller's.
 *   - Limit: align256(rows * in_features / 2) + ceil(rows/128)*128 * in_features/16 must not exceed
 *     SFQ_STATIC_SCRATCH_BYTES (e.g. 2048 rows x 13824, or 5800 rows x 5120). Larger calls are refused with
 *     SFQ_ERR_INVALID_ARGUMENT and a message; split the rows or use sfq_linear_forward.
 *   - The entry point itself calls no cudaMalloc / cudaFree / allocating library routine, on any call. The CUDA
 *     runtime does its own one-time work the first time each kernel variant runs on a device (it loads the
 *     module's code and this array, and the launchers set a shared-memory attribute and look up one driver entry
 *     point), so make one warm-up call per device, with the bias / activation combination you will use, before
 *     you freeze allocations.
 *   - The first call on each device looks up the device address of the array (a host-side query, no
 *     allocation). Make that first call outside of any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels can overlap on the GPU (different
 *     streams, or graph branches) race on it. Serialise them on one stream.
 *   - The array keeps the previous call's bytes; the call rewrites everything it later reads, so earlier calls
 *     never leak into the result.
 *   - A kernel that abandons a bounded wait records it in the array's own status word, not in the word
 *     sfq_device_status reads: read it with sfq_static_status. The first code recorded stays until it is read.
 * Weight layout, bias, activation and numerics are those of sfq_gemm_nvfp4 fed by
 * sfq_quantize_nvfp4_block(GEMM_FEED); results are bit-identical to the runner's native NVFP4 path. */
SFQ_API int sfq_linear_nvfp4_forward_static(const void* d_x_bf16, int rows, const uint8_t* d_w_packed,
                                            const uint8_t* d_w_scale_tiled, float global_scale, const void* d_bias,
                                            int bias_format, int activation, void* d_y_bf16, int out_features,
                                            int in_features, void* stream);
/* Reads and clears the status word of sfq_linear_nvfp4_forward_static on the current device (no counterpart in
 * the reference): 0, or the code of the first bounded wait that one of its kernels abandoned since the last
 * read. Synchronises the device; allocates nothing. */
SFQ_API int sfq_static_status(int* h_code);

#ifdef __cplusplus
}
#endif
#endif /* SFQ_H_ */
