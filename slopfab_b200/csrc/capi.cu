// The C ABI of include/sfq.h: every entry point is a guarded call into the C++
// layer; exceptions become status codes and a thread-local message.
#include "../../include/sfq.h"

#include <cstring>
#include <new>
#include <stdexcept>
#include <string>

#include "../../include/slopfab_b200/linear.hpp"
#include "gemm_tc.cuh"
#include "kernels.cuh"
#include "packers.h"
#include "runtime.h"

namespace {

thread_local std::string g_error;

template <class F> int guarded(F&& f) {
  try {
    f();
    return SFQ_OK;
  } catch (const std::invalid_argument& e) {
    g_error = e.what();
    return SFQ_ERR_INVALID_ARGUMENT;
  } catch (const std::bad_alloc& e) {
    g_error = e.what();
    return SFQ_ERR_OUT_OF_MEMORY;
  } catch (const std::exception& e) {
    g_error = e.what();
    // Same classification by message as the reference's C ABI (src/capi/internal.h:103-120).
    if (g_error.find("out of memory") != std::string::npos || g_error.find("arena exhausted") != std::string::npos)
      return SFQ_ERR_OUT_OF_MEMORY;
    return SFQ_ERR_RUNTIME;
  } catch (...) {
    g_error = "unknown error";
    return SFQ_ERR_RUNTIME;
  }
}

using bf16 = __nv_bfloat16;
namespace sc = slopfab::cuda;

cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

sfq::NormArgs to_norm(const sfq_norm* n) {
  sfq::NormArgs a;
  if (n != nullptr && n->d_norm_weight != nullptr) {
    a.weight = static_cast<const bf16*>(n->d_norm_weight);
    a.scale = n->d_scale;
    a.shift = n->d_shift;
    a.index = n->d_adaln_index;
    a.eps = n->eps;
  }
  return a;
}

sc::QuantWeight to_weight(const sfq_quant_weight* w) {
  if (w == nullptr) throw std::invalid_argument("sfq: null weight descriptor");
  if (w->format < SFQ_F32 || w->format > SFQ_W6A8) throw std::invalid_argument("sfq: unknown weight format");
  sc::QuantWeight q;
  q.format = static_cast<sc::QuantFormat>(w->format);
  q.data = w->data;
  q.out_features = w->out_features;
  q.in_features = w->in_features;
  q.weight_scale = w->weight_scale;
  q.per_channel_scale = w->per_channel_scale != 0;
  q.input_scale = w->input_scale;
  q.full_precision = w->full_precision != 0;
  q.block_scale = w->block_scale;
  q.packed_group_size = w->packed_group_size;
  q.w4_codebook = w->w4_codebook;
  q.global_scale = w->global_scale;
  q.pre_quant_scale = static_cast<const bf16*>(w->pre_quant_scale);
  q.nf4_absmax = w->nf4_absmax;
  q.nf4_quant_map = w->nf4_quant_map;
  q.nf4_nested_quant_map = w->nf4_nested_quant_map;
  q.nf4_nested_absmax = w->nf4_nested_absmax;
  q.nf4_block_size = w->nf4_block_size;
  q.nf4_nested_block_size = w->nf4_nested_block_size;
  q.nf4_nested_offset = w->nf4_nested_offset;
  q.convrot = w->convrot != 0;
  q.convrot_group = w->convrot_group;
  q.bias = w->bias;
  q.bias_format = static_cast<sc::QuantFormat>(w->bias_format);
  return q;
}

sfq::GemmArgs to_gemm(const sfq_epilogue* ep, void* y, int M, int N, int K) {
  sfq::GemmArgs g;
  g.M = M;
  g.N = N;
  g.K = K;
  g.y = static_cast<bf16*>(y);
  g.ldy = N;
  if (ep != nullptr) {
    g.row_scale = ep->d_row_scale;
    g.col_scale = ep->d_col_scale;
    g.global_scale = ep->global_scale;
    g.bias = ep->d_bias;
    if (ep->d_bias != nullptr && ep->bias_format != SFQ_F32 && ep->bias_format != SFQ_BF16)
      throw std::invalid_argument("sfq gemm: bias must be fp32 or bf16");
    g.bias_is_bf16 = ep->bias_format == SFQ_BF16;
    if (ep->activation != SFQ_ACT_NONE && ep->activation != SFQ_ACT_GELU_TANH && ep->activation != SFQ_ACT_SWIGLU)
      throw std::invalid_argument("sfq gemm: unknown activation");
    g.act = ep->activation;
    if (g.act == SFQ_ACT_SWIGLU) g.ldy = N / 2;  // the output has one column per (gate, up) pair
    if ((ep->d_gate != nullptr) != (ep->d_gate_index != nullptr))
      throw std::invalid_argument("sfq gemm: the gated residual needs both the gate table and the row index");
    if (reinterpret_cast<uintptr_t>(ep->d_gate) % 16 != 0)
      throw std::invalid_argument("sfq gemm: the gate table must be 16-byte aligned");
    g.gate = ep->d_gate;
    g.gate_index = ep->d_gate_index;
  }
  g.status = sfq::device_status_word();
  sfq::apply_test_hooks(g);
  return g;
}

}  // namespace

// Shared with capi_runner.cu.
namespace sfq_capi {
int run_guarded(void (*fn)(void*), void* ctx) {
  return guarded([&] { fn(ctx); });
}
sc::QuantWeight weight_from_c(const sfq_quant_weight* w) { return to_weight(w); }
void set_error(const char* text) { g_error = text ? text : ""; }  // for entry points in other files
}  // namespace sfq_capi

extern "C" {

const char* sfq_last_error(void) { return g_error.c_str(); }
int sfq_version(void) { return 100; }

void sfq_quant_weight_init(sfq_quant_weight* w) {
  if (w == nullptr) return;
  std::memset(w, 0, sizeof(*w));
  w->format = SFQ_BF16;
  w->packed_group_size = 16;
  w->global_scale = 1.0f;
  w->nf4_block_size = 64;
  w->nf4_nested_block_size = 256;
  w->convrot_group = 256;
  w->bias_format = SFQ_F32;
}

int sfq_device_status(int* h_code) {
  return guarded([&] {
    const int code = sfq::read_and_clear_device_status();
    if (h_code) *h_code = code;
  });
}

// ---- host packers
int sfq_pack_nvfp4(const float* h_w, int out_features, int in_features, float global_scale, uint8_t* h_data,
                   uint8_t* h_scale_tiled) {
  return guarded([&] { sfq::pack_nvfp4(h_w, out_features, in_features, global_scale, h_data, h_scale_tiled); });
}
int sfq_pack_w4a8(const float* h_w, int out_features, int in_features, int8_t* h_packed, uint8_t* h_group_scale,
                  float* h_channel_scale, float* h_codebook16) {
  return guarded([&] { sfq::pack_w4a8(h_w, out_features, in_features, h_packed, h_group_scale, h_channel_scale, h_codebook16); });
}
int sfq_pack_w6a8(const float* h_w, int out_features, int in_features, int group, int8_t* h_packed,
                  uint8_t* h_group_scale, float* h_channel_scale) {
  return guarded([&] { sfq::pack_w6a8(h_w, out_features, in_features, group, h_packed, h_group_scale, h_channel_scale); });
}
int sfq_pack_int8(const float* h_w, int out_features, int in_features, int convrot_group, int8_t* h_codes,
                  float* h_scale) {
  return guarded([&] { sfq::pack_int8(h_w, out_features, in_features, convrot_group, h_codes, h_scale); });
}

// ---- device unpackers
int sfq_unpack_nvfp4_bf16(const uint8_t* d_data, const uint8_t* d_scale_tiled, float global_scale, void* d_out_bf16,
                          int out_features, int in_features, void* stream) {
  return guarded([&] {
    sfq::unpack_nvfp4_bf16(d_data, d_scale_tiled, global_scale, static_cast<bf16*>(d_out_bf16), out_features,
                           in_features, as_stream(stream));
  });
}
int sfq_unpack_w4a8_int8(const int8_t* d_packed, const uint8_t* d_group_scale, const float* d_codebook, int8_t* d_out,
                         int out_features, int in_features, int group, void* stream) {
  return guarded([&] {
    sfq::unpack_w4a8_int8(d_packed, d_group_scale, d_codebook, d_out, out_features, in_features, group, as_stream(stream));
  });
}
int sfq_unpack_w6a8_int8(const int8_t* d_packed, const uint8_t* d_group_scale, int8_t* d_out, int out_features,
                         int in_features, int group, void* stream) {
  return guarded([&] {
    sfq::unpack_w6a8_int8(d_packed, d_group_scale, d_out, out_features, in_features, group, as_stream(stream));
  });
}
int sfq_unpack_int8_bf16(const int8_t* d_codes, const float* d_scale, void* d_out_bf16, int out_features,
                         int in_features, void* stream) {
  return guarded([&] {
    sfq::unpack_int8_bf16(d_codes, d_scale, static_cast<bf16*>(d_out_bf16), out_features, in_features, as_stream(stream));
  });
}
int sfq_unpack_f8e4m3_bf16(const uint8_t* d_codes, const float* d_scale, void* d_out_bf16, size_t n, void* stream) {
  return guarded([&] { sfq::unpack_f8e4m3_bf16(d_codes, d_scale, static_cast<bf16*>(d_out_bf16), n, as_stream(stream)); });
}
int sfq_unpack_nf4_bf16(const uint8_t* d_packed, const uint8_t* d_absmax, const float* d_quant_map,
                        const float* d_nested_quant_map, const float* d_nested_absmax, int block_size,
                        int nested_block_size, float nested_offset, void* d_out_bf16, int out_features, int in_features,
                        void* stream) {
  return guarded([&] {
    sfq::unpack_nf4_bf16(d_packed, d_absmax, d_quant_map, d_nested_quant_map, d_nested_absmax, block_size,
                         nested_block_size, nested_offset, static_cast<bf16*>(d_out_bf16), out_features, in_features,
                         as_stream(stream));
  });
}
int sfq_pre_quant_scale(const void* d_src_bf16, const void* d_scale_bf16, void* d_dst_bf16, int rows, int dim,
                        void* stream) {
  return guarded([&] {
    sfq::pre_quant_scale(static_cast<const bf16*>(d_src_bf16), static_cast<const bf16*>(d_scale_bf16),
                         static_cast<bf16*>(d_dst_bf16), rows, dim, as_stream(stream));
  });
}
int sfq_unpack_int8_f16(const int8_t* d_codes, const float* d_scale, void* d_out_f16, int out_features,
                        int in_features, int rotation_group, int canonicalize_subnormals, void* stream) {
  return guarded([&] {
    sfq::unpack_int8_f16(d_codes, d_scale, static_cast<__half*>(d_out_f16), out_features, in_features, rotation_group,
                         canonicalize_subnormals, as_stream(stream));
  });
}

// ---- activation side
int sfq_rmsnorm(const void* d_x_bf16, const sfq_norm* norm, void* d_out_bf16, int rows, int dim, void* stream) {
  return guarded([&] {
    sfq::rmsnorm(static_cast<const bf16*>(d_x_bf16), to_norm(norm), static_cast<bf16*>(d_out_bf16), rows, dim,
                 as_stream(stream));
  });
}
int sfq_convrot(const void* d_x_bf16, void* d_out_bf16, int rows, int dim, int group, void* stream) {
  return guarded([&] {
    sfq::convrot(static_cast<const bf16*>(d_x_bf16), static_cast<bf16*>(d_out_bf16), rows, dim, group, as_stream(stream));
  });
}
int sfq_convrot_f32(const float* d_x, float* d_out, int rows, int dim, int group, void* stream) {
  return guarded([&] { sc::launch_convrot_f32(d_x, d_out, rows, dim, group, as_stream(stream)); });
}
int sfq_int8_output_bf16(const int32_t* d_acc, const float* d_row_scale, const float* d_channel_scale, void* d_y_bf16, int rows, int cols,
                         void* stream) {
  return guarded([&] {
    sc::launch_w4a8_output_bf16(d_acc, d_row_scale, d_channel_scale, static_cast<bf16*>(d_y_bf16), rows, cols, as_stream(stream));
  });
}
int sfq_int8_output_f32(int32_t* d_acc_inout, const float* d_row_scale, const float* d_channel_scale, int rows, int cols, void* stream) {
  return guarded([&] { sc::launch_dequant_w4a8_output(d_acc_inout, d_row_scale, d_channel_scale, rows, cols, as_stream(stream)); });
}
int sfq_quantize_f8e4m3(const void* d_x_bf16, float input_scale, uint8_t* d_out, size_t n, void* stream) {
  return guarded([&] { sc::launch_quantize_f8e4m3(static_cast<const bf16*>(d_x_bf16), input_scale, d_out, n, as_stream(stream)); });
}
int sfq_unpack_nf4_f16(const uint8_t* d_packed, const uint8_t* d_absmax, const float* d_quant_map, const float* d_nested_quant_map,
                       const float* d_nested_absmax, int block_size, int nested_block_size, float nested_offset, void* d_out_f16, size_t n,
                       void* stream) {
  return guarded([&] {
    sc::launch_dequant_nf4_f16(d_packed, d_absmax, d_quant_map, d_nested_quant_map, d_nested_absmax, block_size, nested_block_size,
                               nested_offset, static_cast<__half*>(d_out_f16), n, as_stream(stream));
  });
}
int sfq_gemm_nvfp4_reference_layout(const uint8_t* d_xq, const uint8_t* d_xs, const uint8_t* d_w_packed, const uint8_t* d_w_scale_tiled,
                                    float global_scale, void* d_y_bf16, int rows, int out_features, int in_features, void* stream) {
  return guarded([&] {
    sc::nvfp4_gemm_forward_q(d_xq, d_xs, d_w_packed, d_w_scale_tiled, global_scale, static_cast<bf16*>(d_y_bf16), rows, out_features,
                             in_features, as_stream(stream));
  });
}
int sfq_quantize_int8_token(const void* d_x_bf16, const sfq_norm* norm, int8_t* d_q, float* d_row_scale,
                            void* d_normed_out_bf16, int rows, int dim, int apply_convrot, void* stream) {
  return guarded([&] {
    sfq::quantize_int8_token(static_cast<const bf16*>(d_x_bf16), to_norm(norm), d_q, d_row_scale,
                             static_cast<bf16*>(d_normed_out_bf16), rows, dim, apply_convrot != 0, as_stream(stream));
  });
}
int sfq_quantize_nvfp4_block(const void* d_x_bf16, const sfq_norm* norm, uint8_t* d_packed, uint8_t* d_scales,
                             void* d_normed_out_bf16, int rows, int dim, int layout, void* stream) {
  return guarded([&] {
    sfq::quantize_nvfp4_block(static_cast<const bf16*>(d_x_bf16), to_norm(norm), d_packed, d_scales,
                              static_cast<bf16*>(d_normed_out_bf16), rows, dim, layout, as_stream(stream));
  });
}
size_t sfq_nvfp4_act_scale_bytes(int rows, int dim) { return sfq::nvfp4_act_scale_bytes(rows, dim); }

int sfq_gelu_tanh(void* d_x_bf16, size_t n, void* stream) {
  return guarded([&] { sfq::gelu_tanh(static_cast<bf16*>(d_x_bf16), n, as_stream(stream)); });
}
int sfq_swiglu(const void* d_fused_bf16, void* d_out_bf16, int rows, int inner, void* stream) {
  return guarded([&] {
    sfq::swiglu(static_cast<const bf16*>(d_fused_bf16), static_cast<bf16*>(d_out_bf16), rows, inner, as_stream(stream));
  });
}
int sfq_add_gated(void* d_x_bf16, const void* d_branch_bf16, const float* d_gate, const int32_t* d_adaln_index,
                  int rows, int dim, void* stream) {
  return guarded([&] {
    sfq::add_gated(static_cast<bf16*>(d_x_bf16), static_cast<const bf16*>(d_branch_bf16), d_gate, d_adaln_index, rows,
                   dim, as_stream(stream));
  });
}

// ---- GEMMs
int sfq_gemm_int8(const int8_t* d_q, const int8_t* d_w8, const sfq_epilogue* ep, void* d_y_bf16, int M, int N, int K,
                  void* stream) {
  return guarded([&] { sfq::gemm_int8(d_q, d_w8, to_gemm(ep, d_y_bf16, M, N, K), as_stream(stream)); });
}
int sfq_gemm_w4a8_fused(const int8_t* d_q, const uint8_t* d_w_packed, const uint8_t* d_group_scale, const float* d_codebook,
                        const sfq_epilogue* ep, void* d_y_bf16, int M, int N, int K, void* stream) {
  return guarded([&] {
    if (!d_q || !d_w_packed || !d_group_scale || !d_codebook) throw std::invalid_argument("sfq_gemm_w4a8_fused: null operand");
    sfq::GemmArgs g = to_gemm(ep, d_y_bf16, M, N, K);
    g.w4_gscale = d_group_scale;
    g.w4_codebook = d_codebook;
    if (M <= 0 || N <= 0 || K <= 0 || !sfq::gemm_pair_w4a8(d_q, d_w_packed, g, as_stream(stream)))
      throw std::invalid_argument("sfq_gemm_w4a8_fused: needs K % 128 == 0, the plain epilogue and a device that schedules CTA pairs");
  });
}
int sfq_gemm_nvfp4(const uint8_t* d_a_packed, const uint8_t* d_a_scale_tiled, const uint8_t* d_w_packed,
                   const uint8_t* d_w_scale_tiled, const sfq_epilogue* ep, void* d_y_bf16, int M, int N, int K,
                   void* stream) {
  return guarded([&] {
    sfq::GemmArgs g = to_gemm(ep, d_y_bf16, M, N, K);
    g.a_scale_tiled = d_a_scale_tiled;
    g.w_scale_tiled = d_w_scale_tiled;
    sfq::gemm_nvfp4(d_a_packed, d_w_packed, g, as_stream(stream));
  });
}
int sfq_gemm_bf16(const void* d_x_bf16, const void* d_w_bf16, const sfq_epilogue* ep, void* d_y_bf16, int M, int N,
                  int K, void* stream) {
  return guarded([&] {
    sfq::gemm_bf16(static_cast<const bf16*>(d_x_bf16), static_cast<const bf16*>(d_w_bf16),
                   to_gemm(ep, d_y_bf16, M, N, K), as_stream(stream));
  });
}
int sfq_head_norm_rope(void* d_x_bf16, int ld, const void* d_norm_weight_bf16, const float* d_cos, const float* d_sin, int rows, int heads,
                       int head_dim, float eps, void* stream) {
  return guarded([&] {
    sfq::head_norm_rope(static_cast<bf16*>(d_x_bf16), ld, static_cast<const bf16*>(d_norm_weight_bf16), d_cos, d_sin, rows, heads, head_dim,
                        eps, as_stream(stream));
  });
}
int sfq_attention_workspace_bytes(int seq_kv, int kv_heads, int head_dim, size_t* out) {
  return guarded([&] {
    if (!out) throw std::invalid_argument("sfq_attention_workspace_bytes: null output");
    *out = sfq::attention_workspace_bytes(seq_kv, kv_heads, head_dim);
  });
}
int sfq_attention_forward(const void* d_q_bf16, int ld_q, const void* d_k_bf16, const void* d_v_bf16, int ld_kv, void* d_out_bf16,
                          int ld_out, int seq_q, int seq_kv, int heads, int kv_heads, int head_dim, float scale, void* d_workspace,
                          size_t workspace_bytes, void* stream) {
  return guarded([&] {
    sfq::attention_forward(static_cast<const bf16*>(d_q_bf16), ld_q, static_cast<const bf16*>(d_k_bf16), static_cast<const bf16*>(d_v_bf16),
                           ld_kv, static_cast<bf16*>(d_out_bf16), ld_out, seq_q, seq_kv, heads, kv_heads, head_dim, scale, d_workspace,
                           workspace_bytes, as_stream(stream));
  });
}
void sfq_test_gemm_variant(int tile_n, int band_m, int max_ctas) { sfq::set_test_gemm_variant(tile_n, band_m, max_ctas); }
void sfq_test_gemm_lost_load(int iteration, long long wait_cycles) { sfq::set_test_gemm_lost_load(iteration, wait_cycles); }

}  // extern "C"
