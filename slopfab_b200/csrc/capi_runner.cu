// C ABI over slopfab::cuda::LinearRunner (include/sfq.h, "LinearRunner" section).
#include "../../include/sfq.h"

#include <new>
#include <stdexcept>
#include <string>

#include "../../include/slopfab_b200/linear.hpp"
#include "../../include/slopfab_b200/lora.hpp"

namespace sc = slopfab::cuda;
using bf16 = __nv_bfloat16;

// Defined in capi.cu.
namespace sfq_capi {
int run_guarded(void (*fn)(void*), void* ctx);
sc::QuantWeight weight_from_c(const sfq_quant_weight* w);
}  // namespace sfq_capi

struct sfq_runner {
  sc::LinearRunner runner;
};
struct sfq_lora {
  sc::LoraRunner runner;
};

namespace {
template <class F> int guarded(F&& f) {
  return sfq_capi::run_guarded([](void* p) { (*static_cast<F*>(p))(); }, &f);
}
sc::ComputeType to_compute(int c) {
  if (c != SFQ_COMPUTE_BF16 && c != SFQ_COMPUTE_F32) throw std::invalid_argument("sfq: unknown compute type");
  return c == SFQ_COMPUTE_F32 ? sc::ComputeType::kF32 : sc::ComputeType::kBF16;
}
}  // namespace

extern "C" {

int sfq_runner_create(void* stream, sfq_runner** out) {
  return guarded([&] {
    if (out == nullptr) throw std::invalid_argument("sfq_runner_create: null output");
    auto* r = new sfq_runner();
    try {
      r->runner.init(nullptr, static_cast<cudaStream_t>(stream));
    } catch (...) {
      delete r;
      throw;
    }
    *out = r;
  });
}

void sfq_runner_destroy(sfq_runner* r) { delete r; }

int sfq_runner_set_native(sfq_runner* r, int enable) {
  return guarded([&] {
    if (r == nullptr) throw std::invalid_argument("sfq: null runner");
    r->runner.set_native(enable != 0);
  });
}

int sfq_runner_native(const sfq_runner* r) { return r != nullptr && r->runner.native() ? 1 : 0; }

int sfq_runner_set_activation(sfq_runner* r, int activation) {
  return guarded([&] {
    if (r == nullptr) throw std::invalid_argument("sfq: null runner");
    if (activation != SFQ_ACT_NONE && activation != SFQ_ACT_GELU_TANH && activation != SFQ_ACT_SWIGLU)
      throw std::invalid_argument("sfq: unknown activation");
    r->runner.set_activation(activation);
  });
}

int sfq_linear_workspace_bytes(const sfq_quant_weight* w, int rows, int compute, size_t* out) {
  return guarded([&] {
    if (out == nullptr) throw std::invalid_argument("sfq: null output");
    *out = sc::linear_workspace_bytes(sfq_capi::weight_from_c(w), rows, to_compute(compute)) + 256;
  });
}
int sfq_linear_dense_weight_bytes(const sfq_quant_weight* w, size_t* out) {
  return guarded([&] {
    if (out == nullptr) throw std::invalid_argument("sfq: null output");
    *out = sc::linear_dense_weight_bytes(sfq_capi::weight_from_c(w));
  });
}
int sfq_linear_activation_workspace_bytes(const sfq_quant_weight* w, int rows, int compute, size_t* out) {
  return guarded([&] {
    if (out == nullptr) throw std::invalid_argument("sfq: null output");
    *out = sc::linear_activation_workspace_bytes(sfq_capi::weight_from_c(w), rows, to_compute(compute)) + 256;
  });
}

int sfq_linear_forward(sfq_runner* r, const sfq_quant_weight* w, const void* d_x_bf16, int rows, void* d_y_bf16,
                       void* d_workspace, size_t workspace_bytes) {
  return guarded([&] {
    if (r == nullptr) throw std::invalid_argument("sfq: null runner");
    sc::Workspace ws;
    ws.adopt(d_workspace, workspace_bytes);
    r->runner.forward(sfq_capi::weight_from_c(w), static_cast<const bf16*>(d_x_bf16), rows,
                      static_cast<bf16*>(d_y_bf16), ws);
  });
}

int sfq_linear_prepare(sfq_runner* r, const sfq_quant_weight* w, void* d_workspace, size_t workspace_bytes,
                       const void** d_prepared, size_t* consumed_bytes) {
  return guarded([&] {
    if (r == nullptr || d_prepared == nullptr || consumed_bytes == nullptr)
      throw std::invalid_argument("sfq_linear_prepare: null argument");
    sc::Workspace ws;
    ws.adopt(d_workspace, workspace_bytes);
    const sc::QuantWeight qw = sfq_capi::weight_from_c(w);
    *d_prepared = r->runner.prepare(qw, ws);
    if (sc::is_packed_int8(qw.format)) *d_prepared = r->runner.prepared_codes();
    // Bytes from the caller's pointer to the end of what was carved (alignment skip included).
    const size_t skip = size_t(static_cast<const uint8_t*>(ws.base()) - static_cast<const uint8_t*>(d_workspace));
    *consumed_bytes = ws.used() == 0 ? 0 : skip + ws.used();
  });
}

int sfq_linear_forward_prepared(sfq_runner* r, const sfq_quant_weight* w, const void* d_prepared,
                                const void* d_x_bf16, int rows, void* d_y_bf16, void* d_workspace,
                                size_t workspace_bytes) {
  return guarded([&] {
    if (r == nullptr) throw std::invalid_argument("sfq: null runner");
    const sc::QuantWeight qw = sfq_capi::weight_from_c(w);
    sc::Workspace ws;
    ws.adopt(d_workspace, workspace_bytes);
    if (sc::is_packed_int8(qw.format) && d_prepared != nullptr) {
      // The expansion carved by sfq_linear_prepare: run the int8 arm against it directly.
      r->runner.forward_with_codes(qw, static_cast<const int8_t*>(d_prepared), static_cast<const bf16*>(d_x_bf16),
                                   rows, static_cast<bf16*>(d_y_bf16), ws);
      return;
    }
    r->runner.forward_prepared(qw, static_cast<const bf16*>(d_prepared), static_cast<const bf16*>(d_x_bf16), rows,
                               static_cast<bf16*>(d_y_bf16), ws);
  });
}

int sfq_linear_forward_f32(sfq_runner* r, const sfq_quant_weight* w, const float* d_x_f32, int rows, float* d_y_f32, void* d_workspace,
                           size_t workspace_bytes) {
  return guarded([&] {
    if (r == nullptr) throw std::invalid_argument("sfq: null runner");
    const sc::QuantWeight qw = sfq_capi::weight_from_c(w);
    sc::Workspace ws;
    ws.adopt(d_workspace, workspace_bytes);
    r->runner.forward_f32(qw, d_x_f32, rows, d_y_f32, ws);
  });
}
int sfq_adaln_expand(const float* d_w, const float* d_bias, const float* d_code, float* d_out, int num_t, int num_modality,
                     int num_param, int channels, int rank, void* stream) {
  return guarded([&] {
    sc::launch_adaln_expand(d_w, d_bias, d_code, d_out, num_t, num_modality, num_param, channels, rank, static_cast<cudaStream_t>(stream));
  });
}
int sfq_lora_create(sfq_lora** out) {
  return guarded([&] {
    if (!out) throw std::invalid_argument("sfq_lora_create: null output");
    *out = new sfq_lora();
  });
}
void sfq_lora_destroy(sfq_lora* l) { delete l; }
static slopfab::LoraFactors lora_factors(const float* a, const float* b, int rank, int in, int out_total) {
  if (!a || !b || rank <= 0 || in <= 0 || out_total <= 0) throw std::invalid_argument("sfq_lora_attach: bad factor arguments");
  slopfab::LoraFactors f;
  f.rank = rank, f.in = in, f.out = out_total;
  f.a.assign(a, a + size_t(rank) * in);
  f.b.assign(b, b + size_t(out_total) * rank);
  return f;
}
int sfq_lora_attach(sfq_lora* l, const void* key, const float* a, const float* b, int rank, int in_features, int out_total,
                    int row_offset, int out) {
  return guarded([&] {
    if (!l) throw std::invalid_argument("sfq_lora_attach: null runner");
    l->runner.attach(key, {lora_factors(a, b, rank, in_features, out_total)}, row_offset, out);
  });
}
int sfq_lora_attach_staged(sfq_lora* l, const void* key, const float* a, const float* b, int rank, int in_features, int out_total,
                           int row_offset, int out, uint8_t* staged_host, uint8_t* staged_device, size_t* staged_offset) {
  return guarded([&] {
    if (!l) throw std::invalid_argument("sfq_lora_attach_staged: null runner");
    l->runner.attach(key, {lora_factors(a, b, rank, in_features, out_total)}, row_offset, out, staged_host, staged_device, staged_offset);
  });
}
int sfq_lora_apply(sfq_lora* l, const void* key, const void* d_x_bf16, int rows, void* d_y_bf16, void* stream) {
  return guarded([&] {
    if (!l) throw std::invalid_argument("sfq_lora_apply: null runner");
    l->runner.apply(key, static_cast<const __nv_bfloat16*>(d_x_bf16), rows, static_cast<__nv_bfloat16*>(d_y_bf16), nullptr,
                    static_cast<cudaStream_t>(stream), false);
  });
}
int sfq_lora_bytes(const sfq_lora* l, size_t* weight_bytes, size_t* scratch_bytes) {
  return guarded([&] {
    if (!l) throw std::invalid_argument("sfq_lora_bytes: null runner");
    if (weight_bytes) *weight_bytes = l->runner.weight_bytes();
    if (scratch_bytes) *scratch_bytes = l->runner.scratch_bytes();
  });
}

}  // extern "C"
