// C entry points over the reference's OWN code for the quantized-Linear path.
//
// TEST INFRASTRUCTURE ONLY. This file contains no arithmetic of its own: it
// includes the reference's headers and test fixtures where they lie in the
// reference tree and forwards to them, so that Python tests can run the
// reference's host fixtures on the CPU and the reference's CUDA kernels /
// LinearRunner on a GPU, on the same buffers as the new kernels. It is
// compiled, together with the reference's unmodified sources, into
// oracle/_ref/libslopfab_ref.so by oracle/Makefile. The product never loads it.
//
// Every function returns 0 on success and -1 after recording the exception
// text (ref_last_error). Device pointers are plain device addresses; all device
// entry points run on the default stream and synchronise before returning.

#include "tests/detail/nn_weight_fixture.h"  // includes nn_kernels_fixture.h, dtype.h, the cuda headers

#include <cstring>
#include <string>

#include "slopfab/int8_weight.h"

namespace {
thread_local std::string g_error;

template <class F> int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_error = e.what();
    return -1;
  } catch (...) {
    g_error = "unknown exception";
    return -1;
  }
}

void sync() {
  SLOPFAB_CUDA_CHECK(cudaDeviceSynchronize());
}

using bf16 = __nv_bfloat16;
namespace sc = slopfab::cuda;
}  // namespace

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API const char* ref_last_error() { return g_error.c_str(); }

// ---------------------------------------------------------------------------
// Host fixtures (run anywhere)
// ---------------------------------------------------------------------------
REF_API void ref_make_data(float* out, size_t n, uint32_t seed, float scale) {
  const auto v = make_data(n, seed, scale);
  std::memcpy(out, v.data(), n * sizeof(float));
}
REF_API void ref_make_gaussian(float* out, size_t n, uint32_t seed, float sigma) {
  const auto v = make_gaussian(n, seed, sigma);
  std::memcpy(out, v.data(), n * sizeof(float));
}
REF_API uint16_t ref_f32_to_bf16(float f) { return slopfab::f32_to_bf16(f); }
REF_API uint16_t ref_f32_to_f16(float f) { return slopfab::f32_to_f16(f); }
REF_API float ref_f16_to_f32(uint16_t h) { return slopfab::f16_to_f32(h); }
REF_API float ref_e4m3_to_f32(uint8_t v) { return slopfab::f8_e4m3_to_f32(v); }
REF_API float ref_e2m1_to_f32(uint8_t v) { return slopfab::f4_e2m1_to_f32(v); }
REF_API uint8_t ref_host_e4m3(float v) { return host_e4m3(v); }
REF_API uint8_t ref_host_e2m1(float v) { return host_e2m1(v); }
REF_API uint64_t ref_nvfp4_scale_slot(int o, int k, int blocks_per_row) {
  return nvfp4_scale_slot(o, k, blocks_per_row);
}

// make_nvfp4(out, in, global, seed): random codes/scales in storage form.
REF_API void ref_make_nvfp4(int out_features, int in_features, float global, uint32_t seed,
                            uint8_t* packed, uint8_t* stored_scales, uint8_t* plain_scales,
                            float* reference_bf16_values) {
  const Nvfp4Weight w = make_nvfp4(out_features, in_features, global, seed);
  std::memcpy(packed, w.packed.data(), w.packed.size());
  std::memcpy(stored_scales, w.stored.data(), w.stored.size());
  if (plain_scales) std::memcpy(plain_scales, w.scales.data(), w.scales.size());
  if (reference_bf16_values) {
    const auto r = nvfp4_reference(w);
    std::memcpy(reference_bf16_values, r.data(), r.size() * sizeof(float));
  }
}

REF_API void ref_pack_nvfp4(const float* w, int rows, int cols, float global, int high_even,
                            int swizzled, uint8_t* data, uint8_t* scale, float* dense) {
  const std::vector<float> in(w, w + size_t(rows) * cols);
  const NvfpPacked p = pack_nvfp4(in, rows, cols, global, high_even != 0, swizzled != 0);
  std::memcpy(data, p.data.data(), p.data.size());
  std::memcpy(scale, p.scale.data(), p.scale.size());
  if (dense) std::memcpy(dense, p.dense.data(), p.dense.size() * sizeof(float));
}

REF_API void ref_host_quantise_act(const float* x, int rows, int dim, float* out) {
  const std::vector<float> in(x, x + size_t(rows) * dim);
  const auto q = host_quantise_act(in, rows, dim);
  std::memcpy(out, q.data(), q.size() * sizeof(float));
}

REF_API void ref_cpu_matmul_nt(const float* A, const float* B, int M, int N, int K, float* C) {
  const std::vector<float> a(A, A + size_t(M) * K), b(B, B + size_t(N) * K);
  const auto c = cpu_matmul_nt(a, b, M, N, K);
  std::memcpy(C, c.data(), c.size() * sizeof(float));
}

REF_API void ref_cpu_rmsnorm(const float* x, const float* w, const float* scale, const float* shift,
                             const int32_t* a, int rows, int dim, float eps, float* out) {
  const std::vector<float> xv(x, x + size_t(rows) * dim), wv(w, w + dim);
  std::vector<float> r;
  if (scale) {
    int amax = 0;
    for (int i = 0; i < rows; ++i) amax = std::max(amax, a[i]);
    const std::vector<float> sc(scale, scale + size_t(amax + 1) * dim), sh(shift, shift + size_t(amax + 1) * dim);
    const std::vector<int32_t> av(a, a + rows);
    r = cpu_modulate(xv, wv, sc, sh, av, rows, dim, eps, true);
  } else {
    r = cpu_rmsnorm(xv, wv, rows, dim, eps);
  }
  std::memcpy(out, r.data(), r.size() * sizeof(float));
}

REF_API void ref_kron_h4_256(float* out) {  // kron^4(h4), unnormalised, 256x256
  const auto h = kron_power(&kH4[0][0], 4, 4);
  std::memcpy(out, h.data(), h.size() * sizeof(float));
}

REF_API void ref_unpack_int8_weight(const int8_t* codes, const float* scales, int rows, int cols,
                                    int group, int canonicalize, uint16_t* out) {
  slopfab::Int8WeightState s;
  s.rows = rows;
  s.columns = cols;
  s.rotation_group = group;
  s.codes = codes;
  s.scales = scales;
  const auto v = slopfab::unpack_int8_weight(s, canonicalize != 0);
  std::memcpy(out, v.data(), v.size() * sizeof(uint16_t));
}

// ---------------------------------------------------------------------------
// Device kernels of the reference (need a GPU)
// ---------------------------------------------------------------------------
REF_API int ref_dev_dequant_nvfp4(const uint8_t* src, const uint8_t* scale, float global, void* dst,
                                  int out_features, int in_features) {
  return guarded([&] {
    sc::launch_dequant_nvfp4(src, scale, global, static_cast<bf16*>(dst), out_features, in_features, nullptr);
    sync();
  });
}
REF_API int ref_dev_dequant_f8(const uint8_t* src, const float* scale, void* dst, size_t n) {
  return guarded([&] {
    sc::launch_dequant_f8e4m3(src, scale, static_cast<bf16*>(dst), n, nullptr);
    sync();
  });
}
REF_API int ref_dev_dequant_nf4(const uint8_t* src, const uint8_t* absmax, const float* map, const float* nested_map,
                                const float* nested_absmax, int block, int nested_block, float offset, void* dst,
                                int out_features, int in_features) {
  return guarded([&] {
    sc::launch_dequant_nf4(src, absmax, map, nested_map, nested_absmax, block, nested_block, offset,
                           static_cast<bf16*>(dst), out_features, in_features, nullptr);
    sync();
  });
}
REF_API int ref_dev_pre_quant_scale(const void* src, const void* scale, void* dst, int rows, int dim) {
  return guarded([&] {
    sc::launch_pre_quant_scale(static_cast<const bf16*>(src), static_cast<const bf16*>(scale), static_cast<bf16*>(dst),
                               rows, dim, nullptr);
    sync();
  });
}
REF_API int ref_dev_dequant_i8(const int8_t* src, const float* scale, void* dst, int out_features,
                               int in_features) {
  return guarded([&] {
    sc::launch_dequant_i8_per_channel(src, scale, static_cast<bf16*>(dst), out_features, in_features, nullptr);
    sync();
  });
}
REF_API int ref_dev_dequant_w4a8(const int8_t* packed, const uint8_t* gs, const float* codebook,
                                 int8_t* out, int out_features, int in_features, int group) {
  return guarded([&] {
    sc::launch_dequant_w4a8_weight(packed, gs, codebook, out, out_features, in_features, group, nullptr);
    sync();
  });
}
REF_API int ref_dev_dequant_w6a8(const int8_t* packed, const uint8_t* gs, int8_t* out, int out_features,
                                 int in_features, int group) {
  return guarded([&] {
    sc::launch_dequant_w6a8_weight(packed, gs, out, out_features, in_features, group, nullptr);
    sync();
  });
}
REF_API int ref_dev_convrot(const void* in, void* out, int rows, int dim, int group) {
  return guarded([&] {
    sc::launch_convrot(static_cast<const bf16*>(in), static_cast<bf16*>(out), rows, dim, group, nullptr);
    sync();
  });
}
REF_API int ref_dev_quantize_int8_bf16(const void* rotated, int8_t* q, float* scales, int rows, int width) {
  return guarded([&] {
    sc::launch_quantize_w4a8_bf16(static_cast<const bf16*>(rotated), q, scales, rows, width, nullptr);
    sync();
  });
}
REF_API int ref_dev_quantize_int8_f16(const void* x, int8_t* q, float* scales, int rows, int width) {
  return guarded([&] {
    sc::launch_quantize_w4a8_activation(static_cast<const __half*>(x), q, scales, rows, width, nullptr);
    sync();
  });
}
REF_API int ref_dev_output_bf16(const int32_t* acc, const float* rows_s, const float* chan_s, void* y,
                                int rows, int cols) {
  return guarded([&] {
    sc::launch_w4a8_output_bf16(acc, rows_s, chan_s, static_cast<bf16*>(y), rows, cols, nullptr);
    sync();
  });
}
REF_API int ref_dev_quantize_nvfp4_act(const void* x, uint8_t* packed, uint8_t* scales, int rows, int dim) {
  return guarded([&] {
    sc::launch_quantize_nvfp4_activations(static_cast<const bf16*>(x), packed, scales, rows, dim, nullptr);
    sync();
  });
}
REF_API int ref_dev_rmsnorm(const void* x, const void* w, const float* scale, const float* shift,
                            const int32_t* a, void* out, int rows, int dim, float eps) {
  return guarded([&] {
    if (scale)
      sc::launch_rmsnorm_modulate(static_cast<const bf16*>(x), static_cast<const bf16*>(w), scale, shift, a,
                                  static_cast<bf16*>(out), rows, dim, eps, nullptr);
    else
      sc::launch_rmsnorm(static_cast<const bf16*>(x), static_cast<const bf16*>(w), static_cast<bf16*>(out),
                         rows, dim, eps, nullptr);
    sync();
  });
}
REF_API int ref_dev_gelu_tanh(void* x, size_t n) {
  return guarded([&] {
    sc::launch_gelu_tanh(static_cast<bf16*>(x), n, nullptr);
    sync();
  });
}
REF_API int ref_dev_swiglu(const void* fused, void* out, int rows, int inner) {
  return guarded([&] {
    sc::launch_swiglu(static_cast<const bf16*>(fused), static_cast<bf16*>(out), rows, inner, nullptr);
    sync();
  });
}
REF_API int ref_dev_add_gated(void* x, const void* branch, const float* gate, const int32_t* a, int rows,
                              int dim) {
  return guarded([&] {
    sc::launch_add_gated(static_cast<bf16*>(x), static_cast<const bf16*>(branch), gate, a, rows, dim, nullptr);
    sync();
  });
}

// ---------------------------------------------------------------------------
// LinearRunner of the reference
// ---------------------------------------------------------------------------
struct RefWeight {  // plain mirror of the fields the path uses
  int format;       // QuantFormat as int
  const void* data;
  int out_features, in_features;
  const float* weight_scale;
  int per_channel_scale;
  const uint8_t* block_scale;
  uint32_t packed_group_size;
  const float* w4_codebook;
  float global_scale;
  int convrot, convrot_group;
  const void* bias;
  int bias_format;
  const void* pre_quant_scale;
  const uint8_t* nf4_absmax;
  const float* nf4_quant_map;
  const float* nf4_nested_quant_map;
  const float* nf4_nested_absmax;
  int nf4_block_size, nf4_nested_block_size;
  float nf4_nested_offset;
};

namespace {
sc::QuantWeight to_weight(const RefWeight& r) {
  sc::QuantWeight w;
  w.format = static_cast<sc::QuantFormat>(r.format);
  w.data = r.data;
  w.out_features = r.out_features;
  w.in_features = r.in_features;
  w.weight_scale = r.weight_scale;
  w.per_channel_scale = r.per_channel_scale != 0;
  w.block_scale = r.block_scale;
  w.packed_group_size = r.packed_group_size;
  w.w4_codebook = r.w4_codebook;
  w.global_scale = r.global_scale;
  w.convrot = r.convrot != 0;
  w.convrot_group = r.convrot_group;
  w.bias = r.bias;
  w.bias_format = static_cast<sc::QuantFormat>(r.bias_format);
  w.pre_quant_scale = static_cast<const bf16*>(r.pre_quant_scale);
  w.nf4_absmax = r.nf4_absmax;
  w.nf4_quant_map = r.nf4_quant_map;
  w.nf4_nested_quant_map = r.nf4_nested_quant_map;
  w.nf4_nested_absmax = r.nf4_nested_absmax;
  if (r.nf4_block_size > 0) w.nf4_block_size = r.nf4_block_size;
  if (r.nf4_nested_block_size > 0) w.nf4_nested_block_size = r.nf4_nested_block_size;
  w.nf4_nested_offset = r.nf4_nested_offset;
  return w;
}

struct Runner {
  CublasScope blas;
  sc::LinearRunner runner;
  Workspace ws;
  Runner() { runner.init(blas.h, nullptr); }
};
Runner& runner() {
  static Runner r;
  return r;
}
}  // namespace

// y = LinearRunner::forward(w, x). `iters` > 0 additionally times that many
// repeats with CUDA events after 3 warm-ups and stores the mean milliseconds.
REF_API int ref_dev_linear_forward(const RefWeight* rw, const void* x, int rows, void* y, int native,
                                   int iters, float* mean_ms) {
  return guarded([&] {
    Runner& r = runner();
    const sc::QuantWeight w = to_weight(*rw);
    r.runner.set_native(native != 0);
    r.ws.reserve(sc::linear_workspace_bytes(w, rows, sc::ComputeType::kBF16) + 4096);
    r.runner.forward(w, static_cast<const bf16*>(x), rows, static_cast<bf16*>(y), r.ws);
    sync();
    if (iters > 0) {
      for (int i = 0; i < 3; ++i)
        r.runner.forward(w, static_cast<const bf16*>(x), rows, static_cast<bf16*>(y), r.ws);
      cudaEvent_t a, b;
      SLOPFAB_CUDA_CHECK(cudaEventCreate(&a));
      SLOPFAB_CUDA_CHECK(cudaEventCreate(&b));
      SLOPFAB_CUDA_CHECK(cudaEventRecord(a, nullptr));
      for (int i = 0; i < iters; ++i)
        r.runner.forward(w, static_cast<const bf16*>(x), rows, static_cast<bf16*>(y), r.ws);
      SLOPFAB_CUDA_CHECK(cudaEventRecord(b, nullptr));
      SLOPFAB_CUDA_CHECK(cudaEventSynchronize(b));
      float ms = 0;
      SLOPFAB_CUDA_CHECK(cudaEventElapsedTime(&ms, a, b));
      cudaEventDestroy(a);
      cudaEventDestroy(b);
      if (mean_ms) *mean_ms = ms / float(iters);
    }
  });
}

// The int32 accumulators of the packed-int8 arm, produced by the same calls
// LinearRunner::forward_prepared makes (src/cuda/linear.cu:188-203), stopping
// before the output scaling. All buffers are caller-provided device memory.
REF_API int ref_dev_packed_int8_accumulate(const RefWeight* rw, const void* x, int rows, int8_t* codes,
                                           void* rotated, int8_t* activation, float* scales,
                                           int32_t* accum) {
  return guarded([&] {
    Runner& r = runner();
    const sc::QuantWeight w = to_weight(*rw);
    if (w.format == sc::QuantFormat::kW6A8)
      sc::launch_dequant_w6a8_weight(static_cast<const int8_t*>(w.data), w.block_scale, codes,
                                     w.out_features, w.in_features, w.packed_group_size, nullptr);
    else
      sc::launch_dequant_w4a8_weight(static_cast<const int8_t*>(w.data), w.block_scale, w.w4_codebook, codes,
                                     w.out_features, w.in_features, 16, nullptr);
    sc::launch_convrot(static_cast<const bf16*>(x), static_cast<bf16*>(rotated), rows, w.in_features, 256,
                       nullptr);
    sc::launch_quantize_w4a8_bf16(static_cast<const bf16*>(rotated), activation, scales, rows, w.in_features,
                                  nullptr);
    const int32_t one = 1, zero = 0;
    SLOPFAB_CUBLAS_CHECK(sc::cublas_gemm_ex(r.blas.h, CUBLAS_OP_T, CUBLAS_OP_N, w.out_features, rows,
                                            w.in_features, &one, codes, CUDA_R_8I, w.in_features, activation,
                                            CUDA_R_8I, w.in_features, &zero, accum, CUDA_R_32I,
                                            w.out_features, CUBLAS_COMPUTE_32I, CUBLAS_GEMM_DEFAULT));
    sync();
  });
}

// ---- the reference's safetensors reader and format detectors (src/core/safetensors.cpp, w4a8.cpp, nf4.cpp) ----
#include "slopfab/nf4.h"
#include "slopfab/safetensors.h"
#include "slopfab/w4a8.h"

REF_API int ref_st_open(const char* path, void** handle) {
  return guarded([&] {
    auto* st = new slopfab::SafeTensors();
    try {
      st->open(path);
    } catch (...) {
      delete st;
      throw;
    }
    *handle = st;
  });
}
REF_API void ref_st_close(void* handle) { delete static_cast<slopfab::SafeTensors*>(handle); }
// dtype as the reference's DType enumerator value; data pointer into the reference's own mapping.
REF_API int ref_st_find(void* handle, const char* name, int* dtype, int* rank, int64_t* shape8, const void** data,
                        size_t* nbytes) {
  return guarded([&] {
    const slopfab::TensorView& v = static_cast<slopfab::SafeTensors*>(handle)->at(name);
    *dtype = int(v.dtype);
    *rank = int(v.shape.size());
    for (size_t i = 0; i < v.shape.size() && i < 8; ++i) shape8[i] = v.shape[i];
    *data = v.data;
    *nbytes = v.nbytes;
  });
}
REF_API int ref_st_is_packed_int8(void* handle, const char* weight_name, int* yes) {
  return guarded([&] { *yes = slopfab::is_packed_int8_weight(*static_cast<slopfab::SafeTensors*>(handle), weight_name) ? 1 : 0; });
}
REF_API int ref_st_packed_state(void* handle, const char* weight_name, int* bits, int* group, int* rotation) {
  return guarded([&] {
    const auto s = slopfab::read_packed_int8_state(*static_cast<slopfab::SafeTensors*>(handle), weight_name, "test");
    *bits = s.bits;
    *group = s.group_size;
    *rotation = s.convrot_group_size;
  });
}
REF_API int ref_st_is_nf4(void* handle, const char* weight_name, int* yes) {
  return guarded([&] { *yes = slopfab::is_nf4_weight(*static_cast<slopfab::SafeTensors*>(handle), weight_name) ? 1 : 0; });
}
REF_API int ref_st_nf4_state(void* handle, const char* weight_name, int* block, int* nested, float* offset) {
  return guarded([&] {
    const auto s = slopfab::read_nf4_state(*static_cast<slopfab::SafeTensors*>(handle), weight_name, "test", true);
    *block = s.block_size;
    *nested = s.nested_block_size;
    *offset = s.nested_offset;
  });
}

// ---- LoRA side branch (src/cuda/lora.cu): the reference's runner, deterministic or cuBLAS arm
#include "slopfab/cuda/lora.cuh"
REF_API int ref_lora_apply(const float* a, const float* b, int rank, int in, int out_total, int offset, int out,
                           const void* d_x, int rows, void* d_y, int exact) {
  return guarded([&] {
    slopfab::LoraFactors f;
    f.rank = rank, f.in = in, f.out = out_total;
    f.a.assign(a, a + size_t(rank) * in);
    f.b.assign(b, b + size_t(out_total) * rank);
    sc::LoraRunner runner;
    runner.attach(&f, {f}, offset, out);
    cublasHandle_t blas = nullptr;
    SLOPFAB_CUBLAS_CHECK(sc::cublas_create(&blas));
    runner.apply(&f, static_cast<const bf16*>(d_x), rows, static_cast<bf16*>(d_y), blas, nullptr, exact != 0);
    sync();
    SLOPFAB_CUBLAS_CHECK(sc::cublas_destroy(blas));
  });
}

// ---- fp32-compute arm and the adaLN table expansion, the reference's own code
namespace slopfab::cuda {
void launch_adaln_expand(const float* w, const float* bias, const float* code, float* out, int num_t, int num_modality,
                         int num_param, int channels, int rank, cudaStream_t stream);  // src/dit/transformer_support.h:58
}
REF_API int ref_dev_linear_forward_f32(const RefWeight* rw, const float* x, int rows, float* y) {
  return guarded([&] {
    Runner& r = runner();
    const sc::QuantWeight w = to_weight(*rw);
    r.ws.reserve(sc::linear_workspace_bytes(w, rows, sc::ComputeType::kF32) + 4096);
    r.runner.forward_f32(w, x, rows, y, r.ws);
    sync();
  });
}
REF_API int ref_dev_adaln_expand(const float* w, const float* bias, const float* code, float* out, int num_t, int num_modality,
                                 int num_param, int channels, int rank) {
  return guarded([&] {
    sc::launch_adaln_expand(w, bias, code, out, num_t, num_modality, num_param, channels, rank, nullptr);
    sync();
  });
}

// ---- QK-norm and MM-RoPE, the reference's two launches on a contiguous [rows, heads, dim] buffer
REF_API int ref_dev_head_norm_rope(void* x, const void* w, const float* cos_tab, const float* sin_tab, int rows, int heads, int dim,
                                   float eps) {
  return guarded([&] {
    if (w != nullptr) sc::launch_head_rmsnorm(static_cast<bf16*>(x), static_cast<const bf16*>(w), rows, heads, dim, eps, nullptr);
    if (cos_tab != nullptr) sc::launch_rope_h3(static_cast<bf16*>(x), cos_tab, sin_tab, rows, heads, dim, nullptr);
    sync();
  });
}

// ---- token packing (src/dit/packing.cpp): the reference's own build_indices / build_row_timesteps, host only.
// `tags_override` (may be null) replaces the tags build_indices produced, e.g. to mark padding rows with -1.
#include "slopfab/dit/packing.h"
namespace {
slopfab::dit::SequenceLayout make_layout(const int32_t* f) {
  slopfab::dit::SequenceLayout l;
  l.num_text = f[0];
  l.num_condition_video = f[1];
  l.num_condition_audio = f[2];
  l.condition_audio_is_explicit = f[3] != 0;
  l.num_audio_rows = f[4];
  l.num_video_rows = f[5];
  return l;
}
}  // namespace
REF_API int ref_build_indices(const int32_t* layout6, int32_t* text, int32_t* audio, int32_t* video, int32_t* tags) {
  return guarded([&] {
    const auto idx = slopfab::dit::build_indices(make_layout(layout6));
    std::memcpy(text, idx.text.data(), idx.text.size() * 4);
    std::memcpy(audio, idx.audio.data(), idx.audio.size() * 4);
    std::memcpy(video, idx.video.data(), idx.video.size() * 4);
    std::memcpy(tags, idx.tags.data(), idx.tags.size() * 4);
  });
}
// timesteps: 2 values {video, audio} or 4 values {video, audio, condition video, condition audio}.
REF_API int ref_build_row_timesteps(const int32_t* layout6, const int32_t* tags_override, const float* timesteps, int count,
                                    int32_t* indices, int32_t* adaln, float* unique, int* num_unique) {
  return guarded([&] {
    const auto l = make_layout(layout6);
    auto idx = slopfab::dit::build_indices(l);
    if (tags_override) idx.tags.assign(tags_override, tags_override + idx.tags.size());
    const auto rt = count == 4 ? slopfab::dit::build_row_timesteps(l, idx, timesteps[0], timesteps[1], timesteps[2], timesteps[3])
                               : slopfab::dit::build_row_timesteps(l, idx, timesteps[0], timesteps[1]);
    std::memcpy(indices, rt.indices.data(), rt.indices.size() * 4);
    std::memcpy(adaln, rt.adaln.data(), rt.adaln.size() * 4);
    std::memcpy(unique, rt.unique.data(), rt.unique.size() * 4);
    *num_unique = int(rt.unique.size());
  });
}

// ---- the remaining small launchers of the linear headers
REF_API int ref_dev_convrot_f32(const float* in, float* out, int rows, int dim, int group) {
  return guarded([&] {
    sc::launch_convrot_f32(in, out, rows, dim, group, nullptr);
    sync();
  });
}
REF_API int ref_dev_quantize_f8(const void* x, float input_scale, uint8_t* out, size_t n) {
  return guarded([&] {
    sc::launch_quantize_f8e4m3(static_cast<const bf16*>(x), input_scale, out, n, nullptr);
    sync();
  });
}
REF_API int ref_dev_dequant_nf4_f16(const uint8_t* src, const uint8_t* absmax, const float* map, const float* nested_map,
                                    const float* nested_absmax, int block, int nested_block, float offset, void* dst, size_t n) {
  return guarded([&] {
    sc::launch_dequant_nf4_f16(src, absmax, map, nested_map, nested_absmax, block, nested_block, offset, static_cast<__half*>(dst), n, nullptr);
    sync();
  });
}
REF_API int ref_dev_output_f32(int32_t* io, const float* rows_s, const float* chan_s, int rows, int cols) {
  return guarded([&] {
    sc::launch_dequant_w4a8_output(io, rows_s, chan_s, rows, cols, nullptr);
    sync();
  });
}
