// C++ operator API of the B200 quantized-Linear library.
//
// Same names, fields, defaults, argument meaning and error behaviour as the
// reference's operator headers, so a caller of the reference's
// slopfab::cuda::LinearRunner compiles against this header instead:
//   QuantFormat / ComputeType / QuantWeight / LinearRunner / linear_*_bytes
//                                   include/slopfab/cuda/linear.cuh:49-242
//   Workspace                       include/slopfab/cuda/workspace.cuh:21-76
//   launch_* free functions         include/slopfab/cuda/linear.cuh:251-318,
//                                   include/slopfab/cuda/w4a8.cuh:12-36,
//                                   include/slopfab/cuda/nvfp4_gemm.cuh:71-113,
//                                   include/slopfab/cuda/nn_kernels.cuh:28-91
// Errors are C++ exceptions exactly where the reference throws them:
// std::invalid_argument / std::runtime_error for contract violations before a
// launch, and std::runtime_error carrying the CUDA error text after one.
// Everything is asynchronous on the runner's stream; nothing synchronises.
//
// Implemented by libsfq.so (slopfab_b200/csrc). The plain C ABI over the same
// code is include/sfq.h.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

struct cublasContext;
typedef struct cublasContext* cublasHandle_t;

#pragma GCC visibility push(default)
namespace slopfab::cuda {

enum class QuantFormat { kF32, kF16, kBF16, kF8E4M3, kI8, kNVFP4, kNF4, kW4A8, kW6A8 };

inline bool is_packed_int8(QuantFormat format) {
  return format == QuantFormat::kW4A8 || format == QuantFormat::kW6A8;
}

constexpr int kNVFP4BlockSize = 16;

enum class ComputeType { kBF16, kF32 };

struct QuantWeight {
  QuantFormat format = QuantFormat::kBF16;
  const void* data = nullptr;
  int out_features = 0;
  int in_features = 0;
  const float* weight_scale = nullptr;
  bool per_channel_scale = false;
  float input_scale = 0.0f;
  bool full_precision = false;
  const uint8_t* block_scale = nullptr;
  uint32_t packed_group_size = 16;
  const float* w4_codebook = nullptr;
  float global_scale = 1.0f;
  const __nv_bfloat16* pre_quant_scale = nullptr;
  const uint8_t* nf4_absmax = nullptr;
  const float* nf4_quant_map = nullptr;
  const float* nf4_nested_quant_map = nullptr;
  const float* nf4_nested_absmax = nullptr;
  int nf4_block_size = 64;
  int nf4_nested_block_size = 256;
  float nf4_nested_offset = 0.0f;
  bool convrot = false;
  int convrot_group = 256;
  const void* bias = nullptr;
  QuantFormat bias_format = QuantFormat::kF32;

  bool has_bias() const { return bias != nullptr; }
  size_t stored_bytes() const;
};

// A growable device scratch arena with stack-like carving (256-byte grain). `adopt` wraps
// caller-owned memory instead of allocating (used by the C ABI).
class Workspace {
public:
  Workspace() = default;
  ~Workspace();
  Workspace(const Workspace&) = delete;
  Workspace& operator=(const Workspace&) = delete;

  void reserve(size_t bytes);
  void resize(size_t bytes);
  void adopt(void* device_memory, size_t bytes);
  void* alloc(size_t bytes);
  template <typename T> T* alloc_n(size_t count) { return static_cast<T*>(alloc(count * sizeof(T))); }
  void clear() { rewind(0); }
  size_t capacity() const { return capacity_; }
  size_t used() const { return cursor_; }
  const void* base() const { return base_; }

  // Extension (not in the reference): lets a holder of carved bytes learn that they were given back. protect(end)
  // says "the bytes below `end` are in use"; epoch() changes (to a value no Workspace has had before) whenever the
  // cursor later drops below a protected mark, and on every resize / adopt. LinearRunner keeps the W4A8/W6A8
  // expansion of prepare() under this guard.
  void protect(size_t end) {
    if (end > guard_) guard_ = end;
  }
  uint64_t epoch() const { return epoch_; }

  class Scope {
  public:
    explicit Scope(Workspace& w) : ws_(w), mark_(w.cursor_) {}
    ~Scope() { ws_.rewind(mark_); }
    Scope(const Scope&) = delete;
    Scope& operator=(const Scope&) = delete;

  private:
    Workspace& ws_;
    size_t mark_;
  };

private:
  static uint64_t next_epoch();
  void rewind(size_t mark) {
    if (mark < guard_) {
      guard_ = 0;
      epoch_ = next_epoch();
    }
    cursor_ = mark;
  }

  uint8_t* base_ = nullptr;
  size_t capacity_ = 0;
  size_t cursor_ = 0;
  bool owned_ = false;
  size_t guard_ = 0;
  uint64_t epoch_ = next_epoch();
};

size_t linear_workspace_bytes(const QuantWeight& w, int rows, ComputeType compute);
size_t linear_dense_weight_bytes(const QuantWeight& w);
size_t linear_activation_workspace_bytes(const QuantWeight& w, int rows, ComputeType compute);

class LinearRunner {
public:
  LinearRunner() = default;
  ~LinearRunner();
  LinearRunner(const LinearRunner&) = delete;
  LinearRunner& operator=(const LinearRunner&) = delete;

  // The handle is accepted for source compatibility and never used: no library GEMM is on this path.
  void init(cublasHandle_t handle, cudaStream_t stream);
  void set_native(bool enable) { native_ = enable; }
  bool native() const { return native_; }
  // Extension: activation fused into the GEMM epilogue (sfq_activation). Default none. With SFQ_ACT_SWIGLU the weight's
  // rows are [gate | up] and y is [rows, out_features / 2].
  void set_activation(int activation) { activation_ = activation; }

  void forward(const QuantWeight& w, const __nv_bfloat16* x, int rows, __nv_bfloat16* y, Workspace& ws);
  const __nv_bfloat16* prepare(const QuantWeight& w, Workspace& ws);
  void forward_prepared(const QuantWeight& w, const __nv_bfloat16* dense_w, const __nv_bfloat16* x, int rows,
                        __nv_bfloat16* y, Workspace& ws);
  void forward_f32(const QuantWeight& w, const float* x, int rows, float* y, Workspace& ws);

  // Extensions used by the C ABI for W4A8/W6A8: the int8 expansion the last prepare() carved, and a
  // forward that runs against an expansion the caller holds.
  const int8_t* prepared_codes() const { return cached_codes_; }
  void forward_with_codes(const QuantWeight& w, const int8_t* codes, const __nv_bfloat16* x, int rows,
                          __nv_bfloat16* y, Workspace& ws);

private:
  bool takes_native_nvfp4(const QuantWeight& w) const;
  bool cached_valid(const QuantWeight& w, const Workspace& ws) const;
  const int8_t* expanded_weight(const QuantWeight& w, Workspace& ws, bool keep, cudaStream_t stream);
  void run_packed_int8(const QuantWeight& w, const int8_t* codes, const __nv_bfloat16* x, int rows, __nv_bfloat16* y,
                       Workspace& ws, cudaEvent_t codes_ready);
  void ensure_side_stream();

  cudaStream_t stream_ = nullptr;
  bool initialised_ = false;
  bool native_ = false;
  bool native_nvfp4_device_ = false;
  int activation_ = 0;
  // W4A8/W6A8: expansion kept by prepare() for the chunk loop that follows (same weight, same arena).
  const void* cached_key_ = nullptr;
  const int8_t* cached_codes_ = nullptr;
  const void* cached_arena_ = nullptr;
  size_t cached_end_ = 0;
  uint64_t cached_epoch_ = 0;
  // A plain forward() of a W4A8/W6A8 layer expands the weight on this second stream while the activation is
  // quantized on the caller's; the GEMM waits for both. Created on first use.
  cudaStream_t side_ = nullptr;
  cudaEvent_t fork_ = nullptr;
  cudaEvent_t join_ = nullptr;
};

// ---- free launchers, reference names ------------------------------------------------------
void launch_convrot(const __nv_bfloat16* in, __nv_bfloat16* out, int rows, int dim, int group, cudaStream_t stream);
void launch_dequant_i8_per_channel(const int8_t* src, const float* scale, __nv_bfloat16* dst, int out_features,
                                   int in_features, cudaStream_t stream);
void launch_dequant_f8e4m3(const uint8_t* src, const float* scale, __nv_bfloat16* dst, size_t n, cudaStream_t stream);
void launch_dequant_nf4(const uint8_t* src, const uint8_t* absmax, const float* quant_map, const float* nested_quant_map,
                        const float* nested_absmax, int block_size, int nested_block_size, float nested_offset,
                        __nv_bfloat16* dst, int out_features, int in_features, cudaStream_t stream);
void launch_pre_quant_scale(const __nv_bfloat16* src, const __nv_bfloat16* scale, __nv_bfloat16* dst, int rows, int dim,
                            cudaStream_t stream);
void launch_dequant_nvfp4(const uint8_t* src, const uint8_t* block_scale, float global_scale, __nv_bfloat16* dst,
                          int out_features, int in_features, cudaStream_t stream);
void launch_dequant_w6a8_weight(const int8_t* packed, const uint8_t* group_scale, int8_t* output, int out_features,
                                int in_features, int group_size, cudaStream_t stream);
void launch_dequant_w4a8_weight(const int8_t* packed, const uint8_t* group_scale, const float* codebook,
                                int8_t* output, int out_features, int in_features, int group_size,
                                cudaStream_t stream);
void launch_quantize_w4a8_bf16(const __nv_bfloat16* rotated, int8_t* output, float* row_scale, int rows, int width,
                               cudaStream_t stream);
bool nvfp4_gemm_supported(int out_features, int in_features);
bool nvfp4_gemm_shape_supported(int out_features, int in_features) noexcept;
size_t nvfp4_gemm_workspace_bytes(int rows, int in_features);
void launch_quantize_nvfp4_activations(const __nv_bfloat16* x, uint8_t* packed, uint8_t* scales, int rows, int dim,
                                       cudaStream_t stream);
// nvfp4_gemm_forward / _prevalidated / _q (include/slopfab/cuda/nvfp4_gemm.cuh:89-113): y = x W^T * global_scale with fp4
// activations, no bias. The first two quantize x into `ws` (straight into the layout the tcgen05 GEMM reads) and throw
// like the reference when the device or the shape has no native path (`_prevalidated` skips that test). `_q` takes
// activations the caller quantized with launch_quantize_nvfp4_activations, i.e. in the REFERENCE's layout; it converts
// them (nibbles exchanged, scales tiled) into stream-ordered scratch it allocates and frees on `stream`, because the
// reference signature carries no workspace. A caller that shares one quantization between several GEMMs and cares
// about that allocation uses sfq_quantize_nvfp4_block(GEMM_FEED) + sfq_gemm_nvfp4 instead.
void nvfp4_gemm_forward(const __nv_bfloat16* x, const uint8_t* w_packed, const uint8_t* w_scale, float global_scale,
                        __nv_bfloat16* y, int rows, int out_features, int in_features, Workspace& ws, cudaStream_t stream);
void nvfp4_gemm_forward_prevalidated(const __nv_bfloat16* x, const uint8_t* w_packed, const uint8_t* w_scale,
                                     float global_scale, __nv_bfloat16* y, int rows, int out_features, int in_features,
                                     Workspace& ws, cudaStream_t stream);
void nvfp4_gemm_forward_q(const uint8_t* xq, const uint8_t* xs, const uint8_t* w_packed, const uint8_t* w_scale,
                          float global_scale, __nv_bfloat16* y, int rows, int out_features, int in_features,
                          cudaStream_t stream);
// include/slopfab/cuda/w4a8.cuh:30-36: the int32 accumulator of an int8 GEMM scaled to bf16, or to fp32 in place. (The
// runner never materialises that accumulator: its GEMM epilogue applies the same arithmetic.)
void launch_w4a8_output_bf16(const int32_t* input, const float* row_scale, const float* channel_scale, __nv_bfloat16* output,
                             int rows, int cols, cudaStream_t stream);
void launch_dequant_w4a8_output(int32_t* input_output, const float* activation_scale, const float* weight_scale, int rows,
                                int cols, cudaStream_t stream);
// include/slopfab/cuda/linear.cuh:253-313.
void launch_convrot_f32(const float* in, float* out, int rows, int dim, int group, cudaStream_t stream);
void launch_dequant_nf4_f16(const uint8_t* src, const uint8_t* absmax, const float* quant_map, const float* nested_quant_map,
                            const float* nested_absmax, int block_size, int nested_block_size, float nested_offset,
                            __half* dst, size_t n, cudaStream_t stream);
void launch_quantize_f8e4m3(const __nv_bfloat16* src, float input_scale, uint8_t* dst, size_t n, cudaStream_t stream);
void launch_widen_bf16(const __nv_bfloat16* src, float* dst, size_t n, cudaStream_t stream);
void launch_narrow_to_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t stream);
void launch_rmsnorm(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* out, int rows, int dim, float eps,
                    cudaStream_t stream);
void launch_rmsnorm_modulate(const __nv_bfloat16* x, const __nv_bfloat16* w, const float* scale, const float* shift,
                             const int32_t* a, __nv_bfloat16* out, int rows, int dim, float eps, cudaStream_t stream);
void launch_add_gated(__nv_bfloat16* x, const __nv_bfloat16* branch, const float* gate, const int32_t* a, int rows,
                      int dim, cudaStream_t stream);
void launch_swiglu(const __nv_bfloat16* fused, __nv_bfloat16* out, int rows, int inner, cudaStream_t stream);
void launch_gelu_tanh(__nv_bfloat16* x, size_t n, cudaStream_t stream);
// QK-norm over the head dimension and MM-RoPE (include/slopfab/cuda/nn_kernels.cuh:95-134), head_dim 128, contiguous
// [rows, heads, 128] as in the reference; sfq_head_norm_rope does both in one pass and takes a row pitch.
void launch_head_rmsnorm(__nv_bfloat16* x, const __nv_bfloat16* w, int rows, int heads, int dim, float eps, cudaStream_t stream);
void launch_rope_h3(__nv_bfloat16* x, const float* cos, const float* sin, int rows, int heads, int head_dim, cudaStream_t stream);
// adaLN table expansion (src/dit/transformer_support.h:58, src/cuda/dit_kernels.cu:108-134): fp32 fma chain from the
// bias, out[param][timestep][modality][channel]. Same checks and messages as the reference.
void launch_adaln_expand(const float* w, const float* bias, const float* code, float* out, int num_t, int num_modality,
                         int num_param, int channels, int rank, cudaStream_t stream);

}  // namespace slopfab::cuda
#pragma GCC visibility pop
