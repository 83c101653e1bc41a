// slopfab::cuda::LinearRunner and friends for B200: the dispatch of
// src/cuda/linear.cu:113-249 re-targeted at this library's kernels.
//
//   W4A8 / W6A8   expand weight (once per prepare, or per call) -> fused ConvRot +
//                 per-token int8 -> tcgen05 int8 GEMM with the scale / bias epilogue
//                 (three launches instead of six, no int32 [M,N] round trip)
//   NVFP4 native  fused per-16 fp4 quantizer -> tcgen05 block-scaled GEMM
//   anything with a dense form, native off: unpack to bf16 -> [ConvRot] -> tcgen05 bf16 GEMM
//
// Validation, exception types and the null-pointer protocol of prepare /
// forward_prepared follow the reference; see the comments at each check.
#include "../../include/slopfab_b200/linear.hpp"

#include <algorithm>
#include <climits>
#include <atomic>
#include <stdexcept>
#include <string>

#include "gemm_tc.cuh"
#include "kernels.cuh"
#include "runtime.h"

namespace slopfab::cuda {
namespace {

inline size_t align_up(size_t n) { return (n + 255) / 256 * 256; }

inline bool convrot_applies(const QuantWeight& w) {
  return w.convrot && w.convrot_group > 0 && w.in_features % w.convrot_group == 0;
}

// The packed-int8 contract of src/cuda/linear.cu:179-187, same exception type and text.
void validate_packed_int8(const QuantWeight& w) {
  if (!w.block_scale || (w.format == QuantFormat::kW4A8 ? !w.w4_codebook : w.w4_codebook != nullptr) ||
      !w.weight_scale || !w.convrot || w.convrot_group != 256 || w.in_features % 256 || !w.packed_group_size ||
      w.in_features % w.packed_group_size ||
      (w.format == QuantFormat::kW4A8 ? w.packed_group_size != 16 : w.packed_group_size % 16 != 0) ||
      w.in_features > INT32_MAX / (128 * 127) || w.full_precision || w.pre_quant_scale)
    throw std::invalid_argument(
        "W4A8/W6A8 requires group scales, channel scales, compatible codebook and ConvRot-256");
}

bool has_dense_form(const QuantWeight& w) {
  switch (w.format) {
    case QuantFormat::kW4A8:
    case QuantFormat::kW6A8:
      return false;
    default:
      return true;
  }
}

[[noreturn]] void unsupported_format(const QuantWeight& w) {
  throw std::runtime_error("linear: unhandled weight format " + std::to_string(int(w.format)));
}

sfq::GemmArgs epilogue_for(const QuantWeight& w, int rows, __nv_bfloat16* y, int activation) {
  sfq::GemmArgs g;
  g.M = rows;
  g.N = w.out_features;
  g.K = w.in_features;
  g.y = y;
  g.ldy = w.out_features;
  if (w.has_bias()) {
    if (w.bias_format != QuantFormat::kF32 && w.bias_format != QuantFormat::kBF16)
      throw std::runtime_error("linear: unsupported bias format");
    g.bias = w.bias;
    g.bias_is_bf16 = w.bias_format == QuantFormat::kBF16;
  }
  g.act = activation;
  if (activation == SFQ_ACT_SWIGLU) g.ldy = w.out_features / 2;  // y is [rows, out_features / 2]
  g.status = sfq::device_status_word();
  return g;
}

}  // namespace

// ---- QuantWeight ---------------------------------------------------------------------------

size_t QuantWeight::stored_bytes() const {  // src/cuda/linear.cu:9-18
  const size_t n = size_t(out_features) * in_features;
  if (format == QuantFormat::kW6A8) return n * 3 / 4;
  if (format == QuantFormat::kNVFP4 || format == QuantFormat::kNF4 || format == QuantFormat::kW4A8) return (n + 1) / 2;
  switch (format) {
    case QuantFormat::kF32: return 4 * n;
    case QuantFormat::kF16:
    case QuantFormat::kBF16: return 2 * n;
    default: return n;
  }
}

// ---- Workspace -----------------------------------------------------------------------------

uint64_t Workspace::next_epoch() {
  static std::atomic<uint64_t> counter{0};
  return ++counter;
}

Workspace::~Workspace() {
  if (owned_ && base_) cudaFree(base_);
}

void Workspace::reserve(size_t bytes) {
  if (bytes <= capacity_) return;
  resize(bytes);
}

void Workspace::resize(size_t bytes) {
  const size_t want = align_up(bytes);
  if (owned_ && base_) cudaFree(base_);
  base_ = nullptr;
  capacity_ = 0;
  cursor_ = 0;
  guard_ = 0;
  epoch_ = next_epoch();
  owned_ = true;
  if (want == 0) return;
  void* p = nullptr;
  const cudaError_t e = cudaMalloc(&p, want);
  if (e != cudaSuccess) throw std::runtime_error(std::string("Workspace: cudaMalloc failed: ") + cudaGetErrorString(e));
  base_ = static_cast<uint8_t*>(p);
  capacity_ = want;
}

void Workspace::adopt(void* device_memory, size_t bytes) {
  if (owned_ && base_) cudaFree(base_);
  // Carving is 256-byte aligned relative to an aligned base; skip what it takes to get there.
  const uintptr_t addr = reinterpret_cast<uintptr_t>(device_memory);
  const size_t skip = device_memory ? size_t((256 - addr % 256) % 256) : 0;
  base_ = device_memory ? static_cast<uint8_t*>(device_memory) + skip : nullptr;
  capacity_ = bytes > skip ? bytes - skip : 0;
  cursor_ = 0;
  guard_ = 0;
  epoch_ = next_epoch();
  owned_ = false;
}

void* Workspace::alloc(size_t bytes) {
  const size_t need = align_up(bytes);
  if (cursor_ + need > capacity_)
    throw std::runtime_error("Workspace: arena exhausted (need " + std::to_string(cursor_ + need) + " bytes, have " +
                             std::to_string(capacity_) + ")");
  void* p = base_ + cursor_;
  cursor_ += need;
  return p;
}

// ---- sizes ---------------------------------------------------------------------------------

bool nvfp4_gemm_shape_supported(int out_features, int in_features) noexcept {
  return in_features > 0 && out_features > 0 && in_features % 64 == 0 && out_features % 128 == 0;
}

bool nvfp4_gemm_supported(int out_features, int in_features) {
  return sfq::device_is_sm100() && nvfp4_gemm_shape_supported(out_features, in_features);
}

// Quantized activation of the native NVFP4 path: packed nibbles plus the tiled scales (rows padded to 128).
size_t nvfp4_gemm_workspace_bytes(int rows, int in_features) {
  if (rows <= 0) return 0;
  return align_up(size_t(rows) * in_features / 2) + align_up(sfq::nvfp4_act_scale_bytes(rows, in_features));
}

size_t linear_dense_weight_bytes(const QuantWeight& w) {
  if (w.format == QuantFormat::kBF16) return 0;
  // Unlike the reference, prepare() keeps the expanded int8 weight of a W4A8/W6A8 layer for the chunk
  // loop that follows, so this side of the split is N*K bytes rather than zero.
  if (is_packed_int8(w.format)) return align_up(size_t(w.out_features) * w.in_features);
  return align_up(size_t(w.out_features) * w.in_features * sizeof(__nv_bfloat16));
}

size_t linear_activation_workspace_bytes(const QuantWeight& w, int rows, ComputeType compute) {
  const size_t r = rows > 0 ? size_t(rows) : 0;
  if (is_packed_int8(w.format)) {
    if (compute != ComputeType::kBF16) throw std::invalid_argument("W4A8/W6A8 requires BF16 activations");
    return align_up(r * w.in_features) + align_up(r * 4);
  }
  if (compute != ComputeType::kBF16) {
    // forward_f32 reads x and writes y directly; the two optional fp32 front stages each take a copy of the activation
    size_t f32 = 0;
    if (w.pre_quant_scale != nullptr) f32 += align_up(r * w.in_features * sizeof(float));
    if (convrot_applies(w)) f32 += align_up(r * w.in_features * sizeof(float));
    return f32;
  }
  size_t total = 0;
  if (w.pre_quant_scale != nullptr) total += align_up(r * w.in_features * sizeof(__nv_bfloat16));
  if (convrot_applies(w)) total += align_up(r * w.in_features * sizeof(__nv_bfloat16));
  if (w.format == QuantFormat::kNVFP4 && nvfp4_gemm_shape_supported(w.out_features, w.in_features))
    total = std::max(total, nvfp4_gemm_workspace_bytes(rows, w.in_features));
  return total;
}

size_t linear_workspace_bytes(const QuantWeight& w, int rows, ComputeType compute) {
  return linear_dense_weight_bytes(w) + linear_activation_workspace_bytes(w, rows, compute);
}

// ---- LinearRunner --------------------------------------------------------------------------

void LinearRunner::init(cublasHandle_t /*handle*/, cudaStream_t stream) {
  stream_ = stream;
  initialised_ = true;
  native_nvfp4_device_ = sfq::device_is_sm100();
  (void)sfq::device_status_word();  // allocate the status word now, outside any hot loop
}

bool LinearRunner::takes_native_nvfp4(const QuantWeight& w) const {
  // src/cuda/linear.cu:120-139 with the device test moved from sm_120 to sm_100.
  return native_ && !w.full_precision && native_nvfp4_device_ && w.format == QuantFormat::kNVFP4 &&
         w.block_scale != nullptr && !convrot_applies(w) && w.pre_quant_scale == nullptr &&
         nvfp4_gemm_shape_supported(w.out_features, w.in_features);
}

LinearRunner::~LinearRunner() {
  if (fork_) cudaEventDestroy(fork_);
  if (join_) cudaEventDestroy(join_);
  if (side_) cudaStreamDestroy(side_);
}

void LinearRunner::ensure_side_stream() {
  if (side_ != nullptr) return;
  cudaError_t e = cudaStreamCreateWithFlags(&side_, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&fork_, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&join_, cudaEventDisableTiming);
  if (e != cudaSuccess) throw std::runtime_error(std::string("LinearRunner: cannot create the side stream: ") + cudaGetErrorString(e));
}

// The expansion prepare() kept is trusted only while the same arena has not given those bytes back: a clear(), a Scope
// that unwinds below them, a resize or an adopt each move the arena to a new epoch. (Like the dense weight the reference's
// prepare() returns, it also assumes that the packed weight itself is not rewritten between prepare() and the calls that
// follow it.)
bool LinearRunner::cached_valid(const QuantWeight& w, const Workspace& ws) const {
  return cached_key_ == w.data && cached_codes_ != nullptr && cached_arena_ == ws.base() && cached_epoch_ == ws.epoch() &&
         ws.used() >= cached_end_;
}

const int8_t* LinearRunner::expanded_weight(const QuantWeight& w, Workspace& ws, bool keep, cudaStream_t stream) {
  // A previous prepare() on this weight in this arena, still below the cursor: reuse it.
  if (cached_valid(w, ws))
    return cached_codes_;
  int8_t* codes = ws.alloc_n<int8_t>(size_t(w.out_features) * w.in_features);
  if (w.format == QuantFormat::kW6A8)
    sfq::unpack_w6a8_int8(static_cast<const int8_t*>(w.data), w.block_scale, codes, w.out_features, w.in_features,
                          int(w.packed_group_size), stream);
  else
    sfq::unpack_w4a8_int8(static_cast<const int8_t*>(w.data), w.block_scale, w.w4_codebook, codes, w.out_features,
                          w.in_features, 16, stream);
  if (keep) {
    cached_key_ = w.data;
    cached_codes_ = codes;
    cached_arena_ = ws.base();
    cached_end_ = ws.used();
    ws.protect(cached_end_);  // the arena reports (through its epoch) when these bytes are handed out again
    cached_epoch_ = ws.epoch();
  }
  return codes;
}

const __nv_bfloat16* LinearRunner::prepare(const QuantWeight& w, Workspace& ws) {
  if (!initialised_) throw std::runtime_error("LinearRunner::prepare: init() not called");
  cached_key_ = nullptr;  // every prepare() starts a new chunk loop: whatever an older one kept is forgotten
  if (is_packed_int8(w.format)) {
    // Returns null like the reference (there is no dense bf16 form), but leaves the int8 expansion
    // carved in `ws` so the chunk loop that follows does not redo it.
    validate_packed_int8(w);
    cached_key_ = nullptr;
    expanded_weight(w, ws, /*keep=*/true, stream_);
    return nullptr;
  }
  if (takes_native_nvfp4(w)) return nullptr;
  if (w.format == QuantFormat::kBF16) return static_cast<const __nv_bfloat16*>(w.data);
  if (!has_dense_form(w)) unsupported_format(w);
  const size_t n = size_t(w.out_features) * w.in_features;
  __nv_bfloat16* dst = ws.alloc_n<__nv_bfloat16>(n);
  switch (w.format) {  // materialise_bf16, src/cuda/linear_weights.cu:580-634
    case QuantFormat::kNVFP4:
      if (w.block_scale == nullptr) throw std::runtime_error("linear: nvfp4 weight without block_scale");
      sfq::unpack_nvfp4_bf16(static_cast<const uint8_t*>(w.data), w.block_scale, w.global_scale, dst, w.out_features,
                             w.in_features, stream_);
      break;
    case QuantFormat::kI8:
      if (w.weight_scale == nullptr) throw std::runtime_error("linear: int8 weight without weight_scale");
      sfq::unpack_int8_bf16(static_cast<const int8_t*>(w.data), w.weight_scale, dst, w.out_features, w.in_features, stream_);
      break;
    case QuantFormat::kF8E4M3:
      if (w.weight_scale == nullptr) throw std::runtime_error("linear: fp8 weight without weight_scale");
      sfq::unpack_f8e4m3_bf16(static_cast<const uint8_t*>(w.data), w.weight_scale, dst, n, stream_);
      break;
    case QuantFormat::kNF4:
      sfq::unpack_nf4_bf16(static_cast<const uint8_t*>(w.data), w.nf4_absmax, w.nf4_quant_map, w.nf4_nested_quant_map,
                           w.nf4_nested_absmax, w.nf4_block_size, w.nf4_nested_block_size, w.nf4_nested_offset, dst,
                           w.out_features, w.in_features, stream_);
      break;
    case QuantFormat::kF16:
      sfq::convert_f16_bf16(static_cast<const __half*>(w.data), dst, n, stream_);
      break;
    case QuantFormat::kF32:
      sfq::convert_f32_bf16(static_cast<const float*>(w.data), dst, n, stream_);
      break;
    default:
      unsupported_format(w);
  }
  return dst;
}

void LinearRunner::forward(const QuantWeight& w, const __nv_bfloat16* x, int rows, __nv_bfloat16* y, Workspace& ws) {
  if (!initialised_) throw std::runtime_error("LinearRunner::forward: init() not called");
  if (rows <= 0) return;
  Workspace::Scope scope(ws);
  cached_key_ = nullptr;  // a plain forward never trusts an older expansion, of this weight or any other
  if (is_packed_int8(w.format)) {
    forward_prepared(w, nullptr, x, rows, y, ws);
    return;
  }
  forward_prepared(w, prepare(w, ws), x, rows, y, ws);
}

void LinearRunner::forward_prepared(const QuantWeight& w, const __nv_bfloat16* weight, const __nv_bfloat16* x,
                                    int rows, __nv_bfloat16* y, Workspace& ws) {
  if (!initialised_) throw std::runtime_error("LinearRunner::forward_prepared: init() not called");
  if (rows <= 0) return;
  Workspace::Scope scope(ws);

  if (is_packed_int8(w.format)) {
    validate_packed_int8(w);
    if (cached_valid(w, ws)) {
      run_packed_int8(w, cached_codes_, x, rows, y, ws, nullptr);  // expansion kept by prepare()
      return;
    }
    // No expansion at hand: decode the weight on the side stream while this one quantizes the activation.
    ensure_side_stream();
    auto check = [](cudaError_t e) {
      if (e != cudaSuccess) throw std::runtime_error(std::string("LinearRunner: stream fork failed: ") + cudaGetErrorString(e));
    };
    check(cudaEventRecord(fork_, stream_));
    check(cudaStreamWaitEvent(side_, fork_, 0));
    const int8_t* codes = expanded_weight(w, ws, /*keep=*/false, side_);
    check(cudaEventRecord(join_, side_));
    run_packed_int8(w, codes, x, rows, y, ws, join_);
    return;
  }
  if (weight == nullptr && !takes_native_nvfp4(w))
    throw std::runtime_error(
        "LinearRunner::forward_prepared: null dense weight for a layer that does not take the "
        "native nvfp4 GEMM -- call prepare() and pass what it returns");
  if (weight == nullptr) {
    uint8_t* xq = ws.alloc_n<uint8_t>(size_t(rows) * (w.in_features / 2));
    uint8_t* xs = ws.alloc_n<uint8_t>(sfq::nvfp4_act_scale_bytes(rows, w.in_features));
    sfq::quantize_nvfp4_block(x, sfq::NormArgs{}, xq, xs, nullptr, rows, w.in_features, SFQ_NVFP4_ACT_GEMM_FEED,
                              stream_);
    sfq::GemmArgs g = epilogue_for(w, rows, y, activation_);
    g.global_scale = w.global_scale;
    g.a_scale_tiled = xs;
    g.w_scale_tiled = w.block_scale;
    sfq::gemm_nvfp4(xq, static_cast<const uint8_t*>(w.data), g, stream_);
    return;
  }
  // AWQ scales the activation per input channel ahead of everything else (src/cuda/linear.cu:221-237).
  const __nv_bfloat16* xin = x;
  if (w.pre_quant_scale != nullptr) {
    __nv_bfloat16* xs = ws.alloc_n<__nv_bfloat16>(size_t(rows) * w.in_features);
    sfq::pre_quant_scale(xin, w.pre_quant_scale, xs, rows, w.in_features, stream_);
    xin = xs;
  }
  if (convrot_applies(w)) {
    __nv_bfloat16* xr = ws.alloc_n<__nv_bfloat16>(size_t(rows) * w.in_features);
    sfq::convrot(xin, xr, rows, w.in_features, w.convrot_group, stream_);
    xin = xr;
  }
  sfq::GemmArgs g = epilogue_for(w, rows, y, activation_);
  sfq::gemm_bf16(xin, weight, g, stream_);
}

void LinearRunner::forward_with_codes(const QuantWeight& w, const int8_t* codes, const __nv_bfloat16* x, int rows,
                                      __nv_bfloat16* y, Workspace& ws) {
  if (!initialised_) throw std::runtime_error("LinearRunner::forward_with_codes: init() not called");
  if (rows <= 0) return;
  validate_packed_int8(w);
  if (codes == nullptr) throw std::invalid_argument("LinearRunner::forward_with_codes: null int8 weight");
  run_packed_int8(w, codes, x, rows, y, ws, nullptr);
}

void LinearRunner::run_packed_int8(const QuantWeight& w, const int8_t* codes, const __nv_bfloat16* x, int rows,
                                   __nv_bfloat16* y, Workspace& ws, cudaEvent_t codes_ready) {
  Workspace::Scope scope(ws);
  int8_t* q = ws.alloc_n<int8_t>(size_t(rows) * w.in_features);
  float* scales = ws.alloc_n<float>(size_t(rows));
  sfq::quantize_int8_token(x, sfq::NormArgs{}, q, scales, nullptr, rows, w.in_features, /*apply_convrot=*/true,
                           stream_);
  if (codes_ready != nullptr) {
    const cudaError_t e = cudaStreamWaitEvent(stream_, codes_ready, 0);
    if (e != cudaSuccess) throw std::runtime_error(std::string("LinearRunner: stream join failed: ") + cudaGetErrorString(e));
  }
  sfq::GemmArgs g = epilogue_for(w, rows, y, activation_);
  g.row_scale = scales;
  g.col_scale = w.weight_scale;
  sfq::gemm_int8(q, codes, g, stream_);
}

// fp32 activations in, fp32 out (src/cuda/linear.cu:251-285): the weight is used as stored when it is fp32 and in
// its dense bf16 form otherwise (the reference widens that copy to fp32 first; the values are the same), the
// activation first takes the AWQ pre-scale and the ConvRot rotation in fp32 when the weight asks for them, the product
// runs on CUDA cores with fp32 accumulation, the bias is added to the finished sum.
void LinearRunner::forward_f32(const QuantWeight& w, const float* x, int rows, float* y, Workspace& ws) {
  if (!initialised_) throw std::runtime_error("LinearRunner::forward_f32: init() not called");
  if (rows <= 0) return;
  if (is_packed_int8(w.format)) throw std::invalid_argument("W4A8/W6A8 requires BF16 activations");
  Workspace::Scope scope(ws);
  const bool bias_bf16 = w.bias != nullptr && w.bias_format == QuantFormat::kBF16;
  if (w.bias != nullptr && w.bias_format != QuantFormat::kF32 && w.bias_format != QuantFormat::kBF16)
    throw std::runtime_error("linear: bias must be F32 or BF16");
  const void* weight = w.data;
  const bool weight_bf16 = w.format != QuantFormat::kF32;
  if (weight_bf16) {
    const bool was_native = native_;
    native_ = false;  // the dense form, whatever the runner's NVFP4 switch says
    try {
      weight = prepare(w, ws);
    } catch (...) {
      native_ = was_native;
      throw;
    }
    native_ = was_native;
  }
  const float* xin = x;
  if (w.pre_quant_scale != nullptr) {
    float* xs = ws.alloc_n<float>(size_t(rows) * w.in_features);
    sfq::pre_quant_scale_f32(xin, w.pre_quant_scale, xs, rows, w.in_features, stream_);
    xin = xs;
  }
  if (convrot_applies(w)) {
    float* xr = ws.alloc_n<float>(size_t(rows) * w.in_features);
    sfq::convrot_f32(xin, xr, rows, w.in_features, w.convrot_group, stream_);
    xin = xr;
  }
  sfq::linear_f32(xin, weight, weight_bf16, w.bias, bias_bf16, y, rows, w.out_features, w.in_features, stream_);
}

// ---- free launchers ------------------------------------------------------------------------

void launch_head_rmsnorm(__nv_bfloat16* x, const __nv_bfloat16* w, int rows, int heads, int dim, float eps, cudaStream_t stream) {
  if (w == nullptr) throw std::invalid_argument("launch_head_rmsnorm: null weight");
  sfq::head_norm_rope(x, heads * dim, w, nullptr, nullptr, rows, heads, dim, eps, stream);
}
void launch_rope_h3(__nv_bfloat16* x, const float* cos, const float* sin, int rows, int heads, int head_dim, cudaStream_t stream) {
  if (cos == nullptr || sin == nullptr) throw std::invalid_argument("launch_rope_h3: null table");
  sfq::head_norm_rope(x, heads * head_dim, nullptr, cos, sin, rows, heads, head_dim, 0.0f, stream);
}
void launch_adaln_expand(const float* w, const float* bias, const float* code, float* out, int num_t, int num_modality, int num_param,
                         int channels, int rank, cudaStream_t stream) {
  sfq::adaln_expand(w, bias, code, out, num_t, num_modality, num_param, channels, rank, stream);
}
void launch_convrot(const __nv_bfloat16* in, __nv_bfloat16* out, int rows, int dim, int group, cudaStream_t stream) {
  sfq::convrot(in, out, rows, dim, group, stream);
}
void launch_dequant_i8_per_channel(const int8_t* src, const float* scale, __nv_bfloat16* dst, int out_features,
                                   int in_features, cudaStream_t stream) {
  sfq::unpack_int8_bf16(src, scale, dst, out_features, in_features, stream);
}
void launch_dequant_f8e4m3(const uint8_t* src, const float* scale, __nv_bfloat16* dst, size_t n, cudaStream_t stream) {
  sfq::unpack_f8e4m3_bf16(src, scale, dst, n, stream);
}
void launch_dequant_nf4(const uint8_t* src, const uint8_t* absmax, const float* quant_map, const float* nested_quant_map,
                        const float* nested_absmax, int block_size, int nested_block_size, float nested_offset,
                        __nv_bfloat16* dst, int out_features, int in_features, cudaStream_t stream) {
  sfq::unpack_nf4_bf16(src, absmax, quant_map, nested_quant_map, nested_absmax, block_size, nested_block_size,
                       nested_offset, dst, out_features, in_features, stream);
}
void launch_pre_quant_scale(const __nv_bfloat16* src, const __nv_bfloat16* scale, __nv_bfloat16* dst, int rows, int dim,
                            cudaStream_t stream) {
  sfq::pre_quant_scale(src, scale, dst, rows, dim, stream);
}
void launch_dequant_nvfp4(const uint8_t* src, const uint8_t* block_scale, float global_scale, __nv_bfloat16* dst,
                          int out_features, int in_features, cudaStream_t stream) {
  sfq::unpack_nvfp4_bf16(src, block_scale, global_scale, dst, out_features, in_features, stream);
}
void launch_dequant_w6a8_weight(const int8_t* packed, const uint8_t* group_scale, int8_t* output, int out_features,
                                int in_features, int group_size, cudaStream_t stream) {
  sfq::unpack_w6a8_int8(packed, group_scale, output, out_features, in_features, group_size, stream);
}
void launch_dequant_w4a8_weight(const int8_t* packed, const uint8_t* group_scale, const float* codebook,
                                int8_t* output, int out_features, int in_features, int group_size,
                                cudaStream_t stream) {
  sfq::unpack_w4a8_int8(packed, group_scale, codebook, output, out_features, in_features, group_size, stream);
}
void launch_quantize_w4a8_bf16(const __nv_bfloat16* rotated, int8_t* output, float* row_scale, int rows, int width,
                               cudaStream_t stream) {
  sfq::quantize_int8_token(rotated, sfq::NormArgs{}, output, row_scale, nullptr, rows, width, /*apply_convrot=*/false,
                           stream);
}
void launch_quantize_nvfp4_activations(const __nv_bfloat16* x, uint8_t* packed, uint8_t* scales, int rows, int dim,
                                       cudaStream_t stream) {
  sfq::quantize_nvfp4_block(x, sfq::NormArgs{}, packed, scales, nullptr, rows, dim, SFQ_NVFP4_ACT_REFERENCE, stream);
}
void launch_rmsnorm(const __nv_bfloat16* x, const __nv_bfloat16* w, __nv_bfloat16* out, int rows, int dim, float eps,
                    cudaStream_t stream) {
  sfq::NormArgs n;
  n.weight = w;
  n.eps = eps;
  sfq::rmsnorm(x, n, out, rows, dim, stream);
}
void launch_rmsnorm_modulate(const __nv_bfloat16* x, const __nv_bfloat16* w, const float* scale, const float* shift,
                             const int32_t* a, __nv_bfloat16* out, int rows, int dim, float eps, cudaStream_t stream) {
  sfq::NormArgs n;
  n.weight = w;
  n.scale = scale;
  n.shift = shift;
  n.index = a;
  n.eps = eps;
  sfq::rmsnorm(x, n, out, rows, dim, stream);
}
void launch_add_gated(__nv_bfloat16* x, const __nv_bfloat16* branch, const float* gate, const int32_t* a, int rows,
                      int dim, cudaStream_t stream) {
  sfq::add_gated(x, branch, gate, a, rows, dim, stream);
}
void launch_swiglu(const __nv_bfloat16* fused, __nv_bfloat16* out, int rows, int inner, cudaStream_t stream) {
  sfq::swiglu(fused, out, rows, inner, stream);
}
void launch_gelu_tanh(__nv_bfloat16* x, size_t n, cudaStream_t stream) { sfq::gelu_tanh(x, n, stream); }

namespace {
void nvfp4_gemm_feed(const uint8_t* xq, const uint8_t* xs_tiled, const uint8_t* w_packed, const uint8_t* w_scale, float global_scale,
                     __nv_bfloat16* y, int rows, int out_features, int in_features, cudaStream_t stream) {
  sfq::GemmArgs g;
  g.M = rows;
  g.N = out_features;
  g.K = in_features;
  g.y = y;
  g.ldy = out_features;
  g.global_scale = global_scale;
  g.a_scale_tiled = xs_tiled;
  g.w_scale_tiled = w_scale;
  g.status = sfq::device_status_word();
  sfq::gemm_nvfp4(xq, w_packed, g, stream);
}
void require_native_nvfp4(int out_features, int in_features) {  // the refusal of src/cuda/nvfp4_gemm.cu:536-547, device test moved to sm_100
  if (!nvfp4_gemm_supported(out_features, in_features))
    throw std::runtime_error("nvfp4_gemm: native NVFP4 requires a Blackwell (sm_100) GPU and " + std::to_string(out_features) + "x" +
                             std::to_string(in_features) + " needs out % 128 == 0 and in % 64 == 0; the padded block-scale "
                             "layout has never been observed and is not guessed at");
}
}  // namespace

void nvfp4_gemm_forward_prevalidated(const __nv_bfloat16* x, const uint8_t* w_packed, const uint8_t* w_scale, float global_scale,
                                     __nv_bfloat16* y, int rows, int out_features, int in_features, Workspace& ws, cudaStream_t stream) {
  if (rows <= 0 || out_features <= 0) return;
  Workspace::Scope scope(ws);
  uint8_t* xq = ws.alloc_n<uint8_t>(size_t(rows) * (in_features / 2));
  uint8_t* xs = ws.alloc_n<uint8_t>(sfq::nvfp4_act_scale_bytes(rows, in_features));
  sfq::quantize_nvfp4_block(x, sfq::NormArgs{}, xq, xs, nullptr, rows, in_features, SFQ_NVFP4_ACT_GEMM_FEED, stream);
  nvfp4_gemm_feed(xq, xs, w_packed, w_scale, global_scale, y, rows, out_features, in_features, stream);
}

void nvfp4_gemm_forward(const __nv_bfloat16* x, const uint8_t* w_packed, const uint8_t* w_scale, float global_scale, __nv_bfloat16* y,
                        int rows, int out_features, int in_features, Workspace& ws, cudaStream_t stream) {
  if (rows <= 0 || out_features <= 0) return;
  require_native_nvfp4(out_features, in_features);
  nvfp4_gemm_forward_prevalidated(x, w_packed, w_scale, global_scale, y, rows, out_features, in_features, ws, stream);
}

void nvfp4_gemm_forward_q(const uint8_t* xq, const uint8_t* xs, const uint8_t* w_packed, const uint8_t* w_scale, float global_scale,
                          __nv_bfloat16* y, int rows, int out_features, int in_features, cudaStream_t stream) {
  if (rows <= 0 || out_features <= 0) return;
  require_native_nvfp4(out_features, in_features);
  const size_t q_bytes = align_up(size_t(rows) * (in_features / 2));
  const size_t s_bytes = sfq::nvfp4_act_scale_bytes(rows, in_features);
  void* scratch = nullptr;
  cudaError_t e = cudaMallocAsync(&scratch, q_bytes + s_bytes, stream);
  if (e != cudaSuccess) throw std::runtime_error(std::string("nvfp4_gemm_forward_q: scratch allocation failed: ") + cudaGetErrorString(e));
  uint8_t* fq = static_cast<uint8_t*>(scratch);
  uint8_t* fs = fq + q_bytes;
  try {
    sfq::nvfp4_act_to_feed(xq, xs, fq, fs, rows, in_features, stream);
    nvfp4_gemm_feed(fq, fs, w_packed, w_scale, global_scale, y, rows, out_features, in_features, stream);
  } catch (...) {
    cudaFreeAsync(scratch, stream);
    throw;
  }
  e = cudaFreeAsync(scratch, stream);
  if (e != cudaSuccess) throw std::runtime_error(std::string("nvfp4_gemm_forward_q: ") + cudaGetErrorString(e));
}

void launch_w4a8_output_bf16(const int32_t* input, const float* row_scale, const float* channel_scale, __nv_bfloat16* output, int rows,
                             int cols, cudaStream_t stream) {
  sfq::int8_output_bf16(input, row_scale, channel_scale, output, rows, cols, stream);
}
void launch_dequant_w4a8_output(int32_t* input_output, const float* activation_scale, const float* weight_scale, int rows, int cols,
                                cudaStream_t stream) {
  sfq::int8_output_f32_inplace(input_output, activation_scale, weight_scale, rows, cols, stream);
}
void launch_convrot_f32(const float* in, float* out, int rows, int dim, int group, cudaStream_t stream) {
  sfq::convrot_f32(in, out, rows, dim, group, stream);
}
void launch_dequant_nf4_f16(const uint8_t* src, const uint8_t* absmax, const float* quant_map, const float* nested_quant_map,
                            const float* nested_absmax, int block_size, int nested_block_size, float nested_offset, __half* dst, size_t n,
                            cudaStream_t stream) {
  if (!src || !absmax || !quant_map || !nested_quant_map || !nested_absmax || !dst)
    throw std::runtime_error("launch_dequant_nf4_f16: null pointer");
  if (block_size <= 0 || nested_block_size <= 0) throw std::runtime_error("launch_dequant_nf4_f16: invalid block sizes");
  sfq::unpack_nf4_f16(src, absmax, quant_map, nested_quant_map, nested_absmax, block_size, nested_block_size, nested_offset, dst, n, stream);
}
void launch_quantize_f8e4m3(const __nv_bfloat16* src, float input_scale, uint8_t* dst, size_t n, cudaStream_t stream) {
  sfq::quantize_f8e4m3(src, input_scale, dst, n, stream);
}
void launch_widen_bf16(const __nv_bfloat16* src, float* dst, size_t n, cudaStream_t stream) { sfq::widen_bf16(src, dst, n, stream); }
void launch_narrow_to_bf16(const float* src, __nv_bfloat16* dst, size_t n, cudaStream_t stream) { sfq::narrow_to_bf16(src, dst, n, stream); }

}  // namespace slopfab::cuda
