// sfq_linear_nvfp4_forward_static: the native NVFP4 Linear for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc at the point where they run a Linear: a plugin
// that is handed a stream inside someone else's frame loop, a process whose memory pool is owned and
// fully carved by its embedder, or code that runs after the application has frozen its allocations
// to keep latency flat. The regular entry points take a caller-provided workspace for the quantized
// activation; this one keeps that scratch (and the kernel's status word) in a fixed array that lives
// in the library image itself, so the call touches no allocator of any kind.
#include "../../include/sfq.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>

#include "gemm_tc.cuh"
#include "kernels.cuh"
#include "runtime.h"

namespace sfq_capi {
void set_error(const char* text);  // capi.cu: the text behind sfq_last_error()
}

namespace {

constexpr size_t kStatusBytes = 256;
constexpr size_t kScratchBytes = SFQ_STATIC_SCRATCH_BYTES;

// Resident on every GPU that loads the library, until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[kStatusBytes + kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mutex;
unsigned char* g_device_address[kMaxDevices] = {};

// In host code `g_static_scratch` is only a handle for the runtime, not an address a kernel can
// use: the device address is looked up once per device, with that device current.
unsigned char* scratch_on_current_device() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    throw std::runtime_error(std::string("sfq: no usable CUDA device: ") + cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_device_address[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      throw std::runtime_error(std::string("sfq: cannot resolve the static scratch array: ") + cudaGetErrorString(e));
    g_device_address[dev] = static_cast<unsigned char*>(p);
  }
  return g_device_address[dev];
}

}  // namespace

extern "C" {

// Declared in include/sfq.h.
int sfq_linear_nvfp4_forward_static(const void* d_x_bf16, int rows, const uint8_t* d_w_packed,
                                    const uint8_t* d_w_scale_tiled, float global_scale, const void* d_bias,
                                    int bias_format, int activation, void* d_y_bf16, int out_features,
                                    int in_features, void* stream) {
  try {
    if (rows <= 0) return SFQ_OK;
    if (!d_x_bf16 || !d_w_packed || !d_w_scale_tiled || !d_y_bf16)
      throw std::invalid_argument("sfq_linear_nvfp4_forward_static: null buffer");
    if (out_features <= 0 || in_features <= 0 || in_features % 64 != 0 || out_features % 128 != 0)
      throw std::invalid_argument("sfq_linear_nvfp4_forward_static: needs in_features % 64 == 0 and out_features % 128 == 0");
    if (d_bias != nullptr && bias_format != SFQ_F32 && bias_format != SFQ_BF16)
      throw std::invalid_argument("sfq_linear_nvfp4_forward_static: bias must be fp32 or bf16");
    if (activation != SFQ_ACT_NONE && activation != SFQ_ACT_GELU_TANH)
      throw std::invalid_argument("sfq_linear_nvfp4_forward_static: unknown activation");
    const size_t packed_bytes = (size_t(rows) * in_features / 2 + 255) / 256 * 256;
    const size_t scale_bytes = sfq::nvfp4_act_scale_bytes(rows, in_features);
    if (packed_bytes + scale_bytes > kScratchBytes)
      throw std::invalid_argument("sfq_linear_nvfp4_forward_static: rows x in_features = " + std::to_string(rows) + " x " +
                                  std::to_string(in_features) + " needs " + std::to_string(packed_bytes + scale_bytes) +
                                  " bytes of scratch, the static array holds " + std::to_string(kScratchBytes) +
                                  " (use sfq_linear_forward with a workspace, or split the rows)");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char* base = scratch_on_current_device();
    int* status = reinterpret_cast<int*>(base);
    uint8_t* xq = base + kStatusBytes;
    uint8_t* xs = xq + packed_bytes;
    // The array keeps whatever the previous call left. The quantizer overwrites every byte the GEMM
    // reads (packed rows, scale tiles including their zeroed padding rows). The status word is zero
    // when the module is loaded and is cleared only by sfq_static_status, so a code that one call's
    // kernels recorded survives the calls after it until the host has read it.
    sfq::quantize_nvfp4_block(static_cast<const __nv_bfloat16*>(d_x_bf16), sfq::NormArgs{}, xq, xs, nullptr, rows,
                              in_features, SFQ_NVFP4_ACT_GEMM_FEED, s);
    sfq::GemmArgs g;
    g.M = rows;
    g.N = out_features;
    g.K = in_features;
    g.y = static_cast<__nv_bfloat16*>(d_y_bf16);
    g.ldy = out_features;
    g.global_scale = global_scale;
    g.bias = d_bias;
    g.bias_is_bf16 = bias_format == SFQ_BF16;
    g.act = activation;
    g.a_scale_tiled = xs;
    g.w_scale_tiled = d_w_scale_tiled;
    g.status = status;
      sfq::gemm_nvfp4(xq, d_w_packed, g, s);
    return SFQ_OK;
  } catch (const std::invalid_argument& ex) {
    sfq_capi::set_error(ex.what());
    return SFQ_ERR_INVALID_ARGUMENT;
  } catch (const std::exception& ex) {
    sfq_capi::set_error(ex.what());
    return SFQ_ERR_RUNTIME;
  }
}

// Declared in include/sfq.h. Reads and clears the status word that the kernels of the entry point above
// write: a plain copy through the address resolved by the first call on this device, no allocation.
int sfq_static_status(int* h_code) {
  try {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
      throw std::runtime_error(std::string("sfq: no usable CUDA device: ") + cudaGetErrorString(e));
    unsigned char* base = nullptr;
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      base = g_device_address[dev];
    }
    int code = 0;
    if (base != nullptr) {  // otherwise no call has run on this device yet: nothing can have been recorded
      e = cudaDeviceSynchronize();
      if (e == cudaSuccess) e = cudaMemcpy(&code, base, sizeof(int), cudaMemcpyDeviceToHost);
      if (e == cudaSuccess && code != 0) e = cudaMemset(base, 0, sizeof(int));
      if (e != cudaSuccess) throw std::runtime_error(std::string("sfq_static_status: ") + cudaGetErrorString(e));
    }
    if (h_code) *h_code = code;
    return SFQ_OK;
  } catch (const std::exception& ex) {
    sfq_capi::set_error(ex.what());
    return SFQ_ERR_RUNTIME;
  }
}

}  // extern "C"
