#include "runtime.h"

#include <cstdlib>
#include <mutex>
#include <stdexcept>
#include <string>

namespace sfq {
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mutex;
int* g_status[kMaxDevices] = {};
int g_tile_n = 0, g_band_m = 0, g_max_ctas = 0;

int current_device() {
  int dev = -1;
  const cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    throw std::runtime_error(std::string("sfq: no usable CUDA device: ") + cudaGetErrorString(e));
  return dev;
}
}  // namespace

int* device_status_word() {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status[dev] == nullptr) {
    int* p = nullptr;
    cudaError_t e = cudaMalloc(&p, 256);
    if (e == cudaSuccess) e = cudaMemset(p, 0, 256);
    if (e != cudaSuccess) throw std::runtime_error(std::string("sfq: cannot allocate the status word: ") + cudaGetErrorString(e));
    g_status[dev] = p;
  }
  return g_status[dev];
}

int read_and_clear_device_status() {
  int* p = device_status_word();
  int code = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(&code, p, sizeof(int), cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemset(p, 0, sizeof(int));
  if (e != cudaSuccess) throw std::runtime_error(std::string("sfq: reading the status word failed: ") + cudaGetErrorString(e));
  return code;
}

bool device_is_sm100() {
  int dev = 0, major = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return false;
  if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return false;
  return major == 10;
}

void set_tuning(int tile_n, int band_m, int max_ctas) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_tile_n = (tile_n == 128 || tile_n == 256) ? tile_n : 0;
  g_band_m = band_m > 0 ? band_m : 0;
  g_max_ctas = max_ctas > 0 ? max_ctas : 0;
}

void apply_tuning(GemmArgs& g) {
  g.tile_n = g_tile_n;
  g.band_m = g_band_m;
  g.max_ctas = g_max_ctas;
  static const int debug = [] {
    const char* e = std::getenv("SFQ_GEMM_DEBUG");
    return e ? std::atoi(e) : 0;
  }();
  g.debug = debug;
}

}  // namespace sfq
