#include "runtime.h"

#include <cstdlib>
#include <map>
#include <mutex>
#include <utility>
#include <stdexcept>
#include <string>

namespace sfq {
namespace {
std::mutex g_mutex;
int* g_status[kMaxDevices] = {};
// Test hooks of the stand-alone GEMM entry points; each thread has its own, a runner never reads them.
struct GemmHooks {
  int tile_n = 0, band_m = 0, max_ctas = 0;
  int drop_iteration = -1;
  long long wait_cycles = 0;
};
thread_local GemmHooks t_hooks;

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

int current_device_index() { return current_device(); }

int device_sm_count() {
  static PerDevice<int> cache;
  return cache.get([] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  });
}

void reserve_dynamic_smem(const void* kernel, size_t bytes, const char* what) {
  if (bytes <= 48 * 1024) return;  // within the default limit
  static std::mutex m;
  static std::map<std::pair<int, const void*>, size_t> reserved;
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(m);
  size_t& have = reserved[{dev, kernel}];
  if (bytes <= have) return;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(bytes));
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": cannot reserve shared memory: " + cudaGetErrorString(e));
  have = bytes;
}

void set_test_gemm_variant(int tile_n, int band_m, int max_ctas) {
  t_hooks.tile_n = (tile_n == 128 || tile_n == 256) ? tile_n : 0;
  t_hooks.band_m = band_m > 0 ? band_m : 0;
  t_hooks.max_ctas = max_ctas > 0 ? max_ctas : 0;
}

void set_test_gemm_lost_load(int iteration, long long wait_cycles) {
  t_hooks.drop_iteration = iteration >= 0 ? iteration : -1;
  t_hooks.wait_cycles = wait_cycles > 0 ? wait_cycles : 0;
}

void apply_test_hooks(GemmArgs& g) {
  g.tile_n = t_hooks.tile_n;
  g.band_m = t_hooks.band_m;
  g.max_ctas = t_hooks.max_ctas;
  g.test_drop_iteration = t_hooks.drop_iteration;
  g.wait_cycles = t_hooks.wait_cycles;
}

}  // namespace sfq
