// Small process-wide runtime state of the library: the per-device status word
// kernels write when they abandon a bounded wait, the GEMM tuning knobs, and
// the device capability test.
#pragma once

#include <functional>
#include <mutex>

#include "gemm_tc.cuh"

namespace sfq {

// Device pointer to a zero-initialised int on the current device (allocated on first use, kept
// until exit). Throws std::runtime_error when there is no usable CUDA device.
int* device_status_word();
// Copies the word back, clears it, returns it. Synchronises the device.
int read_and_clear_device_status();

bool device_is_sm100();  // compute capability 10.x of the current device

// Index of the current device, checked against the size of the library's per-device tables (kMaxDevices).
constexpr int kMaxDevices = 64;
int current_device_index();
// Multiprocessor count of the current device (looked up once per device).
int device_sm_count();
// Raises a kernel's dynamic shared-memory limit to `bytes` on the CURRENT device when it is not already that high.
// The attribute belongs to the (device, function) pair, so one process that drives several GPUs needs it set on
// each of them; the table behind this call is keyed by both. Throws std::runtime_error on failure.
void reserve_dynamic_smem(const void* kernel, size_t bytes, const char* what);

// Test hooks (thread-local; only the stand-alone sfq_gemm_* entry points apply them, a runner never does).
// Variant: tile_n 128 / 256 selects the one-CTA kernel with that tile width, band_m the raster band, max_ctas the grid.
void set_test_gemm_variant(int tile_n, int band_m, int max_ctas);
// Lost load: the producer skips the loads of pipeline iteration `iteration` (>= 0) while still announcing their bytes, and
// every bounded wait gives up after `wait_cycles` clocks instead of the default second; -1 / 0 switch both off.
void set_test_gemm_lost_load(int iteration, long long wait_cycles);
void apply_test_hooks(GemmArgs& g);

// A value computed once per device (occupancy answers and the like), keyed by the device that is current at the call.
template <class T> class PerDevice {
 public:
  template <class F> T get(F&& compute) {
    const int dev = current_device_index();
    std::lock_guard<std::mutex> lock(mutex_);
    if (!have_[dev]) {
      value_[dev] = compute();
      have_[dev] = true;
    }
    return value_[dev];
  }

 private:
  std::mutex mutex_;
  T value_[kMaxDevices] = {};
  bool have_[kMaxDevices] = {};
};

}  // namespace sfq
