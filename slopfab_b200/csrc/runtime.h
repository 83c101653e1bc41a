// Small process-wide runtime state of the library: the per-device status word
// kernels write when they abandon a bounded wait, the GEMM tuning knobs, and
// the device capability test.
#pragma once

#include "gemm_tc.cuh"

namespace sfq {

// Device pointer to a zero-initialised int on the current device (allocated on first use, kept
// until exit). Throws std::runtime_error when there is no usable CUDA device.
int* device_status_word();
// Copies the word back, clears it, returns it. Synchronises the device.
int read_and_clear_device_status();

bool device_is_sm100();  // compute capability 10.x of the current device

void set_tuning(int tile_n, int band_m, int max_ctas);
void apply_tuning(GemmArgs& g);

}  // namespace sfq
