// LoRA side branch of a Linear on B200: y += (x A^T) B^T with bf16 factors, both products on the tcgen05 bf16 GEMM,
// the addition fused into the second product's epilogue.
//
// Mirrors slopfab::cuda::LoraRunner (include/slopfab/cuda/lora.cuh:14-37, src/cuda/lora.cu:16-93): same names,
// argument meaning and errors. Differences, all of them stated here:
//   * `blas` is accepted and never used (this library has no cuBLAS on any path).
//   * Arithmetic is that of the reference's tensor-core arm (`exact == false`): hidden = bf16(x A^T) with fp32
//     accumulation, y = bf16(y + bf16(hidden B^T)). Its deterministic arm (`exact == true`) fixes the accumulation
//     order of a scalar loop; a tensor-core product cannot reproduce that order, so `exact` is accepted and the
//     result is within the tolerance the reference's own test allows its tensor arm (2^-8 absolute on O(1) data,
//     tests/test_lora_backends.cu:120), not bit-identical to the scalar arm.
//   * Scratch holds the hidden activations of 2048 rows (the reference: hidden + delta of 256 rows); longer inputs
//     are processed in slices of that many rows. There is no delta buffer: the second GEMM adds into y.
//   * Ranks that are not a multiple of 8 are zero-padded on upload (a 16-byte row pitch is what the TMA needs);
//     `in` must be a multiple of 8.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>
#include <map>
#include <vector>

typedef struct cublasContext* cublasHandle_t;  // as in linear.hpp: kept in signatures, never dereferenced

#pragma GCC visibility push(default)
namespace slopfab {

// Host factors in model coordinates (include/slopfab/lora.h:18-23): the update is B @ A, scale folded into B.
struct LoraFactors {
  int rank = 0, in = 0, out = 0;
  std::vector<float> a, b;  // a: [rank, in], b: [out, rank]
};

namespace cuda {

class LoraRunner {
public:
  LoraRunner() = default;
  ~LoraRunner();
  LoraRunner(const LoraRunner&) = delete;
  LoraRunner& operator=(const LoraRunner&) = delete;

  // Uploads rows [row_offset, row_offset + out) of every factor pair's B (a q/k/v slice of a fused projection) and all
  // of A, rounded to bf16. With the three staging arguments the bf16 bytes are written to `staged_host` at
  // `*staged_offset` (advanced in 256-byte steps) and read later from the same offset of `staged_device`; the caller
  // copies the block. Throws std::invalid_argument on incomplete staging arguments, std::runtime_error on a bad slice.
  void attach(const void* key, const std::vector<LoraFactors>& factors, int row_offset, int out, uint8_t* staged_host = nullptr,
              uint8_t* staged_device = nullptr, size_t* staged_offset = nullptr);
  // output[rows, out] += (input[rows, in] A^T) B^T for every factor pair attached under `key`; no-op for an unknown key.
  void apply(const void* key, const __nv_bfloat16* input, int rows, __nv_bfloat16* output, cublasHandle_t blas, cudaStream_t stream,
             bool exact);
  size_t weight_bytes() const;   // resident (non-staged) factor bytes
  size_t scratch_bytes() const;  // hidden activations + the epilogue's unit gate

  static constexpr int kRows = 2048;  // rows per slice

private:
  struct Factors {
    int rank = 0, in = 0, out = 0;  // rank as stored (padded to a multiple of 8)
    __nv_bfloat16* a_own = nullptr;
    __nv_bfloat16* b_own = nullptr;
    const __nv_bfloat16* a_ptr = nullptr;
    const __nv_bfloat16* b_ptr = nullptr;
    size_t own_bytes = 0;
  };
  void reserve(int rank, int out);

  std::map<const void*, std::vector<Factors>> factors_;
  __nv_bfloat16* hidden_ = nullptr;  // [kRows, max rank]
  float* unit_gate_ = nullptr;       // [max out] of 1.0f
  int32_t* gate_index_ = nullptr;    // [kRows] of 0
  size_t hidden_elems_ = 0, gate_elems_ = 0;
};

}  // namespace cuda
}  // namespace slopfab
#pragma GCC visibility pop
