// LoraRunner: the low-rank side branch of a Linear (src/cuda/lora.cu:16-93) on the tcgen05 bf16 GEMM.
//   hidden = bf16(x A^T)                       one GEMM, N = rank
//   y      = bf16(y + bf16(hidden B^T))        one GEMM, K = rank, the addition in its epilogue
// The epilogue used is the gated residual y = bf16(fma(gate, branch, y)) with a gate of ones: fma(1, b, y) is y + b
// rounded once, i.e. launch_add_bf16 (src/cuda/nn_pointwise.cu:241) applied to the rounded product.
#include "../../include/slopfab_b200/lora.hpp"

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <string>

#include "codec.cuh"
#include "gemm_tc.cuh"
#include "runtime.h"

namespace slopfab::cuda {
namespace {

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("LoRA: ") + what + ": " + cudaGetErrorString(e));
}
int padded_rank(int rank) { return (rank + 7) / 8 * 8; }

}  // namespace

LoraRunner::~LoraRunner() {
  for (auto& entry : factors_)
    for (auto& f : entry.second) {
      cudaFree(f.a_own);
      cudaFree(f.b_own);
    }
  cudaFree(hidden_);
  cudaFree(unit_gate_);
  cudaFree(gate_index_);
}

void LoraRunner::reserve(int rank, int out) {
  const size_t need_hidden = size_t(kRows) * size_t(rank);
  if (need_hidden > hidden_elems_) {
    cudaFree(hidden_);
    hidden_ = nullptr;
    hidden_elems_ = 0;
    check(cudaMalloc(&hidden_, need_hidden * sizeof(__nv_bfloat16)), "scratch allocation");
    hidden_elems_ = need_hidden;
  }
  if (size_t(out) > gate_elems_) {
    cudaFree(unit_gate_);
    unit_gate_ = nullptr;
    gate_elems_ = 0;
    check(cudaMalloc(&unit_gate_, size_t(out) * sizeof(float)), "scratch allocation");
    const std::vector<float> ones(size_t(out), 1.0f);
    check(cudaMemcpy(unit_gate_, ones.data(), ones.size() * sizeof(float), cudaMemcpyHostToDevice), "upload");
    gate_elems_ = size_t(out);
  }
  if (gate_index_ == nullptr) {
    check(cudaMalloc(&gate_index_, size_t(kRows) * sizeof(int32_t)), "scratch allocation");
    check(cudaMemset(gate_index_, 0, size_t(kRows) * sizeof(int32_t)), "clear");
  }
}

void LoraRunner::attach(const void* key, const std::vector<LoraFactors>& host, int offset, int out, uint8_t* staged_host,
                        uint8_t* staged_device, size_t* staged_offset) {
  if ((staged_host != nullptr || staged_device != nullptr || staged_offset != nullptr) && !(staged_host && staged_device && staged_offset))
    throw std::invalid_argument("LoRA: incomplete weight staging buffers");
  for (const auto& h : host) {
    if (offset < 0 || out <= 0 || offset > h.out || out > h.out - offset) throw std::runtime_error("LoRA: invalid CUDA output slice");
    if (h.rank <= 0 || h.in <= 0 || h.a.size() != size_t(h.rank) * h.in || h.b.size() != size_t(h.out) * h.rank)
      throw std::runtime_error("LoRA: factor sizes do not match rank / in / out");
    if (h.in % 8 != 0) throw std::runtime_error("LoRA: the input width must be a multiple of 8");
    Factors f;
    f.rank = padded_rank(h.rank);
    f.in = h.in;
    f.out = out;
    // bf16, the rank padded with zeros: A gains zero rows, B zero columns, the product is unchanged
    std::vector<uint16_t> a(size_t(f.rank) * h.in, 0), b(size_t(out) * f.rank, 0);
    for (size_t i = 0; i < h.a.size(); ++i) a[i] = sfq::host_f32_to_bf16(h.a[i]);
    for (int o = 0; o < out; ++o)
      for (int r = 0; r < h.rank; ++r) b[size_t(o) * f.rank + r] = sfq::host_f32_to_bf16(h.b[size_t(o + offset) * h.rank + r]);
    auto upload = [&](const std::vector<uint16_t>& bits, __nv_bfloat16*& own) -> const __nv_bfloat16* {
      const size_t bytes = bits.size() * 2;
      if (staged_host) {
        std::memcpy(staged_host + *staged_offset, bits.data(), bytes);
        const auto* result = reinterpret_cast<const __nv_bfloat16*>(staged_device + *staged_offset);
        *staged_offset += (bytes + 255) / 256 * 256;
        return result;
      }
      check(cudaMalloc(&own, bytes), "factor allocation");
      check(cudaMemcpy(own, bits.data(), bytes, cudaMemcpyHostToDevice), "factor upload");
      f.own_bytes += bytes;
      return own;
    };
    f.a_ptr = upload(a, f.a_own);
    f.b_ptr = upload(b, f.b_own);
    reserve(f.rank, out);
    factors_[key].push_back(f);
  }
}

size_t LoraRunner::weight_bytes() const {
  size_t result = 0;
  for (const auto& entry : factors_)
    for (const auto& f : entry.second) result += f.own_bytes;
  return result;
}

size_t LoraRunner::scratch_bytes() const {
  return hidden_elems_ * sizeof(__nv_bfloat16) + gate_elems_ * sizeof(float) + (gate_index_ ? size_t(kRows) * sizeof(int32_t) : 0);
}

void LoraRunner::apply(const void* key, const __nv_bfloat16* input, int rows, __nv_bfloat16* output, cublasHandle_t, cudaStream_t stream,
                       bool) {
  const auto found = factors_.find(key);
  if (found == factors_.end() || rows <= 0) return;
  if (input == nullptr || output == nullptr) throw std::invalid_argument("LoRA: null activation");
  for (const auto& f : found->second) {
    for (int row = 0; row < rows; row += kRows) {
      const int count = std::min(kRows, rows - row);
      sfq::GemmArgs down;  // hidden = x A^T
      down.M = count, down.N = f.rank, down.K = f.in;
      down.y = hidden_, down.ldy = f.rank;
      down.status = sfq::device_status_word();
      sfq::gemm_bf16(input + size_t(row) * f.in, f.a_ptr, down, stream);
      sfq::GemmArgs up;  // y += hidden B^T
      up.M = count, up.N = f.out, up.K = f.rank;
      up.y = output + size_t(row) * f.out, up.ldy = f.out;
      up.gate = unit_gate_, up.gate_index = gate_index_;
      up.status = down.status;
      sfq::gemm_bf16(hidden_, f.b_ptr, up, stream);
    }
  }
}

}  // namespace slopfab::cuda
