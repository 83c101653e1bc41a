// Drop-in check of the C++ operator API: this file is written the way a caller of the reference's
// slopfab::cuda::LinearRunner is written (cf. tools/w4a8probe.cpp:38-57 and packed_integer_linear,
// tests/test_nn_kernels_linear_synthetic.cu:820-890 in the reference) and must compile and link against
// include/slopfab_b200/linear.hpp + libsfq.so unchanged. With a GPU it also runs the W4A8 known-answer case
// and prints the bf16 outputs for the Python test to compare with the oracle.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "slopfab_b200/linear.hpp"

using namespace slopfab::cuda;

template <class T> T* upload(const std::vector<T>& h) {
  T* d = nullptr;
  if (cudaMalloc(&d, h.size() * sizeof(T)) != cudaSuccess) throw std::runtime_error("cudaMalloc");
  cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice);
  return d;
}

static uint16_t to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return uint16_t((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

int main(int argc, char** argv) {
  constexpr int rows = 3, out = 4, k = 256;
  std::vector<int8_t> packed(out * k / 2, 0);
  for (int o = 0; o < out; ++o)
    for (int i = 0; i < k; ++i) packed[o * k / 2 + i / 2] |= int8_t((((i * 7 + o * 13) % 16) & 15) << ((i & 1) * 4));
  std::vector<uint8_t> scales(out * k / 16);
  const uint8_t sv[] = {0, 0x30, 0x38, 0x48, 0x78};
  for (size_t i = 0; i < scales.size(); ++i) scales[i] = sv[i % 5];
  std::vector<float> book(16), channel = {.25f, .5f, 1.f, 2.f};
  for (int i = 0; i < 16; ++i) book[i] = float(i - 8);
  std::vector<uint16_t> x(rows * k, 0);
  x[k] = to_bf16(1.0f);
  for (int i = 2 * k; i < 3 * k; ++i) x[i] = to_bf16(1.0f);

  QuantWeight w;  // same fields and defaults as the reference's
  w.format = QuantFormat::kW4A8;
  w.packed_group_size = 16;
  w.in_features = k;
  w.out_features = out;
  w.convrot = true;
  w.convrot_group = 256;
  if (w.stored_bytes() != packed.size() || linear_dense_weight_bytes(w) == 0 || !is_packed_int8(w.format)) return 2;
  if (argc > 1 && argv[1][0] == 'l') {  // link-only mode for machines without a GPU
    printf("linked\n");
    return 0;
  }
  w.data = upload(packed);
  w.block_scale = upload(scales);
  w.weight_scale = upload(channel);
  w.w4_codebook = upload(book);
  auto* dx = reinterpret_cast<__nv_bfloat16*>(upload(x));
  __nv_bfloat16* dy = nullptr;
  cudaMalloc(&dy, rows * out * 2);

  LinearRunner runner;
  runner.init(nullptr, nullptr);
  Workspace ws;
  ws.reserve(linear_workspace_bytes(w, rows, ComputeType::kBF16));
  runner.forward(w, dx, rows, dy, ws);
  // prepare + forward_prepared must give the same bits; prepare returns null for packed int8 as in the reference
  __nv_bfloat16* dy2 = nullptr;
  cudaMalloc(&dy2, rows * out * 2);
  {
    Workspace::Scope scope(ws);
    const __nv_bfloat16* dense = runner.prepare(w, ws);
    if (dense != nullptr) return 3;
    runner.forward_prepared(w, dense, dx, rows, dy2, ws);
  }
  bool threw = false;
  try {  // a violated precondition throws std::invalid_argument before anything is launched
    QuantWeight bad = w;
    bad.convrot = false;
    runner.forward(bad, dx, rows, dy, ws);
  } catch (const std::invalid_argument&) {
    threw = true;
  }
  if (cudaDeviceSynchronize() != cudaSuccess || !threw) return 4;
  std::vector<uint16_t> y(rows * out), y2(rows * out);
  cudaMemcpy(y.data(), dy, y.size() * 2, cudaMemcpyDeviceToHost);
  cudaMemcpy(y2.data(), dy2, y2.size() * 2, cudaMemcpyDeviceToHost);
  if (y != y2) return 5;

  // An arena that was cleared and carved again between prepare() and forward_prepared() -- legal with the reference,
  // which expands the packed weight on every call -- must not be trusted for the expansion prepare() kept: here a
  // dense bf16 layer C is prepared over the same bytes, then A runs with the null pointer its prepare() returned.
  {
    ws.clear();
    runner.prepare(w, ws);  // A's int8 expansion at the front of the arena
    ws.clear();
    std::vector<float> cw(size_t(out) * k, 3.0f);  // C: an fp32 weight whose bf16 form (0x4040...) overwrites A's codes
    QuantWeight c;
    c.format = QuantFormat::kF32;
    c.in_features = k;
    c.out_features = out;
    c.data = upload(cw);
    ws.reserve(linear_workspace_bytes(c, rows, ComputeType::kBF16) + linear_workspace_bytes(w, rows, ComputeType::kBF16));
    ws.clear();
    runner.prepare(w, ws);
    ws.clear();
    if (runner.prepare(c, ws) == nullptr) return 6;
    cudaMemset(dy2, 0, rows * out * 2);
    runner.forward_prepared(w, nullptr, dx, rows, dy2, ws);
    if (cudaDeviceSynchronize() != cudaSuccess) return 7;
    cudaMemcpy(y2.data(), dy2, y2.size() * 2, cudaMemcpyDeviceToHost);
    if (y != y2) return 8;
    ws.clear();
  }

  // One process driving two GPUs: the same Linear on device 1 after device 0 (kernel attributes such as the dynamic
  // shared-memory limit are per device). Skipped on a single-GPU machine.
  int devices = 0;
  cudaGetDeviceCount(&devices);
  if (devices >= 2) {
    if (cudaSetDevice(1) != cudaSuccess) return 9;
    QuantWeight w1 = w;
    w1.data = upload(packed);
    w1.block_scale = upload(scales);
    w1.weight_scale = upload(channel);
    w1.w4_codebook = upload(book);
    auto* dx1 = reinterpret_cast<__nv_bfloat16*>(upload(x));
    __nv_bfloat16* dy1 = nullptr;
    cudaMalloc(&dy1, rows * out * 2);
    LinearRunner second;
    second.init(nullptr, nullptr);
    Workspace ws1;
    ws1.reserve(linear_workspace_bytes(w1, rows, ComputeType::kBF16));
    second.forward(w1, dx1, rows, dy1, ws1);
    if (cudaDeviceSynchronize() != cudaSuccess) return 10;
    cudaMemcpy(y2.data(), dy1, y2.size() * 2, cudaMemcpyDeviceToHost);
    if (y != y2) return 11;
    cudaSetDevice(0);
  }
  for (uint16_t v : y) printf("%u ", unsigned(v));
  printf("\n");
  return 0;
}
