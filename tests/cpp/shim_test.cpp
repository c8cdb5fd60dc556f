// Exercises the C++ shims (reference-shaped signatures) end to end on a GPU:
// loader -> MoEWorkspace -> MoERoutedForward / MoEForward (with the router-trace observer
// and slot mode), MoEDeviceDecode[Multi], Fp4Gemm<float|uint16_t>, the quantiser and the
// dequantiser, the BF16 MoE, plus error strings.
// Prints "shim_test PASS" on success.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "q4t/model/moe.h"
#include "q4t/mtp/moe_bf16.h"
#include "q4t/quant/act_quant.h"
#include "q4t/quant/dequant.h"
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
      // the SwiGLU values of this toy layer are of order 1e-7: the down projection's input scale
      // must be small enough for them to survive quantisation, or every routed output is zero
      const bool input = name.find("input") != std::string::npos;
      const float v = !input ? 0.0007f : name.find("down_proj") != std::string::npos ? 2e-9f : 0.004f;
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
  // ---- the fixed-shape decode entries (include/q4t/quant/moe_decode.h:11-36): same result
  // as the generic call on the same rows, bit for bit (the reference's own grouped-vs-per-row
  // check, tests/moe_decode_grouped_test.cpp:328-411)
  {
    std::vector<float> want(size_t(T) * hs), got(want.size());
    cudaMemcpy(want.data(), d_yf, want.size() * 4, cudaMemcpyDeviceToHost);
    quant::MoEWorkspace mw;
    mw.a_packed = static_cast<uint8_t*>(rws);
    cudaMemset(d_yf, 0, size_t(T) * hs * 4);
    s = quant::MoEDeviceDecodeMulti(d_x, d_ids, d_rw, d_yf, L, mw, nullptr, 0, T, k, 0);
    CHECK(s.ok());
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    cudaMemcpy(got.data(), d_yf, got.size() * 4, cudaMemcpyDeviceToHost);
    CHECK(std::memcmp(want.data(), got.data(), got.size() * 4) == 0);
    // single token, top-10: against ten one-slot calls accumulated in slot order
    std::vector<int32_t> ids1 = {3, 0, 7, 12, 5, 9, 1, 15, 2, 11};
    std::vector<float> rw1(10, 0.1f);
    int32_t* d_ids1; float* d_rw1;
    cudaMalloc(reinterpret_cast<void**>(&d_ids1), 40);
    cudaMalloc(reinterpret_cast<void**>(&d_rw1), 40);
    cudaMemcpy(d_ids1, ids1.data(), 40, cudaMemcpyHostToDevice);
    cudaMemcpy(d_rw1, rw1.data(), 40, cudaMemcpyHostToDevice);
    void* ws1; cudaMalloc(&ws1, quant::MoEWorkspace::RequiredBytes(1, 10, hs, is));
    mw.a_packed = static_cast<uint8_t*>(ws1);
    cudaMemset(d_yf, 0, size_t(hs) * 4);
    s = quant::MoEDeviceDecode(d_x, d_ids1, d_rw1, d_yf, L, mw, nullptr, 0, 0);
    CHECK(s.ok());
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    cudaMemcpy(got.data(), d_yf, size_t(hs) * 4, cudaMemcpyDeviceToHost);
    cudaMemset(d_yf, 0, size_t(hs) * 4);
    CHECK(quant::MoERoutedForward(d_x, d_ids1, d_rw1, d_yf, L, ws1, nullptr, 0, 1, 10, 0).ok());
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    cudaMemcpy(want.data(), d_yf, size_t(hs) * 4, cudaMemcpyDeviceToHost);
    CHECK(std::memcmp(want.data(), got.data(), size_t(hs) * 4) == 0);
    bool any = false;
    for (int i = 0; i < hs; ++i) any |= got[i] != 0.0f;
    CHECK(any);
  }
  // ---- Fp4Gemm<float> / Fp4Gemm<uint16_t> (include/q4t/quant/fp4_gemm.h:58-213) and
  // DequantFp4ToBf16Async (include/q4t/quant/dequant.h:22-25): quantise, multiply, and check
  // against a host dot product of the dequantised operands (the reference's 0.02 bound)
  {
    const int M = 8, N = 256, K = 256;
    uint16_t *d_a, *d_w, *d_ad, *d_wd, *d_o16;
    float* d_o32;
    upload_bf16(&d_a, size_t(M) * K);
    upload_bf16(&d_w, size_t(N) * K);
    const float ga = 0.02f * 5 / (6 * 448), gw = ga;
    uint8_t *d_ap, *d_asf, *d_wp, *d_wsf, *d_arm, *d_wrm;
    cudaMalloc(reinterpret_cast<void**>(&d_ap), size_t(M) * K / 2);
    cudaMalloc(reinterpret_cast<void**>(&d_wp), size_t(N) * K / 2);
    cudaMalloc(reinterpret_cast<void**>(&d_asf), q4t_sf_buffer_size(M, K));
    cudaMalloc(reinterpret_cast<void**>(&d_wsf), q4t_sf_buffer_size(N, K));
    cudaMemset(d_asf, 0, q4t_sf_buffer_size(M, K));
    cudaMemset(d_wsf, 0, q4t_sf_buffer_size(N, K));
    CHECK(quant::QuantizeActivationToFp4Async(d_a, d_ap, d_asf, M, K, ga, 0) == cudaSuccess);
    CHECK(quant::QuantizeActivationToFp4Async(d_w, d_wp, d_wsf, N, K, gw, 0) == cudaSuccess);
    cudaMalloc(reinterpret_cast<void**>(&d_o32), size_t(M) * N * 4);
    cudaMalloc(reinterpret_cast<void**>(&d_o16), size_t(M) * N * 2);
    auto r32 = quant::Fp4Gemm<float>(d_wp, d_wsf, d_ap, d_asf, d_o32, M, N, K, gw, ga, nullptr, 0, 0);
    auto r16 = quant::Fp4Gemm<uint16_t>(d_wp, d_wsf, d_ap, d_asf, d_o16, M, N, K, gw, ga, nullptr, 0, 0);
    CHECK(r32.status == 0 && r32.has_algo && r16.status == 0 && r16.has_algo);
    // un-swizzle the scale bytes on the host (SfOffset) for the dequantiser, which takes row-major scales
    std::vector<uint8_t> asw(q4t_sf_buffer_size(M, K)), wsw(q4t_sf_buffer_size(N, K));
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    cudaMemcpy(asw.data(), d_asf, asw.size(), cudaMemcpyDeviceToHost);
    cudaMemcpy(wsw.data(), d_wsf, wsw.size(), cudaMemcpyDeviceToHost);
    std::vector<uint8_t> arm(size_t(M) * K / 16), wrm(size_t(N) * K / 16);
    const int ntk = q4t_sf_num_gtiles(K);
    for (int r = 0; r < M; ++r) for (int g = 0; g < K / 16; ++g) arm[size_t(r) * (K / 16) + g] = asw[q4t_sf_offset(r, g, ntk)];
    for (int r = 0; r < N; ++r) for (int g = 0; g < K / 16; ++g) wrm[size_t(r) * (K / 16) + g] = wsw[q4t_sf_offset(r, g, ntk)];
    cudaMalloc(reinterpret_cast<void**>(&d_arm), arm.size());
    cudaMalloc(reinterpret_cast<void**>(&d_wrm), wrm.size());
    cudaMemcpy(d_arm, arm.data(), arm.size(), cudaMemcpyHostToDevice);
    cudaMemcpy(d_wrm, wrm.data(), wrm.size(), cudaMemcpyHostToDevice);
    cudaMalloc(reinterpret_cast<void**>(&d_ad), size_t(M) * K * 2);
    cudaMalloc(reinterpret_cast<void**>(&d_wd), size_t(N) * K * 2);
    CHECK(quant::DequantFp4ToBf16Async(d_ap, d_arm, d_ad, ga, M, K, 0) == cudaSuccess);
    CHECK(quant::DequantFp4ToBf16Async(d_wp, d_wrm, d_wd, gw, N, K, 0) == cudaSuccess);
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    std::vector<uint16_t> ad(size_t(M) * K), wd(size_t(N) * K), o16(size_t(M) * N);
    std::vector<float> o32(size_t(M) * N);
    cudaMemcpy(ad.data(), d_ad, ad.size() * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(wd.data(), d_wd, wd.size() * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(o32.data(), d_o32, o32.size() * 4, cudaMemcpyDeviceToHost);
    cudaMemcpy(o16.data(), d_o16, o16.size() * 2, cudaMemcpyDeviceToHost);
    auto f = [](uint16_t b) { uint32_t u = uint32_t(b) << 16; float v; std::memcpy(&v, &u, 4); return v; };
    double worst32 = 0, worst16 = 0, scale = 0;
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n) {
        // the dequantised operands are bf16-rounded; the GEMM multiplies the unrounded ones, so this
        // host product is within bf16 rounding of each factor (2^-8 relative per term) of the truth
        double acc = 0;
        for (int c = 0; c < K; ++c) acc += double(f(ad[size_t(m) * K + c])) * f(wd[size_t(n) * K + c]);
        scale = std::max(scale, std::fabs(acc));
        worst32 = std::max(worst32, std::fabs(o32[size_t(m) * N + n] - acc));
        worst16 = std::max(worst16, std::fabs(f(o16[size_t(m) * N + n]) - acc));
      }
    if (!(scale > 0 && worst32 <= 0.02 * scale && worst16 <= 0.02 * scale))
      std::printf("Fp4Gemm: scale %g worst32 %g worst16 %g\n", scale, worst32, worst16);
    CHECK(scale > 0 && worst32 <= 0.02 * scale && worst16 <= 0.02 * scale);
  }
  // ---- the two per-layer hooks of MoEForward: router-trace observer and slot mode
  {
    int32_t* d_cap; cudaMalloc(reinterpret_cast<void**>(&d_cap), size_t(2) * T * k * 4);
    cudaMemset(d_cap, 0xff, size_t(2) * T * k * 4);
    trace::RouterCollector col;
    col.Begin(d_cap, 2, T, k);
    CHECK(model::MoEForward(d_x, L, X, d_y, T, k, ws, ws_bytes, nullptr, 0, 0, &col, 0).ok());
    CHECK(model::MoEForward(d_x, L, X, d_y, T, k, ws, ws_bytes, nullptr, 0, 0, &col, 1).ok());
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    CHECK(col.captured_layers() == 2 && !col.failed());
    std::vector<int32_t> cap(size_t(2) * T * k), ws_ids(size_t(T) * k);
    cudaMemcpy(cap.data(), d_cap, cap.size() * 4, cudaMemcpyDeviceToHost);
    q4t_forward_ws_layout F;
    CHECK(q4t_moe_forward_workspace_layout(T, k, hs, is, sis, E, &F) == Q4T_OK);
    cudaMemcpy(ws_ids.data(), static_cast<uint8_t*>(ws) + F.expert_ids, ws_ids.size() * 4, cudaMemcpyDeviceToHost);
    for (size_t i = 0; i < ws_ids.size(); ++i) {
      CHECK(cap[i] == ws_ids[i] && cap[ws_ids.size() + i] == ws_ids[i]);
      CHECK(ws_ids[i] >= 0 && ws_ids[i] < E);
    }
    // slot mode with every expert resident in slot (E-1-e): the same layer through permuted
    // weights must give the same bits as the plain layout
    std::vector<uint16_t> y_plain(size_t(T) * hs), y_slots(y_plain.size());
    cudaMemcpy(y_plain.data(), d_y, y_plain.size() * 2, cudaMemcpyDeviceToHost);
    quant::MoEWeightLayout S = L;
    S.slot_mode = true;
    const size_t gup = size_t(2) * is * (hs / 2), gus = L.gu_sf_block(), dnp = size_t(hs) * (is / 2), dns = L.dn_sf_block();
    cudaMalloc(reinterpret_cast<void**>(&S.gu_packed), E * gup);
    cudaMalloc(reinterpret_cast<void**>(&S.gu_sf), E * gus);
    cudaMalloc(reinterpret_cast<void**>(&S.dn_packed), E * dnp);
    cudaMalloc(reinterpret_cast<void**>(&S.dn_sf), E * dns);
    cudaMalloc(reinterpret_cast<void**>(&S.gu_w_scale2), E * 4);
    cudaMalloc(reinterpret_cast<void**>(&S.gu_input_scale), E * 4);
    cudaMalloc(reinterpret_cast<void**>(&S.dn_w_scale2), E * 4);
    cudaMalloc(reinterpret_cast<void**>(&S.dn_input_scale), E * 4);
    std::vector<int32_t> table(E);
    for (int e = 0; e < E; ++e) {
      const int slot = E - 1 - e;
      table[e] = slot;
      cudaMemcpy(S.gu_packed + slot * gup, L.gu_packed + e * gup, gup, cudaMemcpyDeviceToDevice);
      cudaMemcpy(S.gu_sf + slot * gus, L.gu_sf + e * gus, gus, cudaMemcpyDeviceToDevice);
      cudaMemcpy(S.dn_packed + slot * dnp, L.dn_packed + e * dnp, dnp, cudaMemcpyDeviceToDevice);
      cudaMemcpy(S.dn_sf + slot * dns, L.dn_sf + e * dns, dns, cudaMemcpyDeviceToDevice);
      cudaMemcpy(S.gu_w_scale2 + slot, L.gu_w_scale2 + e, 4, cudaMemcpyDeviceToDevice);
      cudaMemcpy(S.gu_input_scale + slot, L.gu_input_scale + e, 4, cudaMemcpyDeviceToDevice);
      cudaMemcpy(S.dn_w_scale2 + slot, L.dn_w_scale2 + e, 4, cudaMemcpyDeviceToDevice);
      cudaMemcpy(S.dn_input_scale + slot, L.dn_input_scale + e, 4, cudaMemcpyDeviceToDevice);
    }
    int32_t* d_table; cudaMalloc(reinterpret_cast<void**>(&d_table), E * 4);
    cudaMemcpy(d_table, table.data(), E * 4, cudaMemcpyHostToDevice);
    quant::MoEResidency res(S, d_table, E);
    s = model::MoEForward(d_x, res.Layout(), X, d_y, T, k, ws, ws_bytes, nullptr, 0, 0, nullptr, -1, &res);
    if (!s.ok()) std::printf("MoEForward(slot mode): %s\n", s.message().c_str());
    CHECK(s.ok());
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    cudaMemcpy(y_slots.data(), d_y, y_slots.size() * 2, cudaMemcpyDeviceToHost);
    CHECK(std::memcmp(y_plain.data(), y_slots.data(), y_plain.size() * 2) == 0);
    CHECK(model::MoEForward(d_x, L, X, d_y, T, k, ws, ws_bytes, nullptr, 0, 0, nullptr, -1, &res).message() ==
          "slot mode: routed weights must be the residency layout");
  }
  // ---- MoEForward with the frame's gated residual write fused in: y as before, and
  // out[t, b, c] = bf16(fma(y[t, c], gate[t, b], R[t, b, c])) checked on the host
  {
    const int hc = 4;
    std::vector<uint16_t> y_plain(size_t(T) * hs), y_fused(y_plain.size());
    CHECK(model::MoEForward(d_x, L, X, d_y, T, k, ws, ws_bytes, nullptr, 0, 0).ok());
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    cudaMemcpy(y_plain.data(), d_y, y_plain.size() * 2, cudaMemcpyDeviceToHost);
    std::vector<uint16_t> res_h(size_t(T) * hc * hs), gate_h(size_t(T) * hc), out_h(res_h.size());
    for (size_t i = 0; i < res_h.size(); ++i) res_h[i] = static_cast<uint16_t>(0x3c00u + (i * 37u) % 0x300u);   // 0.0078 .. 0.5
    for (size_t i = 0; i < gate_h.size(); ++i) gate_h[i] = static_cast<uint16_t>(0x3f00u + (i * 11u) % 0x100u); // 0.5 .. 2
    uint16_t *d_res, *d_gate, *d_out;
    cudaMalloc(reinterpret_cast<void**>(&d_res), res_h.size() * 2);
    cudaMalloc(reinterpret_cast<void**>(&d_gate), gate_h.size() * 2);
    cudaMalloc(reinterpret_cast<void**>(&d_out), res_h.size() * 2);
    cudaMemcpy(d_res, res_h.data(), res_h.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(d_gate, gate_h.data(), gate_h.size() * 2, cudaMemcpyHostToDevice);
    model::GatedResidualWrite wr;
    wr.residual = d_res; wr.inject_gate = d_gate; wr.out = d_out; wr.hc = hc;
    s = model::MoEForwardAndWrite(d_x, L, X, d_y, T, k, ws, ws_bytes, wr, 0);
    if (!s.ok()) std::printf("MoEForwardAndWrite: %s\n", s.message().c_str());
    CHECK(s.ok());
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    cudaMemcpy(y_fused.data(), d_y, y_fused.size() * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(out_h.data(), d_out, out_h.size() * 2, cudaMemcpyDeviceToHost);
    CHECK(std::memcmp(y_plain.data(), y_fused.data(), y_plain.size() * 2) == 0);
    auto to_f = [](uint16_t b) { uint32_t u = uint32_t(b) << 16; float f; std::memcpy(&f, &u, 4); return f; };
    auto to_b = [](float f) { uint32_t u; std::memcpy(&u, &f, 4); u += 0x7fffu + ((u >> 16) & 1u); return uint16_t(u >> 16); };
    size_t bad = 0;
    for (int t = 0; t < T; ++t)
      for (int b = 0; b < hc; ++b)
        for (int c = 0; c < hs; ++c) {
          const size_t at = (size_t(t) * hc + b) * hs + c;
          bad += out_h[at] != to_b(std::fma(to_f(y_fused[size_t(t) * hs + c]), to_f(gate_h[size_t(t) * hc + b]), to_f(res_h[at])));
        }
    CHECK(bad == 0);
    wr.hc = 0;
    CHECK(!model::MoEForwardAndWrite(d_x, L, X, d_y, T, k, ws, ws_bytes, wr, 0).ok());
  }
  // ---- MoEForward with the stack's residual + RMSNorm step fused in, against the layer followed
  // by q4t_residual_rmsnorm_bf16: the same residual stream and the same normalised row, bit for bit
  {
    std::vector<uint16_t> res_h(size_t(T) * hs), x_a(res_h.size()), x_b(res_h.size()), h_a(res_h.size()), h_b(res_h.size());
    for (size_t i = 0; i < res_h.size(); ++i) res_h[i] = static_cast<uint16_t>(0x3c00u + (i * 53u) % 0x400u);
    uint16_t *d_xa, *d_xb, *d_ha, *d_hb;
    for (uint16_t** ptr : {&d_xa, &d_xb, &d_ha, &d_hb}) cudaMalloc(reinterpret_cast<void**>(ptr), res_h.size() * 2);
    cudaMemcpy(d_xa, res_h.data(), res_h.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(d_xb, res_h.data(), res_h.size() * 2, cudaMemcpyHostToDevice);
    CHECK(model::MoEForward(d_x, L, X, d_y, T, k, ws, ws_bytes, nullptr, 0, 0).ok());
    CHECK(q4t_residual_rmsnorm_bf16(d_xa, d_y, d_ha, T, hs, 1e-6f, nullptr) == Q4T_OK);
    model::ResidualNormWrite nw;
    nw.residual = d_xb; nw.out = d_hb; nw.eps = 1e-6f;
    s = model::MoEForwardAndNorm(d_x, L, X, d_y, T, k, ws, ws_bytes, nw, 0);
    if (!s.ok()) std::printf("MoEForwardAndNorm: %s\n", s.message().c_str());
    CHECK(s.ok());
    CHECK(cudaDeviceSynchronize() == cudaSuccess);
    cudaMemcpy(x_a.data(), d_xa, x_a.size() * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(x_b.data(), d_xb, x_b.size() * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(h_a.data(), d_ha, h_a.size() * 2, cudaMemcpyDeviceToHost);
    cudaMemcpy(h_b.data(), d_hb, h_b.size() * 2, cudaMemcpyDeviceToHost);
    CHECK(std::memcmp(x_a.data(), x_b.data(), x_a.size() * 2) == 0);
    CHECK(std::memcmp(h_a.data(), h_b.data(), h_a.size() * 2) == 0);
    nw.out = nullptr;
    CHECK(!model::MoEForwardAndNorm(d_x, L, X, d_y, T, k, ws, ws_bytes, nw, 0).ok());
  }
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
