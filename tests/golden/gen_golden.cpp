// Generates golden vectors for the NVFP4 MoE path by running the REFERENCE's
// own header code (include/q4t/quant/format.h, swizzle.h, included from the
// reference tree with -I) on the inputs of the reference's unit tests:
//   * act-quant case of tests/quant_fp4_test.cpp:303-361 (M=5, K=64,
//     std::mt19937(7), normal(0,1), global scale 0.00167);
//   * W4A4 GEMM cases of tests/quant_fp4_test.cpp:367-471 (std::mt19937(1234),
//     shapes 640x2560 and 2560x640, weight_scale_2 0.29, input_scale 0.41),
//     all four M of that test (1, 8, 64, 256); the expected value is that
//     test's CPU check (dequantise both sides, sequential fp32 dot).  To keep
//     the fixture small the M = 256 cases store the expected rows 0, 8, 16, ...
//     only (gemm*_m256_out_rows8); the operands are stored in full;
//   * encoder tables: FloatToE4m3 over every non-negative bf16 bit pattern and
//     FloatToE2m1Code over every bf16 bit pattern.
// The quantisation loop below follows HostQuantize (tests/quant_fp4_test.cpp:
// 69-97) but calls the reference's primitives for every rounding decision.
// Output: raw little-endian blobs described by a manifest on stdout; the
// Python driver beside this file packs them into golden.npz.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <random>
#include <string>
#include <vector>

#include "q4t/quant/format.h"
#include "q4t/quant/swizzle.h"

using namespace q4t::quant;

static void dump(const std::string& dir, const char* name, const void* p, size_t bytes,
                 const char* dtype, const std::vector<size_t>& shape) {
  std::string path = dir + "/" + name + ".bin";
  FILE* f = std::fopen(path.c_str(), "wb");
  std::fwrite(p, 1, bytes, f);
  std::fclose(f);
  std::printf("%s %s", name, dtype);
  for (size_t d : shape) std::printf(" %zu", d);
  std::printf("\n");
}

static float bf16_round(float v, uint16_t* bits) {
  uint32_t u;
  std::memcpy(&u, &v, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  u &= 0xffff0000u;
  if (bits) *bits = static_cast<uint16_t>(u >> 16);
  float r;
  std::memcpy(&r, &u, 4);
  return r;
}

struct Q {
  std::vector<uint8_t> packed, sf;
};
static Q quantize(const std::vector<float>& v, int rows, int K, float gs) {
  Q q;
  const int groups = K / 16;
  q.packed.assign(size_t(rows) * K / 2, 0);
  q.sf.assign(size_t(rows) * groups, 0);
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < groups; ++g) {
      const float* a = &v[size_t(r) * K + g * 16];
      float gmax = 0.0f;
      for (int j = 0; j < 16; ++j) gmax = std::fmax(gmax, std::fabs(a[j]));
      const float block = gmax > 0.0f ? gmax / 6.0f : 1.0f;
      const uint8_t sf = FloatToE4m3(block / gs);
      const float eff = E4m3ToFloat(sf) * gs;
      const float inv = eff > 0.0f ? 1.0f / eff : 0.0f;
      q.sf[size_t(r) * groups + g] = sf;
      for (int j = 0; j < 8; ++j) {
        const int lo = FloatToE2m1Code(a[2 * j] * inv);
        const int hi = FloatToE2m1Code(a[2 * j + 1] * inv);
        q.packed[size_t(r) * (K / 2) + g * 8 + j] = uint8_t((hi << 4) | (lo & 0xF));
      }
    }
  return q;
}
static std::vector<float> dequant(const Q& q, int rows, int K, float gs) {
  const int groups = K / 16;
  std::vector<float> out(size_t(rows) * K);
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < groups; ++g) {
      const float s = E4m3ToFloat(q.sf[size_t(r) * groups + g]) * gs;
      for (int j = 0; j < 8; ++j) {
        const uint8_t b = q.packed[size_t(r) * (K / 2) + g * 8 + j];
        out[size_t(r) * K + g * 16 + 2 * j] = E2m1ToFloat(b & 0xF) * s;
        out[size_t(r) * K + g * 16 + 2 * j + 1] = E2m1ToFloat(b >> 4) * s;
      }
    }
  return out;
}

int main(int argc, char** argv) {
  const std::string dir = argc > 1 ? argv[1] : ".";
  {  // act-quant case
    const int M = 5, K = 64;
    std::mt19937 rng(7);
    std::normal_distribution<float> dist(0.0f, 1.0f);
    std::vector<float> a(size_t(M) * K), af(a.size());
    std::vector<uint16_t> abits(a.size());
    for (auto& x : a) x = dist(rng);
    for (size_t i = 0; i < a.size(); ++i) af[i] = bf16_round(a[i], &abits[i]);
    const float gs = 0.00167f;
    Q q = quantize(af, M, K, gs);
    std::vector<uint8_t> sw = SwizzleSf(q.sf.data(), M, K);
    dump(dir, "actq_x_bf16", abits.data(), abits.size() * 2, "u2", {size_t(M), size_t(K)});
    dump(dir, "actq_packed", q.packed.data(), q.packed.size(), "u1", {size_t(M), size_t(K / 2)});
    dump(dir, "actq_sf_rm", q.sf.data(), q.sf.size(), "u1", {size_t(M), size_t(K / 16)});
    dump(dir, "actq_sf_swz", sw.data(), sw.size(), "u1", {sw.size()});
  }
  {  // GEMM cases
    const float iw = 0.29f, ia = 0.41f;
    const int shapes[2][2] = {{640, 2560}, {2560, 640}};
    const int Ms[4] = {1, 8, 64, 256};
    std::mt19937 rng(1234);
    std::normal_distribution<float> dist(0.0f, 1.0f);
    for (int s = 0; s < 2; ++s) {
      const int N = shapes[s][0], K = shapes[s][1];
      std::vector<float> w(size_t(N) * K);
      for (auto& x : w) x = dist(rng);
      Q wq = quantize(w, N, K, iw);
      std::vector<uint8_t> wsw = SwizzleSf(wq.sf.data(), N, K);
      std::vector<float> wd = dequant(wq, N, K, iw);
      char nm[64];
      std::snprintf(nm, sizeof nm, "gemm%d_w_packed", s);
      dump(dir, nm, wq.packed.data(), wq.packed.size(), "u1", {size_t(N), size_t(K / 2)});
      std::snprintf(nm, sizeof nm, "gemm%d_w_sf_swz", s);
      dump(dir, nm, wsw.data(), wsw.size(), "u1", {wsw.size()});
      for (int M : Ms) {
        std::vector<float> a(size_t(M) * K);
        for (auto& x : a) x = dist(rng);  // consumed for every M to keep the stream in step
        Q aq = quantize(a, M, K, ia);
        std::vector<uint8_t> asw = SwizzleSf(aq.sf.data(), M, K);
        std::vector<float> ad = dequant(aq, M, K, ia);
        const int row_step = M > 64 ? 8 : 1;  // rows of the expected output that are stored
        const int rows_out = (M + row_step - 1) / row_step;
        std::vector<float> out(size_t(rows_out) * N);
        for (int mi = 0; mi < rows_out; ++mi) {
          const int m = mi * row_step;
          for (int n = 0; n < N; ++n) {
            float acc = 0.0f;
            for (int k = 0; k < K; ++k) acc += ad[size_t(m) * K + k] * wd[size_t(n) * K + k];
            out[size_t(mi) * N + n] = acc;
          }
        }
        std::snprintf(nm, sizeof nm, "gemm%d_m%d_a_packed", s, M);
        dump(dir, nm, aq.packed.data(), aq.packed.size(), "u1", {size_t(M), size_t(K / 2)});
        std::snprintf(nm, sizeof nm, "gemm%d_m%d_a_sf_swz", s, M);
        dump(dir, nm, asw.data(), asw.size(), "u1", {asw.size()});
        std::snprintf(nm, sizeof nm, row_step == 1 ? "gemm%d_m%d_out" : "gemm%d_m%d_out_rows8", s, M);
        dump(dir, nm, out.data(), out.size() * 4, "f4", {size_t(rows_out), size_t(N)});
      }
    }
  }
  {  // encoder tables over bf16 inputs
    std::vector<uint8_t> e4(32768), e2(65536);
    for (uint32_t b = 0; b < 65536; ++b) {
      const uint32_t u = b << 16;
      float f;
      std::memcpy(&f, &u, 4);
      if (b < 32768) e4[b] = (f != f) ? 0xFF : FloatToE4m3(f);
      e2[b] = (f != f) ? 0xFF : uint8_t(FloatToE2m1Code(f));
    }
    dump(dir, "e4m3_of_bf16", e4.data(), e4.size(), "u1", {e4.size()});
    dump(dir, "e2m1_of_bf16", e2.data(), e2.size(), "u1", {e2.size()});
  }
  return 0;
}
