// Thin extern "C" wrapper over the REFERENCE's own GPU implementation of the routed experts,
// compiled from the reference tree where it lies: src/quant/moe_gemm.cu (MoERoutedForward,
// its gather-quantise / SwiGLU-quantise / combine kernels), src/quant/act_quant.cu and
// src/quant/lt_cache.cpp, i.e. the per-expert cuBLASLt NVFP4 GEMM loop the engine runs.
// The resulting oracle/_ref/libq4t_ref_gpu.so is test infrastructure only: the GPU tests
// run it on the same inputs as this repository's kernels and compare gu_out / dn_out / y bit
// for bit, which pins the tensor-core GEMM parity that the CPU oracle can only assert against
// the reference's documents.  Nothing of the product links or loads it.
//
// The BF16 routed experts of the MTP draft layer come from src/mtp/moe_bf16.cu with the GEMV
// helpers its Bf16Gemm dispatches to (src/model/gemv.cu, gemv_hc_inject.cu, small_m_gemm.cu).
//
// src/quant/moe_decode.cu does not compile with CUDA 12.9 (it needs cuBLASLt's grouped-layout
// API); its two entry points are only reached for M <= 8 at hidden 2560 / intermediate 640 and
// are stubbed here to fail loudly.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>
#include <string>

#include "q4t/mtp/moe_bf16.h"
#include "q4t/quant/act_quant.h"
#include "q4t/quant/fp4_gemm.h"
#include "q4t/quant/moe_decode.h"
#include "q4t/quant/moe_gemm.h"
#include "q4t/quant/moe_weights.h"

namespace q4t::quant {
Status MoEDeviceDecode(const uint16_t*, const int32_t*, const float*, float*, const MoEWeightLayout&,
                       const MoEWorkspace&, void*, size_t, cudaStream_t) {
  return Status::Fail("MoEDeviceDecode is not part of this build of the reference");
}
Status MoEDeviceDecodeMulti(const uint16_t*, const int32_t*, const float*, float*, const MoEWeightLayout&,
                            const MoEWorkspace&, void*, size_t, int, int, cudaStream_t) {
  return Status::Fail("MoEDeviceDecodeMulti is not part of this build of the reference");
}
}  // namespace q4t::quant

// LoadMoeBf16 (same file as the BF16 forward) reads a checkpoint through the reference's
// loader, which is not part of this build; the tests hand over device tensors directly.
namespace q4t::io {
Status WeightLoader::LoadTensorToDevice(const std::string&, void*, size_t, cudaStream_t) const {
  return Status::Fail("the checkpoint loader is not part of this build of the reference");
}
}  // namespace q4t::io

namespace {
thread_local std::string g_msg;
}

extern "C" {

const char* ref_gpu_last_error() { return g_msg.c_str(); }

size_t ref_gpu_workspace_bytes(int M, int k, int hs, int moe_is) {
  return q4t::quant::MoEWorkspace::RequiredBytes(M, k, hs, moe_is);
}

// Offsets of the four regions MoERoutedForward leaves in its workspace.
void ref_gpu_workspace_regions(int M, int k, int hs, int moe_is, size_t out[4]) {
  const size_t R = static_cast<size_t>(M) * k;
  out[0] = 0;
  out[1] = R * (hs / 2);
  out[2] = out[1] + q4t::quant::SfBufferSize(static_cast<int>(R), hs);
  out[3] = out[2] + R * (2 * moe_is) * 2;
}

// All pointers except the four *_h tables are device pointers.
int ref_gpu_moe_routed_forward(const uint16_t* x, const int32_t* ids, const float* rw, float* y, int E, int hs,
                               int moe_is, uint8_t* gu_packed, uint8_t* gu_sf, uint8_t* dn_packed, uint8_t* dn_sf,
                               float* gu_ws2, float* gu_in, float* dn_ws2, float* dn_in, const float* gu_ws2_h,
                               const float* gu_in_h, const float* dn_ws2_h, const float* dn_in_h, void* workspace,
                               void* gemm_ws, size_t gemm_ws_bytes, int M, int k, void* stream) {
  q4t::quant::MoEWeightLayout L;
  L.E = E;
  L.hs = hs;
  L.moe_is = moe_is;
  L.gu_packed = gu_packed;
  L.gu_sf = gu_sf;
  L.dn_packed = dn_packed;
  L.dn_sf = dn_sf;
  L.gu_w_scale2 = gu_ws2;
  L.gu_input_scale = gu_in;
  L.dn_w_scale2 = dn_ws2;
  L.dn_input_scale = dn_in;
  L.gu_w_scale2_h.assign(gu_ws2_h, gu_ws2_h + E);
  L.gu_input_scale_h.assign(gu_in_h, gu_in_h + E);
  L.dn_w_scale2_h.assign(dn_ws2_h, dn_ws2_h + E);
  L.dn_input_scale_h.assign(dn_in_h, dn_in_h + E);
  q4t::Status s = q4t::quant::MoERoutedForward(x, ids, rw, y, L, workspace, gemm_ws, gemm_ws_bytes, M, k,
                                               static_cast<cudaStream_t>(stream));
  if (!s.ok()) {
    g_msg = s.message();
    return 1;
  }
  return 0;
}

// The reference's Fp4Gemm<uint16_t> / Fp4Gemm<float> (cuBLASLt NVFP4 matmul).  Returns the
// cuBLAS status (0 = success); *has_algo tells whether the heuristic found an algorithm.
int ref_gpu_fp4_gemm(const uint8_t* w_packed, const uint8_t* w_sf, const uint8_t* a_packed, const uint8_t* a_sf,
                     void* out, int out_is_bf16, int M, int N, int K, float inv_w, float inv_a, void* gemm_ws,
                     size_t gemm_ws_bytes, int* has_algo, void* stream) {
  q4t::quant::Fp4GemmResult r =
      out_is_bf16 ? q4t::quant::Fp4Gemm<uint16_t>(w_packed, w_sf, a_packed, a_sf, static_cast<uint16_t*>(out), M, N, K,
                                                  inv_w, inv_a, gemm_ws, gemm_ws_bytes, static_cast<cudaStream_t>(stream))
                  : q4t::quant::Fp4Gemm<float>(w_packed, w_sf, a_packed, a_sf, static_cast<float*>(out), M, N, K, inv_w,
                                               inv_a, gemm_ws, gemm_ws_bytes, static_cast<cudaStream_t>(stream));
  if (has_algo) *has_algo = r.has_algo ? 1 : 0;
  return static_cast<int>(r.status);
}

// The reference's BF16 routed experts of the MTP draft layer (src/mtp/moe_bf16.cu:271-426:
// per-expert gather, cuBLASLt / GEMV BF16 projections, SwiGLU, router-weighted atomicAdd into
// y).  gu [E, 2*moe_is, hs] and down [E, hs, moe_is] are device bf16; y fp32 [M, hs] zeroed by
// the caller.  The call synchronises the stream once (the reference reads the counts back).
size_t ref_gpu_moe_bf16_workspace_bytes(int M, int k, int hs, int moe_is, int E) {
  return q4t::mtp::MoeBf16WorkspaceBytes(M, k, hs, moe_is, E);
}
int ref_gpu_moe_bf16_routed_forward(const uint16_t* x, const int32_t* ids, const float* rw, float* y, int E, int hs,
                                    int moe_is, uint16_t* gu, uint16_t* down, void* workspace, void* gemm_ws,
                                    size_t gemm_ws_bytes, int M, int k, void* stream) {
  q4t::mtp::MoeBf16Weights W;
  W.E = E;
  W.hs = hs;
  W.moe_is = moe_is;
  W.gu = gu;
  W.down = down;
  q4t::Status s = q4t::mtp::MoeBf16RoutedForward(x, ids, rw, y, W, workspace, gemm_ws, gemm_ws_bytes, M, k,
                                                 static_cast<cudaStream_t>(stream));
  W.gu = nullptr;   // borrowed: nothing for the destructor-less struct to release
  W.down = nullptr;
  if (!s.ok()) {
    g_msg = s.message();
    return 1;
  }
  return 0;
}

int ref_gpu_quantize_activation(const uint16_t* bf16, uint8_t* packed, uint8_t* sf, int M, int K, float global_scale,
                                void* stream) {
  return static_cast<int>(
      q4t::quant::QuantizeActivationToFp4Async(bf16, packed, sf, M, K, global_scale, static_cast<cudaStream_t>(stream)));
}
}
