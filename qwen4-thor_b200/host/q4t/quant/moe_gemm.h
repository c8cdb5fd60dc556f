// MoEWorkspace / MoERoutedForward / MoEDeviceDecode[Multi] / Fp4Gemm with the
// reference's signatures (include/q4t/quant/moe_gemm.h:34-74,
// include/q4t/quant/moe_decode.h:11-36, include/q4t/quant/fp4_gemm.h:58-213),
// forwarded to the C ABI.  The cuBLASLt workspace arguments are accepted and
// ignored: no library GEMM runs on this path.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

#include "q4t/quant/moe_weights.h"
#include "q4t/status.h"
#include "q4t_moe_b200.h"

namespace q4t::quant {

// Largest expert count the engine's router supports (src/model/moe.cu:141-145);
// RequiredBytes has no E argument, so workspaces are sized for it.
constexpr int kMoEMaxExperts = 512;

struct MoEWorkspace {
  size_t a_packed_bytes = 0, a_sf_bytes = 0, gu_out_bytes = 0, dn_out_bytes = 0;
  size_t TotalBytes() const { return a_packed_bytes + a_sf_bytes + gu_out_bytes + dn_out_bytes; }
  // Includes this implementation's routing tables and tile-local scale blocks,
  // which follow the four reference regions.
  static size_t RequiredBytes(int M, int k, int hs, int moe_is) {
    return q4t_moe_routed_workspace_bytes(M, k, hs, moe_is, kMoEMaxExperts);
  }
  uint8_t* a_packed = nullptr;
  uint8_t* a_sf = nullptr;
  uint16_t* gu_out = nullptr;
  uint16_t* dn_out = nullptr;
  void Init(uint8_t* base) {
    size_t off = 0;
    a_packed = base + off;
    off += a_packed_bytes;
    a_sf = base + off;
    off += a_sf_bytes;
    gu_out = reinterpret_cast<uint16_t*>(base + off);
    off += gu_out_bytes;
    dn_out = reinterpret_cast<uint16_t*>(base + off);
  }
};

inline Status MoERoutedForward(const uint16_t* x, const int32_t* expert_ids, const float* router_w, float* y,
                               const MoEWeightLayout& weights, void* workspace, void* /*gemm_ws*/,
                               size_t /*gemm_ws_bytes*/, int M, int k, cudaStream_t stream) {
  const q4t_routed_weights w = weights.Abi();
  // the reference takes no workspace size: the caller promised RequiredBytes()
  const size_t bytes = q4t_moe_routed_workspace_bytes(M, k, w.hs, w.moe_is, w.E);
  if (q4t_moe_routed_forward(x, expert_ids, router_w, y, &w, workspace, bytes, M, k, 0, stream) != Q4T_OK)
    return Status::Fail(q4t_last_error());
  return Status();
}

inline Status MoEDeviceDecode(const uint16_t* x, const int32_t* expert_ids, const float* router_w, float* y,
                              const MoEWeightLayout& weights, const MoEWorkspace& ws, void* gemm_ws,
                              size_t gemm_ws_bytes, cudaStream_t stream) {
  return MoERoutedForward(x, expert_ids, router_w, y, weights, ws.a_packed, gemm_ws, gemm_ws_bytes, 1, 10, stream);
}
inline Status MoEDeviceDecodeMulti(const uint16_t* x, const int32_t* expert_ids, const float* router_w, float* y,
                                   const MoEWeightLayout& weights, const MoEWorkspace& ws, void* gemm_ws,
                                   size_t gemm_ws_bytes, int T, int k, cudaStream_t stream) {
  return MoERoutedForward(x, expert_ids, router_w, y, weights, ws.a_packed, gemm_ws, gemm_ws_bytes, T, k, stream);
}

struct Fp4GemmResult {
  int status = 1;  // 0 = success, as CUBLAS_STATUS_SUCCESS
  bool has_algo = false;
};
template <typename OutT>
inline Fp4GemmResult Fp4Gemm(const uint8_t* w_packed, const uint8_t* w_sf, const uint8_t* a_packed,
                             const uint8_t* a_sf, OutT* out, int M, int N, int K, float inv_w_global,
                             float inv_a_global, void* /*workspace*/, size_t /*workspace_bytes*/,
                             cudaStream_t stream) {
  static_assert(std::is_same<OutT, float>::value || std::is_same<OutT, uint16_t>::value,
                "Fp4Gemm output must be float (f32) or uint16_t (bf16)");
  Fp4GemmResult r;
  const int rc = q4t_fp4_gemm(w_packed, w_sf, a_packed, a_sf, out, std::is_same<OutT, uint16_t>::value ? 1 : 0, M, N,
                              K, inv_w_global, inv_a_global, stream);
  r.status = rc == Q4T_OK ? 0 : 1;
  r.has_algo = rc == Q4T_OK;
  return r;
}

}  // namespace q4t::quant
