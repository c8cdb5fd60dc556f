// MoEExtraWeights / MoEForwardWorkspaceBytes / MoEForward with the reference's
// signatures (include/q4t/model/moe.h:39-114), forwarded to the C ABI.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "q4t/quant/moe_gemm.h"
#include "q4t/quant/moe_weights.h"
#include "q4t/status.h"
#include "q4t_moe_b200.h"

namespace q4t::trace { class RouterCollector; }
namespace q4t::quant { class MoEResidency; }

namespace q4t::model {

struct MoEExtraWeights {
  int E = 0, hs = 0, shared_is = 0;
  uint16_t* gate = nullptr;
  uint16_t* shared_gu = nullptr;
  uint16_t* shared_down = nullptr;
  uint16_t* shared_gate_scalar = nullptr;
  void Free() {
    cudaFree(gate);
    cudaFree(shared_gu);
    cudaFree(shared_down);
    cudaFree(shared_gate_scalar);
    gate = shared_gu = shared_down = shared_gate_scalar = nullptr;
  }
  q4t_extra_weights Abi() const { return q4t_extra_weights{E, hs, shared_is, gate, shared_gu, shared_down, shared_gate_scalar}; }
};

struct MoEForwardDiagnostics {
  bool partition_requested = false, partition_applied = false, partition_fallback = false;
  size_t chunks = 0, singleton_chunks = 0, actual_executed_chunks = 0, actual_singleton_dispatches = 0;
  std::vector<int32_t> executed_token_rows;
};

inline size_t MoEForwardWorkspaceBytes(int T, int k, int hs, int moe_is, int shared_is, int E) {
  return q4t_moe_forward_workspace_bytes(T, k, hs, moe_is, shared_is, E);
}

// trace / residency: the router-trace hook and the slot-mode residency tier of
// the engine are not part of this library; passing them is reported as an error
// instead of being ignored.
inline Status MoEForward(const uint16_t* x, const quant::MoEWeightLayout& routed, const MoEExtraWeights& extra,
                         uint16_t* y, int T, int k, void* workspace, size_t workspace_bytes, void* /*gemm_ws*/,
                         size_t /*gemm_ws_bytes*/, cudaStream_t stream, trace::RouterCollector* trace = nullptr,
                         int /*layer_id*/ = -1, const quant::MoEResidency* residency = nullptr,
                         MoEForwardDiagnostics* diagnostics = nullptr) {
  if (diagnostics) *diagnostics = {};
  if (residency != nullptr) return Status::Fail("slot-mode residency is not supported by the B200 MoE library");
  if (trace != nullptr) return Status::Fail("router trace capture is not supported by the B200 MoE library");
  const q4t_routed_weights rw = routed.Abi();
  const q4t_extra_weights ew = extra.Abi();
  if (q4t_moe_forward(x, &rw, &ew, y, T, k, workspace, workspace_bytes, nullptr, 0, stream) != Q4T_OK)
    return Status::Fail(q4t_last_error());
  return Status();
}

}  // namespace q4t::model
