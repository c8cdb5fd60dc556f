// MoEExtraWeights / MoEForwardWorkspaceBytes / MoEForward with the reference's
// signatures (include/q4t/model/moe.h:39-114), forwarded to the C ABI.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "q4t/quant/moe_gemm.h"
#include "q4t/io/weight_loader.h"
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

// Router and shared-expert BF16 weights of one layer from the checkpoint (reference
// src/model/moe.cu:344-398): `prefix`.gate.weight [E,hs], .shared_expert.{gate,up,down}_proj
// .weight (gate rows first, then up rows, in shared_gu), .shared_expert_gate.weight [1,hs].
// A tensor of another byte size is refused.  No FP8 shadows.
inline Status LoadMoEExtra(const io::WeightLoader& loader, const std::string& prefix, int E, int hs, int shared_is,
                           MoEExtraWeights* out, cudaStream_t stream) {
  if (E <= 0 || hs <= 0 || shared_is <= 0) return Status::Fail("bad dims");
  out->E = E;
  out->hs = hs;
  out->shared_is = shared_is;
  const size_t gate_b = static_cast<size_t>(E) * hs * 2, proj_b = static_cast<size_t>(shared_is) * hs * 2;
  const size_t scalar_b = static_cast<size_t>(hs) * 2;
  if (cudaMalloc(reinterpret_cast<void**>(&out->gate), gate_b) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&out->shared_gu), 2 * proj_b) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&out->shared_down), proj_b) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&out->shared_gate_scalar), scalar_b) != cudaSuccess)
    return Status::Fail("cudaMalloc failed");
  std::vector<uint8_t> host;
  auto load = [&](const std::string& name, uint16_t* dst, size_t bytes) {
    host.resize(bytes);
    Status s = loader.ReadTensor(name, host.data(), bytes);
    if (!s.ok()) return s;
    // the staging buffer is reused by the next tensor: finish the copy first
    if (cudaMemcpyAsync(dst, host.data(), bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
      return Status::Fail("upload failed: " + name);
    return Status();
  };
  Status s;
  if (!(s = load(prefix + ".gate.weight", out->gate, gate_b)).ok()) return s;
  if (!(s = load(prefix + ".shared_expert.gate_proj.weight", out->shared_gu, proj_b)).ok()) return s;
  if (!(s = load(prefix + ".shared_expert.up_proj.weight", out->shared_gu + static_cast<size_t>(shared_is) * hs, proj_b)).ok())
    return s;
  if (!(s = load(prefix + ".shared_expert.down_proj.weight", out->shared_down, proj_b)).ok()) return s;
  return load(prefix + ".shared_expert_gate.weight", out->shared_gate_scalar, scalar_b);
}

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
