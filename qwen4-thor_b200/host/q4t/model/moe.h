// MoEExtraWeights / MoEForwardWorkspaceBytes / MoEForward with the reference's
// signatures (include/q4t/model/moe.h:39-114), forwarded to the C ABI.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "q4t/quant/moe_gemm.h"
#include "q4t/io/weight_loader.h"
#include "q4t/quant/moe_residency.h"
#include "q4t/quant/moe_weights.h"
#include "q4t/status.h"
#include "q4t/trace/router_collector.h"
#include "q4t_moe_b200.h"

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

// trace: the router-trace observer.  As in the reference (src/model/moe.cu:485-488) the
// collector receives the ORIGINAL selected expert ids of this layer through
// CaptureLayer(layer_id, ids, T, k, stream), a device-to-device copy ordered on the stream;
// the ids are read from the workspace's expert_ids region, which nothing overwrites after
// the top-k, so the copy is enqueued behind the layer.
// residency: slot mode (include/q4t/model/moe.h:96-103 of the reference).  `routed` must be
// residency->Layout() (E = slot count); the selected experts are mapped to slots on the
// device through residency->DeviceSlotOfExpert() with no host round trip, and experts
// that are not resident contribute nothing (the engine's tier decides what is resident).
// The gated residual write that follows the layer (GatedResidualFrame::Write,
// src/model/decoder_layer.cu:708 of the reference), when it is to be fused into the layer's
// last kernel: out[t, b, :] = bf16(residual[t, b, :] + y[t, :] * inject_gate[t, b]).
struct GatedResidualWrite {
  const uint16_t* residual = nullptr;     // [T, hc, hs] bf16, the frame's residual
  const uint16_t* inject_gate = nullptr;  // [T, hc] bf16, the frame's prepared gate
  uint16_t* out = nullptr;                // [T, hc, hs] bf16
  int hc = 0;
};

// The step between this layer and the next in a decode stack without hyper-connections,
// residual <- bf16(residual + y) and out <- RMSNorm(residual) (no weight), when it is to be
// fused into the layer's last kernel instead of running as a launch of its own.
struct ResidualNormWrite {
  uint16_t* residual = nullptr;   // [T, hs] bf16, the residual stream (read and written)
  uint16_t* out = nullptr;        // [T, hs] bf16, the next layer's normalised input
  float eps = 1e-6f;
};

namespace detail {
inline Status RunMoEForward(const uint16_t* x, const quant::MoEWeightLayout& routed, const MoEExtraWeights& extra,
                            uint16_t* y, int T, int k, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                            trace::RouterCollector* trace, int layer_id, const quant::MoEResidency* residency,
                            MoEForwardDiagnostics* diagnostics, const GatedResidualWrite* write,
                            const ResidualNormWrite* norm = nullptr) {
  if (diagnostics) *diagnostics = {};
  const q4t_routed_weights rw = routed.Abi();
  const q4t_extra_weights ew = extra.Abi();
  q4t_forward_options opt{};
  if (residency != nullptr) {
    if (residency->Slots() < k) return Status::Fail("residency slots below top-k");  // moe.cu:507
    if (residency->Slots() != routed.E || !routed.slot_mode)
      return Status::Fail("slot mode: routed weights must be the residency layout");
    opt.slot_of_expert = residency->DeviceSlotOfExpert();
  }
  if (write != nullptr && write->hc > 0) {
    opt.hc_count = write->hc;
    opt.hc_residual = write->residual;
    opt.hc_inject_gate = write->inject_gate;
    opt.hc_out = write->out;
  }
  if (norm != nullptr && norm->residual != nullptr) {
    opt.norm_residual = norm->residual;
    opt.norm_out = norm->out;
    opt.norm_eps = norm->eps;
  }
  if (residency != nullptr || opt.hc_count > 0 || opt.norm_residual != nullptr) {
    if (q4t_moe_forward_ex(x, &rw, &ew, y, T, k, workspace, workspace_bytes, &opt, stream) != Q4T_OK)
      return Status::Fail(q4t_last_error());
  } else if (q4t_moe_forward(x, &rw, &ew, y, T, k, workspace, workspace_bytes, nullptr, 0, stream) != Q4T_OK) {
    return Status::Fail(q4t_last_error());
  }
  if (trace != nullptr && T > 0) {
    q4t_forward_ws_layout F;
    if (q4t_moe_forward_workspace_layout(T, k, ew.hs, rw.moe_is, ew.shared_is, ew.E, &F) != Q4T_OK)
      return Status::Fail(q4t_last_error());
    const int32_t* ids = reinterpret_cast<const int32_t*>(static_cast<const uint8_t*>(workspace) + F.expert_ids);
    Status s = trace->CaptureLayer(static_cast<uint32_t>(layer_id), ids, T, k, stream);
    if (!s.ok()) return s;
  }
  return Status();
}
}  // namespace detail

inline Status MoEForward(const uint16_t* x, const quant::MoEWeightLayout& routed, const MoEExtraWeights& extra,
                         uint16_t* y, int T, int k, void* workspace, size_t workspace_bytes, void* /*gemm_ws*/,
                         size_t /*gemm_ws_bytes*/, cudaStream_t stream, trace::RouterCollector* trace = nullptr,
                         int layer_id = -1, const quant::MoEResidency* residency = nullptr,
                         MoEForwardDiagnostics* diagnostics = nullptr) {
  return detail::RunMoEForward(x, routed, extra, y, T, k, workspace, workspace_bytes, stream, trace, layer_id, residency,
                               diagnostics, nullptr);
}

// MoEForward followed by the frame's Write in one call (no counterpart in the reference, which
// runs CombineWithGateKernel as a launch of its own): the call site in DecoderLayerForward
// passes the frame's residual, gate and branch count and drops its mlp_frame.Write launch.
inline Status MoEForwardAndWrite(const uint16_t* x, const quant::MoEWeightLayout& routed, const MoEExtraWeights& extra,
                                 uint16_t* y, int T, int k, void* workspace, size_t workspace_bytes,
                                 const GatedResidualWrite& write, cudaStream_t stream,
                                 trace::RouterCollector* trace = nullptr, int layer_id = -1,
                                 const quant::MoEResidency* residency = nullptr) {
  if (write.hc <= 0 || !write.residual || !write.inject_gate || !write.out)
    return Status::Fail("gated residual write needs a residual, a gate and an output");
  return detail::RunMoEForward(x, routed, extra, y, T, k, workspace, workspace_bytes, stream, trace, layer_id, residency,
                               nullptr, &write);
}

// MoEForward followed by the residual add and the next layer's RMSNorm in one call.
inline Status MoEForwardAndNorm(const uint16_t* x, const quant::MoEWeightLayout& routed, const MoEExtraWeights& extra,
                                uint16_t* y, int T, int k, void* workspace, size_t workspace_bytes,
                                const ResidualNormWrite& norm, cudaStream_t stream,
                                trace::RouterCollector* trace = nullptr, int layer_id = -1,
                                const quant::MoEResidency* residency = nullptr) {
  if (!norm.residual || !norm.out) return Status::Fail("residual + RMSNorm write needs a residual and an output");
  return detail::RunMoEForward(x, routed, extra, y, T, k, workspace, workspace_bytes, stream, trace, layer_id, residency,
                               nullptr, nullptr, &norm);
}

}  // namespace q4t::model
