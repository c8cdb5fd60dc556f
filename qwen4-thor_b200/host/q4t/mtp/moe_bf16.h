// The MTP draft layer's BF16 MoE with the reference's signatures (include/q4t/mtp/
// moe_bf16.h:36-123), inline on the C ABI.  gemm_ws / gemm_ws_bytes are accepted and
// ignored (no library GEMM on the path).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

#include "q4t/io/weight_loader.h"
#include "q4t/model/moe.h"
#include "q4t/status.h"
#include "q4t_moe_b200.h"

namespace q4t::mtp {

struct MoeBf16Weights {
  int E = 0, hs = 0, moe_is = 0;
  uint16_t* gu = nullptr;    // [E, 2*moe_is, hs]
  uint16_t* down = nullptr;  // [E, hs, moe_is]
  void Free() {
    cudaFree(gu);
    cudaFree(down);
    gu = down = nullptr;
  }
  q4t_bf16_expert_weights Abi() const { return q4t_bf16_expert_weights{E, hs, moe_is, 0, gu, down}; }
};

// {prefix}.experts.gate_up_proj ([E, 2*moe_is, hs]) and {prefix}.experts.down_proj ([E, hs, moe_is]),
// read in slices of a few experts so that the host staging buffer stays small.
inline Status LoadMoeBf16(const io::WeightLoader& loader, const std::string& prefix, int E, int hs, int moe_is,
                          MoeBf16Weights* out, cudaStream_t stream) {
  if (E <= 0 || hs <= 0 || moe_is <= 0) return Status::Fail("bad dims");
  out->E = E;
  out->hs = hs;
  out->moe_is = moe_is;
  const size_t gu_b = static_cast<size_t>(E) * 2 * moe_is * hs * 2, dn_b = static_cast<size_t>(E) * hs * moe_is * 2;
  if (cudaMalloc(reinterpret_cast<void**>(&out->gu), gu_b) != cudaSuccess ||
      cudaMalloc(reinterpret_cast<void**>(&out->down), dn_b) != cudaSuccess)
    return Status::Fail("cudaMalloc failed");
  std::vector<uint8_t> host;
  auto load = [&](const std::string& name, uint16_t* dst, size_t bytes) {
    const io::TensorInfo* t = loader.FindTensor(name);
    if (!t) return Status::Fail("missing tensor: " + name);
    if (t->dtype != io::Dtype::kBF16 || t->byte_size() != bytes) return Status::Fail("dtype/size mismatch: " + name);
    host.resize(bytes);
    Status s = loader.ReadTensor(name, host.data(), bytes);
    if (!s.ok()) return s;
    if (cudaMemcpyAsync(dst, host.data(), bytes, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
        cudaStreamSynchronize(stream) != cudaSuccess)
      return Status::Fail("upload failed: " + name);
    return Status();
  };
  Status s = load(prefix + ".experts.gate_up_proj", out->gu, gu_b);
  if (!s.ok()) return s;
  return load(prefix + ".experts.down_proj", out->down, dn_b);
}

inline size_t MoeBf16WorkspaceBytes(int M, int k, int hs, int moe_is, int E) {
  return q4t_moe_bf16_workspace_bytes(M, k, hs, moe_is, E);
}

inline Status MoeBf16RoutedForward(const uint16_t* x, const int32_t* expert_ids, const float* router_w, float* y,
                                   const MoeBf16Weights& weights, void* workspace, void* /*gemm_ws*/,
                                   size_t /*gemm_ws_bytes*/, int M, int k, cudaStream_t stream) {
  const q4t_bf16_expert_weights w = weights.Abi();
  if (q4t_moe_bf16_routed_forward(x, expert_ids, router_w, y, &w, workspace,
                                  q4t_moe_bf16_workspace_bytes(M, k, weights.hs, weights.moe_is, weights.E), M, k,
                                  stream) != Q4T_OK)
    return Status::Fail(q4t_last_error());
  return Status();
}

// workspace_bytes must be at least q4t_moe_bf16_forward_workspace_bytes(T, k, hs, moe_is, shared_is, E).
inline Status MoeBf16Forward(const uint16_t* x, const MoeBf16Weights& routed, const model::MoEExtraWeights& extra,
                             uint16_t* y, int T, int k, void* workspace, size_t workspace_bytes, void* /*gemm_ws*/,
                             size_t /*gemm_ws_bytes*/, cudaStream_t stream) {
  const q4t_bf16_expert_weights w = routed.Abi();
  const q4t_extra_weights ew = extra.Abi();
  if (q4t_moe_bf16_forward(x, &w, &ew, y, T, k, workspace, workspace_bytes, stream) != Q4T_OK)
    return Status::Fail(q4t_last_error());
  return Status();
}

}  // namespace q4t::mtp
