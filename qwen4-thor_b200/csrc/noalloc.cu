// Routed-expert forward for callers that cannot allocate device memory.
//
// Some hosts seal their device-memory budget once start-up is over: every
// byte is accounted for (weights, KV pages, a fixed reservation) and any later
// cudaMalloc either fails against the quota or is simply not allowed from the
// calling context (a decode loop that must never block in the allocator, a
// verification tool attached to a process whose memory is fully reserved).
// Such a caller has no workspace to hand to q4t_moe_routed_forward.  This
// file gives it one that already exists: a fixed scratch array that lives in
// the library's own device image.
//
// The array is a module-scope __device__ object, so each GPU that loads the
// library carries its Q4T_NOALLOC_SCRATCH_BYTES from load until exit whether
// or not this entry point is ever used.  Host code must not use the array's
// name as a pointer: on the host that name is only a handle for the runtime.
// The device address is obtained once per device with cudaGetSymbolAddress,
// with that device current, and that address is what the kernels receive.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "../../include/q4t_moe_b200.h"

int q4t_internal_fail(int code, const char* msg);  // api.cu: sets the thread's error message

namespace {

static __device__ __align__(256) unsigned char g_noalloc_scratch[Q4T_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 16;
struct ScratchSlot {
  bool ready = false;
  void* device_ptr = nullptr;
};
ScratchSlot g_slot[kMaxDevices];
std::mutex g_slot_mutex;

// Device address of the scratch array on the current device; resolved on the
// first call per device.
int scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return q4t_internal_fail(Q4T_ERR_DEVICE, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return q4t_internal_fail(Q4T_ERR_DEVICE, "device index out of range");
  std::lock_guard<std::mutex> lock(g_slot_mutex);
  ScratchSlot& s = g_slot[dev];
  if (!s.ready) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      const std::string msg = std::string("cudaGetSymbolAddress(no-alloc scratch): ") + cudaGetErrorString(e);
      return q4t_internal_fail(Q4T_ERR_CUDA, msg.c_str());
    }
    s.device_ptr = p;
    s.ready = true;
  }
  *out = s.device_ptr;
  return Q4T_OK;
}

}  // namespace

extern "C" int32_t q4t_moe_routed_forward_noalloc(const uint16_t* x, const int32_t* expert_ids,
                                                  const float* router_w, float* y,
                                                  const q4t_routed_weights* weights, int32_t M, int32_t k,
                                                  uint32_t flags, void* stream) {
  if (!weights) return q4t_internal_fail(Q4T_ERR_INVALID, "null weights");
  if (M <= 0 || k <= 0 || weights->E <= 0 || weights->hs <= 0 || weights->moe_is <= 0)
    return q4t_internal_fail(Q4T_ERR_INVALID, "invalid MoE forward dims");
  const size_t need = q4t_moe_routed_workspace_bytes(M, k, weights->hs, weights->moe_is, weights->E);
  if (need == 0 || need > static_cast<size_t>(Q4T_NOALLOC_SCRATCH_BYTES)) {
    const std::string msg = "this batch needs " + std::to_string(need) +
                            " bytes of scratch; the built-in scratch of the no-allocation entry point holds " +
                            std::to_string(static_cast<size_t>(Q4T_NOALLOC_SCRATCH_BYTES)) +
                            " (use q4t_moe_routed_forward with a caller-owned workspace)";
    return q4t_internal_fail(Q4T_ERR_WORKSPACE, msg.c_str());
  }
  void* scratch = nullptr;
  const int rc = scratch_address(&scratch);
  if (rc != Q4T_OK) return rc;
  // The shared routine clears the status words it relies on at the start of
  // every call; every other table in the scratch is rewritten before it is
  // read, so stale contents of an earlier call are never consumed.
  return q4t_moe_routed_forward(x, expert_ids, router_w, y, weights, scratch, Q4T_NOALLOC_SCRATCH_BYTES, M, k,
                                flags, stream);
}

extern "C" int32_t q4t_moe_noalloc_status(int32_t M, int32_t k, int32_t hs, int32_t moe_is, int32_t E) {
  const size_t need = q4t_moe_routed_workspace_bytes(M, k, hs, moe_is, E);
  if (need == 0 || need > static_cast<size_t>(Q4T_NOALLOC_SCRATCH_BYTES))
    return q4t_internal_fail(Q4T_ERR_INVALID, "these dimensions do not fit the built-in scratch");
  void* scratch = nullptr;
  const int rc = scratch_address(&scratch);
  if (rc != Q4T_OK) return rc;
  return q4t_moe_workspace_status(scratch, M, k, hs, moe_is, E);
}
