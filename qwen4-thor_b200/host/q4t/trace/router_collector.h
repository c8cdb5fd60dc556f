// Stand-in for the engine's router-trace collector (include/q4t/trace/router_collector.h of
// the reference): the one member MoEForward calls, with the reference's signature and its
// device-side behaviour (src/trace/router_collector.cpp:245-266: the selected ids of layer l,
// int32 [rows, top_k], are copied device-to-device on the stream into slot l of a capture
// buffer; a call that does not fit the announced shape stops the capture and is not an
// error).  An engine build includes its own header instead; the MoEForward shim compiles
// against either because only CaptureLayer is used.  Request bookkeeping, the pinned-host
// ring and the writer thread of the real collector are the engine's business.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>

#include "q4t/status.h"

namespace q4t::trace {

class RouterCollector {
 public:
  // device_ids: caller-owned device buffer of layers * rows * top_k int32.
  void Begin(int32_t* device_ids, uint32_t layers, uint32_t rows, uint32_t top_k) {
    device_ = device_ids;
    layers_ = layers;
    rows_ = rows;
    top_k_ = top_k;
    next_ = 0;
    failed_ = false;
  }
  Status CaptureLayer(uint32_t layer, const int32_t* ids, int rows, int top_k, cudaStream_t stream) {
    if (!device_ || failed_) return Status();
    if (layer != next_ || layer >= layers_ || rows != static_cast<int>(rows_) || top_k != static_cast<int>(top_k_)) {
      failed_ = true;  // an observation that breaks the contract stops the capture only
      return Status();
    }
    const size_t count = static_cast<size_t>(rows) * top_k;
    const cudaError_t e =
        cudaMemcpyAsync(device_ + layer * count, ids, count * sizeof(int32_t), cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) {
      failed_ = true;
      return Status::Fail("trace device copy: " + std::string(cudaGetErrorString(e)));
    }
    ++next_;
    return Status();
  }
  uint32_t captured_layers() const { return next_; }
  bool failed() const { return failed_; }

 private:
  int32_t* device_ = nullptr;
  uint32_t layers_ = 0, rows_ = 0, top_k_ = 0, next_ = 0;
  bool failed_ = false;
};

}  // namespace q4t::trace
