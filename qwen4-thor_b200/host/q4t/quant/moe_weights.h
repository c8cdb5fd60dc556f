// MoEWeightLayout and the expert loader with the reference's shape
// (include/q4t/quant/moe_weights.h:43-123, src/quant/moe_weights.cpp:43-321).
// The loader is generic over the tensor source: `read(name, dst, bytes)` copies
// the checkpoint tensor `name` into host memory and returns false on failure,
// which is what io::WeightLoader::ReadTensor does in the engine.
#pragma once
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstdlib>
#include <mutex>
#include <string>
#include <thread>
#include <type_traits>
#include <vector>

#include "q4t/io/weight_loader.h"
#include "q4t/quant/swizzle.h"
#include "q4t/status.h"
#include "q4t_moe_b200.h"

namespace q4t::quant {

struct MoEWeightLayout {
  int E = 0, hs = 0, moe_is = 0;
  bool slot_mode = false;
  uint8_t* gu_packed = nullptr;
  uint8_t* gu_sf = nullptr;
  uint8_t* dn_packed = nullptr;
  uint8_t* dn_sf = nullptr;
  float* gu_w_scale2 = nullptr;
  float* gu_input_scale = nullptr;
  float* dn_w_scale2 = nullptr;
  float* dn_input_scale = nullptr;
  std::vector<float> gu_w_scale2_h, gu_input_scale_h, dn_w_scale2_h, dn_input_scale_h;

  size_t gu_sf_block() const { return SfBufferSize(2 * moe_is, hs); }
  size_t dn_sf_block() const { return SfBufferSize(hs, moe_is); }
  uint8_t* gu_packed_expert(int e) const { return gu_packed + static_cast<size_t>(e) * moe_is * hs; }
  uint8_t* gu_sf_expert(int e) const { return gu_sf + static_cast<size_t>(e) * gu_sf_block(); }
  uint8_t* dn_packed_expert(int e) const { return dn_packed + static_cast<size_t>(e) * hs * (moe_is / 2); }
  uint8_t* dn_sf_expert(int e) const { return dn_sf + static_cast<size_t>(e) * dn_sf_block(); }
  size_t TotalBytes() const {
    return static_cast<size_t>(2 * E * moe_is) * (hs / 2) + static_cast<size_t>(E) * gu_sf_block() +
           static_cast<size_t>(E * hs) * (moe_is / 2) + static_cast<size_t>(E) * dn_sf_block() +
           4 * static_cast<size_t>(E) * sizeof(float);
  }
  // POD image handed to the C ABI.
  q4t_routed_weights Abi() const {
    float uniform = gu_input_scale_h.empty() ? 0.0f : gu_input_scale_h[0];
    for (float v : gu_input_scale_h)
      if (v != uniform) uniform = 0.0f;
    return q4t_routed_weights{E, hs, moe_is, slot_mode ? 1 : 0, gu_packed, gu_sf, dn_packed, dn_sf,
                              gu_w_scale2, gu_input_scale, dn_w_scale2, dn_input_scale,
                              uniform > 0.0f ? uniform : 0.0f, 0};
  }
};

inline std::string MoEExpertTensorName(int layer, int e, const char* proj, const char* suffix) {
  return "model.language_model.layers." + std::to_string(layer) + ".mlp.experts." + std::to_string(e) + "." + proj +
         "." + suffix;
}

// Loads one layer's experts through `read`; on success the caller owns the eight
// device buffers of `out` (cudaFree).  Gate and up share gate's two scalars.
template <class ReadTensor,
          std::enable_if_t<std::is_invocable_r_v<bool, ReadTensor&, const std::string&, void*, size_t>, int> = 0>
Status LoadMoEWeights(ReadTensor&& read, int layer_id, int E, int hs, int moe_is, MoEWeightLayout* out,
                      cudaStream_t stream) {
  if (E <= 0 || hs <= 0 || moe_is <= 0) return Status::Fail("invalid MoE dims");
  if ((hs % 32) != 0 || (moe_is % 32) != 0) return Status::Fail("hs and moe_is must be multiples of 32 (FP4 GEMM)");
  if ((2 * moe_is) % 128 != 0 || (hs % 128) != 0)
    return Status::Fail("2*moe_is and hs must be multiples of 128 (per-expert SF blocks)");
  out->E = E;
  out->hs = hs;
  out->moe_is = moe_is;
  const size_t gu_blk = out->gu_sf_block(), dn_blk = out->dn_sf_block();
  const size_t gu_w = static_cast<size_t>(moe_is) * (hs / 2), dn_w = static_cast<size_t>(hs) * (moe_is / 2);
  const size_t gu_s = static_cast<size_t>(moe_is) * (hs / 16), dn_s = static_cast<size_t>(hs) * (moe_is / 16);
  auto alloc = [](void* p, size_t bytes) { return cudaMalloc(reinterpret_cast<void**>(p), bytes) == cudaSuccess; };
  if (!alloc(&out->gu_packed, 2 * gu_w * E) || !alloc(&out->gu_sf, gu_blk * E) || !alloc(&out->dn_packed, dn_w * E) ||
      !alloc(&out->dn_sf, dn_blk * E) || !alloc(&out->gu_w_scale2, sizeof(float) * E) ||
      !alloc(&out->gu_input_scale, sizeof(float) * E) || !alloc(&out->dn_w_scale2, sizeof(float) * E) ||
      !alloc(&out->dn_input_scale, sizeof(float) * E))
    return Status::Fail("cudaMalloc failed");
  out->gu_w_scale2_h.resize(E);
  out->gu_input_scale_h.resize(E);
  out->dn_w_scale2_h.resize(E);
  out->dn_input_scale_h.resize(E);
  // Experts are independent (disjoint device ranges, read-only checkpoint), so a pool of
  // min(hardware threads, E) workers reads, packs and uploads them, each with its own
  // staging buffers; Q4T_MOE_THREADS overrides the count (src/quant/moe_weights.cpp:111-125
  // of the reference).  `read` is called from several threads at once.  Each worker copies
  // with the blocking cudaMemcpy, so its staging is free for its next expert on return;
  // `stream` orders only the final scalar upload.
  int nthreads = static_cast<int>(std::thread::hardware_concurrency());
  if (nthreads < 1) nthreads = 1;
  if (nthreads > E) nthreads = E;
  if (const char* env = std::getenv("Q4T_MOE_THREADS")) {
    const int v = std::atoi(env);
    if (v > 0) nthreads = v < E ? v : E;
  }
  int device = 0;
  cudaGetDevice(&device);
  std::atomic<int> next_expert{0};
  std::atomic<bool> failed{false};
  std::mutex err_mu;
  std::string err;
  auto fail = [&](const std::string& msg) {
    std::lock_guard<std::mutex> lock(err_mu);
    if (!failed.exchange(true)) err = msg;
  };
  auto worker = [&]() {
    if (cudaSetDevice(device) != cudaSuccess) return fail("cudaSetDevice failed in a loader thread");
    std::vector<uint8_t> gate_w(gu_w), up_w(gu_w), down_w(dn_w), gate_s(gu_s), up_s(gu_s), down_s(dn_s);
    std::vector<uint8_t> gu_p(2 * gu_w), gu_sf(gu_blk), dn_p(dn_w), dn_sf(dn_blk);
    for (int e = next_expert.fetch_add(1); e < E && !failed.load(); e = next_expert.fetch_add(1)) {
      auto name = [&](const char* proj, const char* suffix) { return MoEExpertTensorName(layer_id, e, proj, suffix); };
      float sc[4];
      if (!read(name("gate_proj", "weight"), gate_w.data(), gate_w.size()) ||
          !read(name("up_proj", "weight"), up_w.data(), up_w.size()) ||
          !read(name("down_proj", "weight"), down_w.data(), down_w.size()) ||
          !read(name("gate_proj", "weight_scale"), gate_s.data(), gate_s.size()) ||
          !read(name("up_proj", "weight_scale"), up_s.data(), up_s.size()) ||
          !read(name("down_proj", "weight_scale"), down_s.data(), down_s.size()) ||
          !read(name("gate_proj", "weight_scale_2"), &sc[0], sizeof(float)) ||
          !read(name("gate_proj", "input_scale"), &sc[1], sizeof(float)) ||
          !read(name("down_proj", "weight_scale_2"), &sc[2], sizeof(float)) ||
          !read(name("down_proj", "input_scale"), &sc[3], sizeof(float)))
        return fail("MoE expert load failed (layer " + std::to_string(layer_id) + ")");
      if (q4t_pack_expert_host(gate_w.data(), up_w.data(), down_w.data(), gate_s.data(), up_s.data(), down_s.data(), hs,
                               moe_is, gu_p.data(), gu_sf.data(), dn_p.data(), dn_sf.data()) != Q4T_OK)
        return fail(q4t_last_error());
      out->gu_w_scale2_h[e] = sc[0];
      out->gu_input_scale_h[e] = sc[1];
      out->dn_w_scale2_h[e] = sc[2];
      out->dn_input_scale_h[e] = sc[3];
      if (cudaMemcpy(out->gu_packed_expert(e), gu_p.data(), gu_p.size(), cudaMemcpyHostToDevice) != cudaSuccess ||
          cudaMemcpy(out->gu_sf_expert(e), gu_sf.data(), gu_blk, cudaMemcpyHostToDevice) != cudaSuccess ||
          cudaMemcpy(out->dn_packed_expert(e), dn_p.data(), dn_p.size(), cudaMemcpyHostToDevice) != cudaSuccess ||
          cudaMemcpy(out->dn_sf_expert(e), dn_sf.data(), dn_blk, cudaMemcpyHostToDevice) != cudaSuccess)
        return fail("expert upload failed");
    }
  };
  if (nthreads == 1) {
    worker();
  } else {
    std::vector<std::thread> pool;
    pool.reserve(static_cast<size_t>(nthreads));
    for (int i = 0; i < nthreads; ++i) pool.emplace_back(worker);
    for (std::thread& th : pool) th.join();
  }
  if (failed.load()) return Status::Fail(err);
  const size_t sb = sizeof(float) * E;
  if (cudaMemcpyAsync(out->gu_w_scale2, out->gu_w_scale2_h.data(), sb, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaMemcpyAsync(out->gu_input_scale, out->gu_input_scale_h.data(), sb, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaMemcpyAsync(out->dn_w_scale2, out->dn_w_scale2_h.data(), sb, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaMemcpyAsync(out->dn_input_scale, out->dn_input_scale_h.data(), sb, cudaMemcpyHostToDevice, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return Status::Fail("scale upload failed");
  return Status();
}

// The consumer's NVFP4 layout, checked on the checkpoint's metadata before anything is
// allocated or read (reference include/q4t/quant/moe_tensor_contract.h:11-48): per expert
// and projection a U8 weight [rows, cols/2], an F8_E4M3 weight_scale [rows, cols/16] and
// two FP32 scalars (rank 0 or a one-element vector).
inline Status ValidateMoEExpert(const io::WeightLoader& loader, int layer, int expert, int hs, int moe_is) {
  for (const char* proj : {"down_proj", "gate_proj", "up_proj"}) {
    const bool down = proj[0] == 'd';
    const int64_t rows = down ? hs : moe_is, cols = down ? moe_is : hs;
    for (const char* suffix : {"weight", "weight_scale", "weight_scale_2", "input_scale"}) {
      const std::string name = MoEExpertTensorName(layer, expert, proj, suffix);
      const io::TensorInfo* t = loader.FindTensor(name);
      if (!t) return Status::Fail("missing MoE tensor: " + name);
      const std::string kind(suffix);
      if (kind == "weight" || kind == "weight_scale") {
        const int64_t width = cols / (kind == "weight" ? 2 : 16);
        const io::Dtype want = kind == "weight" ? io::Dtype::kU8 : io::Dtype::kF8E4M3;
        if (t->dtype != want || t->shape.size() != 2 || t->shape[0] != rows || t->shape[1] != width ||
            t->byte_size() != static_cast<uint64_t>(rows * width))
          return Status::Fail("MoE tensor dtype/shape/size mismatch: " + name);
      } else {
        const bool scalar = t->shape.empty() || (t->shape.size() == 1 && t->shape[0] == 1);
        if (t->dtype != io::Dtype::kF32 || !scalar || t->byte_size() != sizeof(float))
          return Status::Fail("MoE scalar dtype/shape/size mismatch: " + name);
      }
    }
  }
  return Status();
}

// The engine's own signature (reference include/q4t/quant/moe_weights.h:121-123): every
// expert's metadata is validated first, then the tensors are read through the loader.
inline Status LoadMoEWeights(const io::WeightLoader& loader, int layer_id, int E, int hs, int moe_is,
                             MoEWeightLayout* out, cudaStream_t stream) {
  if (E <= 0 || hs <= 0 || moe_is <= 0) return Status::Fail("invalid MoE dims");
  for (int e = 0; e < E; ++e) {
    Status s = ValidateMoEExpert(loader, layer_id, e, hs, moe_is);
    if (!s.ok()) return s;
  }
  return LoadMoEWeights(
      [&](const std::string& name, void* dst, size_t bytes) { return loader.ReadTensor(name, dst, bytes).ok(); },
      layer_id, E, hs, moe_is, out, stream);
}

}  // namespace q4t::quant
