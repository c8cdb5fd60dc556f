// Checkpoint loading through the reference-shaped io / quant / model shims.
//   loader_test host  <dir> <layer> <E> <hs> <is> <out.bin>
//       CPU only: validates the expert contract, reads every expert through io::WeightLoader,
//       packs it with q4t_pack_expert_host and dumps gu_packed | gu_sf | dn_packed | dn_sf |
//       4 x float[E].
//   loader_test device <dir> <layer> <E> <hs> <is> <sis> <T> <k> <x.bin> <y.bin>
//       GPU: LoadMoEWeights + LoadMoEExtra + MoEForward on the bf16 rows of x.bin, dumps y.
//   loader_test check <dir> <layer> <E> <hs> <is>
//       prints the contract check's message ("ok" when it passes).
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "q4t/io/weight_loader.h"
#include "q4t/model/moe.h"
#include "q4t/quant/moe_weights.h"

using namespace q4t;

static bool write_all(const char* path, const std::vector<std::vector<uint8_t>>& parts) {
  std::FILE* f = std::fopen(path, "wb");
  if (!f) return false;
  for (const auto& p : parts)
    if (!p.empty() && std::fwrite(p.data(), 1, p.size(), f) != p.size()) return false;
  return std::fclose(f) == 0;
}

int main(int argc, char** argv) {
  if (argc < 7) {
    std::printf("usage: see the header comment\n");
    return 2;
  }
  const std::string mode = argv[1], dir = argv[2];
  const int layer = std::atoi(argv[3]), E = std::atoi(argv[4]), hs = std::atoi(argv[5]), is = std::atoi(argv[6]);
  io::WeightIndex* index_raw = nullptr;
  Status s = io::WeightIndex::Open(dir + "/model.safetensors.index.json", &index_raw);
  if (!s.ok()) {
    std::printf("index: %s\n", s.message().c_str());
    return 1;
  }
  std::unique_ptr<io::WeightIndex> index(index_raw);
  io::WeightLoader* loader_raw = nullptr;
  s = io::WeightLoader::Create(dir, *index, 2, &loader_raw);
  std::unique_ptr<io::WeightLoader> loader(loader_raw);
  if (!s.ok()) return 1;

  if (mode == "check") {
    for (int e = 0; e < E; ++e) {
      s = quant::ValidateMoEExpert(*loader, layer, e, hs, is);
      if (!s.ok()) {
        std::printf("%s\n", s.message().c_str());
        return 0;
      }
    }
    std::printf("ok shards=%zu tensors=%zu open=%zu\n", index->num_shards(), index->num_tensors(), loader->open_shards());
    return 0;
  }
  if (mode == "host") {
    if (argc < 8) return 2;
    const size_t gu_w = size_t(is) * (hs / 2), dn_w = size_t(hs) * (is / 2);
    const size_t gu_s = size_t(is) * (hs / 16), dn_s = size_t(hs) * (is / 16);
    const size_t gu_blk = q4t_sf_buffer_size(2 * is, hs), dn_blk = q4t_sf_buffer_size(hs, is);
    std::vector<uint8_t> gu_all(2 * gu_w * E), gu_sf_all(gu_blk * E), dn_all(dn_w * E), dn_sf_all(dn_blk * E);
    std::vector<uint8_t> scal(sizeof(float) * 4 * E);
    std::vector<uint8_t> gw(gu_w), uw(gu_w), dw(dn_w), gs(gu_s), us(gu_s), ds(dn_s);
    for (int e = 0; e < E; ++e) {
      s = quant::ValidateMoEExpert(*loader, layer, e, hs, is);
      if (!s.ok()) {
        std::printf("%s\n", s.message().c_str());
        return 1;
      }
      auto name = [&](const char* proj, const char* suffix) { return quant::MoEExpertTensorName(layer, e, proj, suffix); };
      float sc[4];
      bool ok = loader->ReadTensor(name("gate_proj", "weight"), gw.data(), gw.size()).ok() &&
                loader->ReadTensor(name("up_proj", "weight"), uw.data(), uw.size()).ok() &&
                loader->ReadTensor(name("down_proj", "weight"), dw.data(), dw.size()).ok() &&
                loader->ReadTensor(name("gate_proj", "weight_scale"), gs.data(), gs.size()).ok() &&
                loader->ReadTensor(name("up_proj", "weight_scale"), us.data(), us.size()).ok() &&
                loader->ReadTensor(name("down_proj", "weight_scale"), ds.data(), ds.size()).ok() &&
                loader->ReadTensor(name("gate_proj", "weight_scale_2"), &sc[0], 4).ok() &&
                loader->ReadTensor(name("gate_proj", "input_scale"), &sc[1], 4).ok() &&
                loader->ReadTensor(name("down_proj", "weight_scale_2"), &sc[2], 4).ok() &&
                loader->ReadTensor(name("down_proj", "input_scale"), &sc[3], 4).ok();
      if (!ok) {
        std::printf("read failed for expert %d\n", e);
        return 1;
      }
      if (q4t_pack_expert_host(gw.data(), uw.data(), dw.data(), gs.data(), us.data(), ds.data(), hs, is,
                               gu_all.data() + 2 * gu_w * e, gu_sf_all.data() + gu_blk * e, dn_all.data() + dn_w * e,
                               dn_sf_all.data() + dn_blk * e) != Q4T_OK) {
        std::printf("pack: %s\n", q4t_last_error());
        return 1;
      }
      for (int j = 0; j < 4; ++j) std::memcpy(scal.data() + (size_t(j) * E + e) * 4, &sc[j], 4);
    }
    if (!write_all(argv[7], {gu_all, gu_sf_all, dn_all, dn_sf_all, scal})) return 1;
    std::printf("host PASS\n");
    return 0;
  }
  if (mode == "device") {
    if (argc < 12) return 2;
    const int sis = std::atoi(argv[7]), T = std::atoi(argv[8]), k = std::atoi(argv[9]);
    quant::MoEWeightLayout L;
    s = quant::LoadMoEWeights(*loader, layer, E, hs, is, &L, 0);
    if (!s.ok()) {
      std::printf("LoadMoEWeights: %s\n", s.message().c_str());
      return 1;
    }
    model::MoEExtraWeights X;
    s = model::LoadMoEExtra(*loader, "model.language_model.layers." + std::to_string(layer) + ".mlp", E, hs, sis, &X, 0);
    if (!s.ok()) {
      std::printf("LoadMoEExtra: %s\n", s.message().c_str());
      return 1;
    }
    std::vector<uint16_t> x(size_t(T) * hs), y(size_t(T) * hs);
    std::FILE* f = std::fopen(argv[10], "rb");
    if (!f || std::fread(x.data(), 2, x.size(), f) != x.size()) return 1;
    std::fclose(f);
    uint16_t *d_x, *d_y;
    void* ws;
    const size_t ws_bytes = model::MoEForwardWorkspaceBytes(T, k, hs, is, sis, E);
    if (cudaMalloc(reinterpret_cast<void**>(&d_x), x.size() * 2) != cudaSuccess ||
        cudaMalloc(reinterpret_cast<void**>(&d_y), y.size() * 2) != cudaSuccess || cudaMalloc(&ws, ws_bytes) != cudaSuccess)
      return 1;
    cudaMemcpy(d_x, x.data(), x.size() * 2, cudaMemcpyHostToDevice);
    s = model::MoEForward(d_x, L, X, d_y, T, k, ws, ws_bytes, nullptr, 0, 0);
    if (!s.ok()) {
      std::printf("MoEForward: %s\n", s.message().c_str());
      return 1;
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return 1;
    cudaMemcpy(y.data(), d_y, y.size() * 2, cudaMemcpyDeviceToHost);
    std::vector<uint8_t> yb(y.size() * 2);
    std::memcpy(yb.data(), y.data(), yb.size());
    if (!write_all(argv[11], {yb})) return 1;
    std::printf("device PASS uniform_scale=%g\n", double(L.Abi().gu_input_scale_uniform));
    return 0;
  }
  return 2;
}
