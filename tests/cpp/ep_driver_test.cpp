// The C++ expert-parallel drivers (host/q4t/parallel/ep_driver.h) on real ranks: one process
// per GPU, NCCL between them.  Every rank builds the same seeded layer, runs the whole batch
// through the single-GPU MoEForward as the expected result, then runs its share of the
// tokens through PeerExpertParallel and RowExchangeExpertParallel and compares bit for bit.
//
//   ep_driver_test <rank> <world> <id-file>      (rank 0 writes the NCCL id to <id-file>)
//
// Prints "ep_driver_test PASS rank <r>" on success.
#include <cuda_runtime.h>
#include <nccl.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <random>
#include <vector>

#include "q4t/parallel/ep_driver.h"

using namespace q4t;

#define CHECK(c)                                                                          \
  do {                                                                                    \
    if (!(c)) {                                                                           \
      std::printf("ep_driver_test FAIL rank %d %s:%d %s\n", g_rank, __FILE__, __LINE__, #c); \
      return 1;                                                                           \
    }                                                                                     \
  } while (0)
#define CHECK_OK(s)                                                                                \
  do {                                                                                             \
    Status st__ = (s);                                                                             \
    if (!st__.ok()) {                                                                              \
      std::printf("ep_driver_test FAIL rank %d %s:%d %s\n", g_rank, __FILE__, __LINE__, st__.message().c_str()); \
      return 1;                                                                                    \
    }                                                                                              \
  } while (0)

static int g_rank = 0;

static uint16_t bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

// Random bf16 tensor on the device (same values on every rank: the generator is seeded).
static uint16_t* device_normal(std::mt19937& rng, size_t n, float sd) {
  std::normal_distribution<float> nd(0.f, sd);
  std::vector<uint16_t> h(n);
  for (auto& v : h) v = bf16(nd(rng));
  uint16_t* d = nullptr;
  cudaMalloc(reinterpret_cast<void**>(&d), n * 2);
  cudaMemcpy(d, h.data(), n * 2, cudaMemcpyHostToDevice);
  return d;
}

struct Layer {
  q4t_routed_weights routed{};
  q4t_extra_weights extra{};
};

// E experts quantised on the device with the library's own quantiser (amax / (6 * 448) per
// projection, gate and up sharing one scale), as the synthetic layers of the benchmark are.
static int build_layer(std::mt19937& rng, int E, int hs, int is, int sis, Layer* L) {
  const size_t gu_rows = size_t(2) * is, gu_blk = q4t_sf_buffer_size(2 * is, hs), dn_blk = q4t_sf_buffer_size(hs, is);
  uint8_t *gu_p, *gu_s, *dn_p, *dn_s;
  cudaMalloc(reinterpret_cast<void**>(&gu_p), size_t(E) * gu_rows * (hs / 2));
  cudaMalloc(reinterpret_cast<void**>(&gu_s), size_t(E) * gu_blk);
  cudaMalloc(reinterpret_cast<void**>(&dn_p), size_t(E) * hs * (is / 2));
  cudaMalloc(reinterpret_cast<void**>(&dn_s), size_t(E) * dn_blk);
  cudaMemset(gu_s, 0, size_t(E) * gu_blk);
  cudaMemset(dn_s, 0, size_t(E) * dn_blk);
  std::vector<float> ws2(E, 0.02f * 4.5f / (6 * 448)), in_gu(E, 5.0f / (6 * 448)), in_dn(E, 2.0f / (6 * 448));
  for (int e = 0; e < E; ++e) {
    uint16_t* w = device_normal(rng, gu_rows * hs, 0.02f);
    if (q4t_quantize_activation_fp4(w, gu_p + size_t(e) * gu_rows * (hs / 2), gu_s + size_t(e) * gu_blk, int(gu_rows), hs,
                                    ws2[e], nullptr) != Q4T_OK)
      return 1;
    cudaDeviceSynchronize();
    cudaFree(w);
    w = device_normal(rng, size_t(hs) * is, 0.02f);
    if (q4t_quantize_activation_fp4(w, dn_p + size_t(e) * hs * (is / 2), dn_s + size_t(e) * dn_blk, hs, is, ws2[e],
                                    nullptr) != Q4T_OK)
      return 1;
    cudaDeviceSynchronize();
    cudaFree(w);
  }
  float* scal;
  cudaMalloc(reinterpret_cast<void**>(&scal), size_t(4) * E * 4);
  cudaMemcpy(scal, ws2.data(), E * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(scal + E, in_gu.data(), E * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(scal + 2 * E, ws2.data(), E * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(scal + 3 * E, in_dn.data(), E * 4, cudaMemcpyHostToDevice);
  L->routed = q4t_routed_weights{E, hs, is, 0, gu_p, gu_s, dn_p, dn_s, scal, scal + E, scal + 2 * E, scal + 3 * E, in_gu[0], 0};
  L->extra = q4t_extra_weights{E, hs, sis, device_normal(rng, size_t(E) * hs, 0.02f),
                               device_normal(rng, size_t(2) * sis * hs, 0.02f), device_normal(rng, size_t(hs) * sis, 0.02f),
                               device_normal(rng, hs, 0.02f)};
  return 0;
}

// This rank's contiguous block of experts: a view into the full layer.
static q4t_routed_weights block_of(const q4t_routed_weights& f, int lo, int n) {
  q4t_routed_weights w = f;
  w.E = n;
  w.gu_packed = f.gu_packed + size_t(lo) * 2 * f.moe_is * (f.hs / 2);
  w.gu_sf = f.gu_sf + size_t(lo) * q4t_sf_buffer_size(2 * f.moe_is, f.hs);
  w.dn_packed = f.dn_packed + size_t(lo) * f.hs * (f.moe_is / 2);
  w.dn_sf = f.dn_sf + size_t(lo) * q4t_sf_buffer_size(f.hs, f.moe_is);
  w.gu_w_scale2 = f.gu_w_scale2 + lo;
  w.gu_input_scale = f.gu_input_scale + lo;
  w.dn_w_scale2 = f.dn_w_scale2 + lo;
  w.dn_input_scale = f.dn_input_scale + lo;
  return w;
}

int main(int argc, char** argv) {
  if (argc < 4) {
    std::printf("usage: ep_driver_test <rank> <world> <id-file>\n");
    return 2;
  }
  const int rank = g_rank = std::atoi(argv[1]), world = std::atoi(argv[2]);
  const char* id_file = argv[3];
  int ndev = 0;
  CHECK(cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0);
  CHECK(cudaSetDevice(rank % ndev) == cudaSuccess);
  // rendezvous through a file: rank 0 publishes the NCCL id, the others wait for it
  ncclUniqueId id;
  if (rank == 0) {
    CHECK(ncclGetUniqueId(&id) == ncclSuccess);
    std::string tmp = std::string(id_file) + ".tmp";
    std::ofstream(tmp, std::ios::binary).write(reinterpret_cast<const char*>(&id), sizeof(id));
    CHECK(std::rename(tmp.c_str(), id_file) == 0);
  } else {
    bool got = false;
    for (int i = 0; i < 600 && !got; ++i) {   // at most a minute
      std::ifstream f(id_file, std::ios::binary);
      if (f && f.read(reinterpret_cast<char*>(&id), sizeof(id))) got = true;
      else usleep(100000);
    }
    CHECK(got);
  }
  ncclComm_t comm;
  CHECK(ncclCommInitRank(&comm, world, id, rank) == ncclSuccess);
  cudaStream_t stream;
  CHECK(cudaStreamCreate(&stream) == cudaSuccess);

  const int E = 16, hs = 512, is = 128, sis = 128, k = 3, T_all = 96 * world, T = T_all / world;
  std::mt19937 rng(1234);
  Layer L;
  CHECK(build_layer(rng, E, hs, is, sis, &L) == 0);
  uint16_t* x_all = device_normal(rng, size_t(T_all) * hs, 1.0f);

  // expected: the single-GPU layer over the whole batch
  uint16_t* y_ref;
  CHECK(cudaMalloc(reinterpret_cast<void**>(&y_ref), size_t(T_all) * hs * 2) == cudaSuccess);
  const size_t fws = q4t_moe_forward_workspace_bytes(T_all, k, hs, is, sis, E);
  void* ws;
  CHECK(cudaMalloc(&ws, fws) == cudaSuccess);
  CHECK(q4t_moe_forward(x_all, &L.routed, &L.extra, y_ref, T_all, k, ws, fws, nullptr, 0, stream) == Q4T_OK);
  CHECK(cudaStreamSynchronize(stream) == cudaSuccess);
  std::vector<uint16_t> want(size_t(T) * hs), got(want.size());
  cudaMemcpy(want.data(), y_ref + size_t(rank) * T * hs, want.size() * 2, cudaMemcpyDeviceToHost);

  parallel::EpShape shape;
  shape.world = world; shape.rank = rank; shape.tokens_per_rank = T; shape.k = k; shape.experts = E;
  shape.hs = hs; shape.moe_is = is; shape.shared_is = sis;
  const q4t_routed_weights mine = block_of(L.routed, rank * (E / world), E / world);
  const uint16_t* x = x_all + size_t(rank) * T * hs;
  uint16_t* y;
  CHECK(cudaMalloc(reinterpret_cast<void**>(&y), size_t(T) * hs * 2) == cudaSuccess);

  for (int collectives = 0; collectives < 2; ++collectives) {
    // peer memory; ids and orderings by flag kernels over peer memory (0) or by ncclAllGather /
    // ncclAllReduce (1); several steps over the same buffers
    parallel::PeerExpertParallel drv;
    CHECK_OK(drv.Init(comm, stream, shape, mine, L.extra, /*expert_map=*/0, nullptr, nullptr, collectives != 0));
    for (int step = 0; step < 4; ++step) {
      cudaMemsetAsync(y, 0, size_t(T) * hs * 2, stream);
      CHECK_OK(drv.Step(x, y, stream));
      CHECK(cudaStreamSynchronize(stream) == cudaSuccess);
      CHECK_OK(drv.CheckStatus());
      cudaMemcpy(got.data(), y, got.size() * 2, cudaMemcpyDeviceToHost);
      CHECK(std::memcmp(got.data(), want.data(), got.size() * 2) == 0);
    }
  }
  {  // bf16 rows both ways over grouped ncclSend / ncclRecv
    parallel::RowExchangeExpertParallel drv;
    CHECK_OK(drv.Init(comm, shape, mine, L.extra, T_all * k));
    cudaMemsetAsync(y, 0, size_t(T) * hs * 2, stream);
    CHECK_OK(drv.Step(x, y, stream));
    CHECK(cudaStreamSynchronize(stream) == cudaSuccess);
    cudaMemcpy(got.data(), y, got.size() * 2, cudaMemcpyDeviceToHost);
    CHECK(std::memcmp(got.data(), want.data(), got.size() * 2) == 0);
  }
  ncclCommDestroy(comm);
  std::printf("ep_driver_test PASS rank %d of %d\n", rank, world);
  return 0;
}
