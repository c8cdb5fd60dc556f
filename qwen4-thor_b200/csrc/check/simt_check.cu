// Verification GEMM on CUDA cores: exact integer evaluation of the NVFP4 dot
// product, out = float(exact * alpha).  It is the device-side twin of the CPU
// oracle's exact mode and exists so that tests can check the tensor-core
// kernels at sizes the CPU cannot reach.  Part of libq4t_moe_b200_check.so, the test-only
// companion of the product library; the product never links it.
#include "../kernels.h"
#include "../q4t_device.cuh"
#include "check_kernels.h"

namespace q4t {

namespace {

__device__ __forceinline__ int e2m1_twice(uint32_t c) {
  // twice the e2m1 value: 0,1,2,3,4,6,8,12 with sign
  const int m = (c & 6u) ? static_cast<int>(2u + (c & 1u)) << (((c >> 1) & 3u) - 1u)
                         : static_cast<int>(c & 1u);
  return (c & 8u) ? -m : m;
}
__device__ __forceinline__ void e4m3_parts(uint32_t c, int& mant, int& ex) {
  ex = static_cast<int>((c >> 3) & 15u);
  mant = static_cast<int>(c & 7u);
  if (ex == 0) ex = 1;
  else if (ex == 15 && mant == 7) mant = 0;
  else mant += 8;
}

// One warp per output element; lanes stride over the groups of 16.
__global__ void __launch_bounds__(256) fp4_gemm_check_kernel(
    const uint8_t* __restrict__ w_packed, const uint8_t* __restrict__ w_sf,
    const uint8_t* __restrict__ a_packed, const uint8_t* __restrict__ a_sf, float* __restrict__ out,
    int M, int N, int K, float alpha) {
  const int64_t o = static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5);
  if (o >= static_cast<int64_t>(M) * N) return;
  const int m = static_cast<int>(o / N), n = static_cast<int>(o % N);
  const int lane = threadIdx.x & 31, groups = K >> 4;
  const uint32_t ntk = (groups + 3) >> 2;
  long long acc = 0;
  for (int g = lane; g < groups; g += 32) {
    const uint2 av = *reinterpret_cast<const uint2*>(a_packed + (static_cast<size_t>(m) * groups + g) * 8);
    const uint2 wv = *reinterpret_cast<const uint2*>(w_packed + (static_cast<size_t>(n) * groups + g) * 8);
    const uint32_t aw[2] = {av.x, av.y}, ww[2] = {wv.x, wv.y};
    int s = 0;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      s += e2m1_twice((aw[j >> 3] >> (4 * (j & 7))) & 15u) * e2m1_twice((ww[j >> 3] >> (4 * (j & 7))) & 15u);
    int ma, ea, mw, ew;
    e4m3_parts(a_sf[sf_offset(m, g, ntk)], ma, ea);
    e4m3_parts(w_sf[sf_offset(n, g, ntk)], mw, ew);
    acc += static_cast<long long>(s) * (ma * mw) * (1ll << (ea + ew - 2));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (lane == 0)
    out[o] = static_cast<float>(ldexp(static_cast<double>(acc), -20) * static_cast<double>(alpha));
}

}  // namespace

cudaError_t launch_fp4_gemm_check(const uint8_t* w_packed, const uint8_t* w_sf, const uint8_t* a_packed,
                                  const uint8_t* a_sf, float* out, int M, int N, int K, float alpha,
                                  cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(M) * N;
  if (total == 0) return cudaSuccess;
  fp4_gemm_check_kernel<<<static_cast<unsigned>((total + 7) / 8), 256, 0, stream>>>(
      w_packed, w_sf, a_packed, a_sf, out, M, N, K, alpha);
  return cudaGetLastError();
}

}  // namespace q4t
