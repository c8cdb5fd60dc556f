// Launch interface of the test-only check library (libq4t_moe_b200_check.so).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace q4t {

cudaError_t launch_encoder_selftest(int which, uint64_t first, uint64_t count, unsigned long long* d_mismatches,
                                    uint32_t* d_first_bad, cudaStream_t stream);
// Exact integer evaluation of the NVFP4 dot product on CUDA cores, out = float(exact * alpha).
// Swizzled scales on both sides.
cudaError_t launch_fp4_gemm_check(const uint8_t* w_packed, const uint8_t* w_sf, const uint8_t* a_packed,
                                  const uint8_t* a_sf, float* out, int M, int N, int K, float alpha,
                                  cudaStream_t stream);

}  // namespace q4t
