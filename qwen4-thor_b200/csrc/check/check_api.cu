// C ABI of libq4t_moe_b200_check.so (include/q4t_moe_b200_check.h): device-side checkers the
// GPU tests use.  Built beside the product library, never linked into it.
#include "../../../include/q4t_moe_b200_check.h"

#include <cuda_runtime.h>

#include <string>

#include "check_kernels.h"

namespace {
thread_local std::string g_error;
int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}
int fail_cuda(const char* what, cudaError_t e) {
  g_error = std::string(what) + ": " + cudaGetErrorString(e);
  return Q4T_ERR_CUDA;
}
}  // namespace

extern "C" {

const char* q4t_check_last_error(void) { return g_error.c_str(); }

int32_t q4t_fp4_gemm_check(const uint8_t* w_packed, const uint8_t* w_sf, const uint8_t* a_packed,
                           const uint8_t* a_sf, float* out, int32_t M, int32_t N, int32_t K,
                           float inv_w_global, float inv_a_global, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K % 16) return fail(Q4T_ERR_INVALID, "invalid GEMM dims");
  cudaError_t e = q4t::launch_fp4_gemm_check(w_packed, w_sf, a_packed, a_sf, out, M, N, K,
                                             inv_w_global * inv_a_global, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("check GEMM launch", e);
}

int32_t q4t_selftest_encoders(int32_t which, uint64_t first, uint64_t count, uint64_t* mismatches,
                              uint32_t* first_bad, void* stream) {
  if (!mismatches || !first_bad) return fail(Q4T_ERR_INVALID, "null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned long long* d_m = nullptr;
  uint32_t* d_b = nullptr;
  cudaError_t e;
  if ((e = cudaMalloc(&d_m, 8)) != cudaSuccess) return fail_cuda("cudaMalloc", e);
  if ((e = cudaMalloc(&d_b, 4)) != cudaSuccess) {
    cudaFree(d_m);
    return fail_cuda("cudaMalloc", e);
  }
  cudaMemsetAsync(d_m, 0, 8, st);
  cudaMemsetAsync(d_b, 0xff, 4, st);
  e = q4t::launch_encoder_selftest(which, first, count, d_m, d_b, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  unsigned long long m = 0;
  if (e == cudaSuccess) e = cudaMemcpy(&m, d_m, 8, cudaMemcpyDeviceToHost);
  if (e == cudaSuccess) e = cudaMemcpy(first_bad, d_b, 4, cudaMemcpyDeviceToHost);
  cudaFree(d_m);
  cudaFree(d_b);
  if (e != cudaSuccess) return fail_cuda("encoder self-check", e);
  *mismatches = m;
  return Q4T_OK;
}

}  // extern "C"
