/* C ABI of libq4t_moe_b200_check.so: device-side checkers for the GPU tests of
 * libq4t_moe_b200.so.  A separate shared object, so that nothing test-only is
 * exported by (or linked into) the library a runtime binds.  No counterpart in
 * the reference.  Status codes are those of q4t_moe_b200.h.                   */
#ifndef Q4T_MOE_B200_CHECK_H_
#define Q4T_MOE_B200_CHECK_H_

#include "q4t_moe_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Message of the calling thread's last failing call into this library.        */
const char* q4t_check_last_error(void);

/* Sweep float bit patterns [first, first+count) through the kernels' hardware
 * encoders and through a compare-chain restatement of format.h and return the
 * number of disagreements in *mismatches (host pointer).  which: 0 = e2m1,
 * 1 = ue4m3 (non-negative inputs only), 2 = the epilogue's branch-free
 * reciprocal against IEEE 1/x on [1, 2^126).  Synchronises the stream.        */
int32_t q4t_selftest_encoders(int32_t which, uint64_t first, uint64_t count,
                              uint64_t* mismatches, uint32_t* first_bad,
                              void* stream);
/* Exact-arithmetic NVFP4 GEMM on CUDA cores (fp32 out = float(exact * alpha),
 * alpha = inv_w_global * inv_a_global); the device twin of the CPU oracle's
 * exact mode, for checking the tensor-core path at sizes the CPU cannot
 * reach.  Same operand layout as q4t_fp4_gemm, any N, K % 16 == 0.            */
int32_t q4t_fp4_gemm_check(const uint8_t* w_packed, const uint8_t* w_sf,
                           const uint8_t* a_packed, const uint8_t* a_sf,
                           float* out, int32_t M, int32_t N, int32_t K,
                           float inv_w_global, float inv_a_global, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* Q4T_MOE_B200_CHECK_H_ */
