// Encoder self-check (part of libq4t_moe_b200_check.so, the test-only companion of the
// product library): sweeps float bit patterns through the kernels' hardware encoders and
// through the compare-chain restatement of the reference's format.h.
#include "../kernels.h"
#include "../q4t_device.cuh"
#include "check_kernels.h"

namespace q4t {

namespace {

__global__ void encoder_selftest_kernel(int which, uint64_t first, uint64_t count,
                                        unsigned long long* mismatches, uint32_t* first_bad) {
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  unsigned long long bad = 0;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
    const uint32_t bits = static_cast<uint32_t>(first + i);
    const float f = __uint_as_float(bits);
    if (f != f) continue;
    bool differ;
    if (which == 0) {
      const uint32_t hw = e2m1x2_encode_hw(f, -f);
      const uint32_t sw = e2m1_encode_sw(f) | (e2m1_encode_sw(-f) << 4);
      differ = hw != sw;
    } else if (which == 1) {
      if (f < 0.0f || bits == 0x80000000u) continue;
      differ = e4m3_encode_hw(f) != e4m3_encode_sw(f);
    } else {  // branch-free reciprocal against the IEEE routine on [1, 2^126)
      if (!(f >= 1.0f && f < Q4T_RCP_FAST_MAX)) continue;
      differ = __float_as_uint(rcp_rn_ge1(f)) != __float_as_uint(__frcp_rn(f));
    }
    if (differ) {
      ++bad;
      atomicMin(first_bad, bits);
    }
  }
  if (bad) atomicAdd(mismatches, bad);
}

}  // namespace

cudaError_t launch_encoder_selftest(int which, uint64_t first, uint64_t count,
                                    unsigned long long* d_mismatches, uint32_t* d_first_bad,
                                    cudaStream_t stream) {
  encoder_selftest_kernel<<<1184, 256, 0, stream>>>(which, first, count, d_mismatches, d_first_bad);
  return cudaGetLastError();
}

}  // namespace q4t
