// QuantizeActivationToFp4Async / DequantFp4ToBf16Async with the reference's
// signatures (include/q4t/quant/act_quant.h:30-34, include/q4t/quant/dequant.h:22-25).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "q4t_moe_b200.h"

namespace q4t::quant {
inline cudaError_t QuantizeActivationToFp4Async(const uint16_t* bf16, uint8_t* packed_out, uint8_t* sf_out, int M,
                                                int K, float global_scale, cudaStream_t stream) {
  return q4t_quantize_activation_fp4(bf16, packed_out, sf_out, M, K, global_scale, stream) == Q4T_OK
             ? cudaSuccess
             : cudaErrorInvalidValue;
}
inline cudaError_t DequantFp4ToBf16Async(const uint8_t* packed, const uint8_t* group_scale, uint16_t* bf16_out,
                                         float inv_global_scale, int N, int K, cudaStream_t stream) {
  return q4t_dequant_fp4_to_bf16(packed, group_scale, bf16_out, inv_global_scale, N, K, stream) == Q4T_OK
             ? cudaSuccess
             : cudaErrorInvalidValue;
}
}  // namespace q4t::quant
