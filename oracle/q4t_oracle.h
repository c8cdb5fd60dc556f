/*
 * CPU oracle for the NVFP4 W4A4 MoE layer.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the arithmetic the reference engine
 * (thomas-hiddenpeak/qwen4-thor) performs on its routed-expert MoE path.  It
 * exists so that the CUDA library can be checked against an independent
 * implementation; nothing in the shipped library calls it.  Only the test
 * suite, the smoke check and the benchmark's CPU-baseline leg may load it.
 *
 * Parity status: the format / layout primitives are pinned bit-for-bit
 * against the reference's own headers (oracle/_ref, built from the reference
 * tree) and against the known-answer vectors in the reference's unit tests.
 * The NVFP4 GEMM results of the reference come from a closed library
 * (cuBLASLt); for those the oracle offers an exact-arithmetic mode that the
 * reference's own audits found equal to the library output after BF16
 * rounding.  That equality is not pinned here at bit level.
 *
 * Every function cites the reference file:line it follows.
 */
#ifndef Q4T_ORACLE_H_
#define Q4T_ORACLE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- scalar format primitives (include/q4t/quant/format.h:41-164) ---- */
float q4o_e2m1_to_float(uint8_t code);
int q4o_float_to_e2m1(float v);
float q4o_e4m3_to_float(uint8_t code);
uint8_t q4o_float_to_e4m3(float v);
void q4o_float_to_e4m3_bulk(const float* in, size_t n, uint8_t* out);
void q4o_float_to_e2m1_bulk(const float* in, size_t n, uint8_t* out);

/* ---- bf16 helpers (round to nearest even, as __float2bfloat16_rn) ---- */
uint16_t q4o_float_to_bf16(float f);
float q4o_bf16_to_float(uint16_t b);

/* ---- scale-factor swizzle (include/q4t/quant/swizzle.h:34-83) ---- */
size_t q4o_sf_offset(int row, int group, int num_g_tiles);
int q4o_sf_num_gtiles(int K);
size_t q4o_sf_buffer_size(int rows, int K);
void q4o_swizzle_sf(const uint8_t* row_major, int rows, int K, uint8_t* out);

/* ---- quantiser (tests/quant_fp4_test.cpp:69-97, src/quant/act_quant.cu:47-92) ----
 * v: float [rows,K]; packed: [rows,K/2]; sf_rm: row-major [rows,K/16]. */
void q4o_quantize_f32(const float* v, int rows, int K, float global_scale,
                      uint8_t* packed, uint8_t* sf_rm);
/* bf16 input, swizzled SF output of q4o_sf_buffer_size(rows,K) bytes (zero filled
 * first), i.e. what QuantizeActivationToFp4Async leaves in its two buffers. */
void q4o_quantize_bf16(const uint16_t* x, int rows, int K, float global_scale,
                       uint8_t* packed, uint8_t* sf_swizzled);
/* src/quant/dequant.cu:31-57: bf16(e2m1 * (e4m3 * inv_global)), row-major SF. */
void q4o_dequant_to_bf16(const uint8_t* packed, const uint8_t* sf_rm, int N,
                         int K, float inv_global, uint16_t* out);
/* tests/quant_fp4_test.cpp:99-121: float dequant, row-major SF. */
void q4o_dequant_to_f32(const uint8_t* packed, const uint8_t* sf_rm, int rows,
                        int K, float global_scale, float* out);

/* ---- NVFP4 GEMM: out[M,N] = alpha * A[M,K] . W[N,K]^T, swizzled SF on both.
 * mode 0: dequantise both sides to fp32, sequential fp32 dot, times nothing
 *         (the global scales are folded into the dequantised values), fp32 out
 *         (tests/quant_fp4_test.cpp:438-452).
 * mode 1: exact integer dot, (double)exact * (double)alpha -> float
 *         (the value the reference's audits found cuBLASLt to return before
 *         the output conversion).  alpha = inv_w_global * inv_a_global in fp32
 *         (include/q4t/quant/fp4_gemm.h:205).                                  */
void q4o_fp4_gemm(const uint8_t* w_packed, const uint8_t* w_sf,
                  const uint8_t* a_packed, const uint8_t* a_sf, float* out,
                  int M, int N, int K, float inv_w_global, float inv_a_global,
                  int mode);

/* ---- BF16 linear y[M,N] = bf16(x[M,K] . w[N,K]^T) ----
 * mode 0: sequential fp32 dot (tests/model_moe_test.cpp:272-280).
 * mode 1: the warp-per-output order of src/model/gemv.cu:56-119 (lane l takes
 *         8-element chunks l, l+32, ...; even/odd accumulators with fused
 *         multiply-add; x+y; shuffle-down tree), which the reference uses
 *         for M <= 8 outside prefill mode.                                     */
void q4o_bf16_linear(const uint16_t* x, const uint16_t* w, uint16_t* y, int M,
                     int N, int K, int mode);

/* ---- router top-k (src/model/moe.cu:134-212) ----
 * logits bf16 [T,E]; ids [T,k]; weights [T,k].  Selection by (value desc,
 * id asc); softmax over the selected k in selection order.                    */
void q4o_router_topk(const uint16_t* logits, int T, int E, int k, int32_t* ids,
                     float* weights);

/* ---- token -> expert permutation, defined as the stable order (expert asc,
 * flat (token,slot) index asc); the reference (src/quant/moe_gemm.cu:133-149,
 * 251-261) fixes only the multiset of rows per expert.  Ids outside [0,E) are
 * dropped (moe_gemm.cu:140); row_of_flat of a dropped slot is -1.
 * counts[E], offsets[E+1], row_of_flat[R], flat_of_row[R].                    */
void q4o_permutation(const int32_t* ids, int T, int k, int E, int32_t* counts,
                     int32_t* offsets, int32_t* row_of_flat,
                     int32_t* flat_of_row);

/* One MoE layer's weights, host memory, in the reference's device layout
 * (include/q4t/quant/moe_weights.h:43-109, include/q4t/model/moe.h:39-56).   */
typedef struct {
  int E, hs, moe_is, shared_is;
  const uint8_t* gu_packed;      /* [E*2*moe_is, hs/2]                       */
  const uint8_t* gu_sf;          /* E blocks of sf_buffer_size(2*moe_is, hs) */
  const uint8_t* dn_packed;      /* [E*hs, moe_is/2]                         */
  const uint8_t* dn_sf;          /* E blocks of sf_buffer_size(hs, moe_is)   */
  const float* gu_w_scale2;      /* [E] */
  const float* gu_input_scale;   /* [E] */
  const float* dn_w_scale2;      /* [E] */
  const float* dn_input_scale;   /* [E] */
  const uint16_t* gate;          /* [E, hs] router (bf16); may be NULL       */
  const uint16_t* shared_gu;     /* [2*shared_is, hs]                        */
  const uint16_t* shared_down;   /* [hs, shared_is]                          */
  const uint16_t* shared_gate_scalar; /* [hs]                                */
} q4o_layer;

/* Optional taps on the routed path, all indexed by the stable grouped row
 * (see q4o_permutation).  Any pointer may be NULL.                            */
typedef struct {
  uint8_t* a_packed;   /* [R, hs/2]     input codes                          */
  uint8_t* a_sf;       /* [R, hs/16]    input scales, row-major              */
  uint16_t* gu_out;    /* [R, 2*moe_is] bf16 gate|up                         */
  uint8_t* i_packed;   /* [R, moe_is/2] intermediate codes                   */
  uint8_t* i_sf;       /* [R, moe_is/16]                                     */
  uint16_t* dn_out;    /* [R, hs]       bf16                                 */
} q4o_taps;

/* Routed experts: y[T,hs] (fp32) += sum_slot w * expert(x)  (the caller zeroes
 * y, as for MoERoutedForward, include/q4t/quant/moe_gemm.h:55-74).
 * mode 0 ("test twin", tests/model_moe_test.cpp:336-372): fp32 dequantised
 *   sequential dots, no bf16 rounding of gu/dn outputs, expf, y += w*acc.
 * mode 1 ("device order", src/quant/moe_gemm.cu:158-288): exact dots times
 *   alpha, bf16 gu_out and dn_out, sigmoid 1/(1+exp(-g)) with (g*s)*u, slot
 *   order fused multiply-add combine.
 * Returns 0, or -1 on invalid dimensions.                                     */
int q4o_routed_forward(const uint16_t* x, const int32_t* ids, const float* rw,
                       float* y, const q4o_layer* L, int T, int k, int mode,
                       q4o_taps* taps);

/* y[T,hs] (fp32) += slot-order fused multiply-add of bf16 rows [*, hs] taken
 * through row_of_flat [T*k] (-1 = skipped), weights rw [T*k]
 * (src/quant/moe_gemm.cu:273-288).                                            */
void q4o_combine_rows(const uint16_t* rows, const int32_t* row_of_flat, const float* rw,
                      int T, int k, int hs, float* y);

/* Shared expert + gated combine (src/model/moe.cu:276-321, 955-971):
 * y_bf16 = bf16(routed + sigmoid(x . gate_scalar) * shared_down).
 * linear_mode is passed to q4o_bf16_linear; mode 1 also reproduces the
 * 256-thread strided partial sums and tree of the gate dot.                   */
void q4o_shared_combine(const uint16_t* x, const float* routed,
                        const q4o_layer* L, int T, int linear_mode,
                        uint16_t* y);

/* Whole layer (src/model/moe.cu:427-976).  logits_mode / linear_mode as for
 * q4o_bf16_linear, routed_mode as for q4o_routed_forward.  Optional outputs
 * (NULL to skip): logits bf16 [T,E], ids [T,k], rw [T,k], routed f32 [T,hs]. */
int q4o_moe_forward(const uint16_t* x, const q4o_layer* L, int T, int k,
                    int logits_mode, int routed_mode, int linear_mode,
                    uint16_t* y, uint16_t* logits_out, int32_t* ids_out,
                    float* rw_out, float* routed_out);

/* RMSNorm used between layers of the stacked decode benchmark
 * (src/model/hyperconnection.cu:55-110): bf16(x * rsqrt(mean(x^2)+eps)).     */
void q4o_rmsnorm_bf16(const uint16_t* x, int T, int hs, float eps,
                      uint16_t* out);
void q4o_residual_rmsnorm_bf16(uint16_t* x, const uint16_t* y, int T, int hs, float eps, uint16_t* h);
/* out[t,b,:] = bf16(residual[t,b,:] + y[t,:] * gate[t,b]) (src/model/hyperconnection.cu:286-305). */
void q4o_gated_residual_write(const uint16_t* y, const uint16_t* residual, const uint16_t* gate, int T, int hc, int hs,
                              uint16_t* out);
void q4o_moe_bf16_routed_forward(const uint16_t* x, const int32_t* ids, const float* rw, const uint16_t* gu,
                                 const uint16_t* down, int T, int k, int E, int hs, int is, float* y);

void q4o_set_num_threads(int n);
int q4o_num_threads(void);

#ifdef __cplusplus
}
#endif
#endif /* Q4T_ORACLE_H_ */
