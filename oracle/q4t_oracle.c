/*
 * CPU oracle for the NVFP4 W4A4 MoE layer.  TEST INFRASTRUCTURE ONLY: see
 * q4t_oracle.h.  Build with -ffp-contract=off so that every fused
 * multiply-add below is an explicit fmaf() and nothing else is contracted.
 */
#include "q4t_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------ */
/* bf16                                                                       */
/* ------------------------------------------------------------------------ */

static inline uint32_t f2u(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static inline float u2f(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t q4o_float_to_bf16(float f) {
  uint32_t u = f2u(f);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* NaN, as the device cvt */
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}
float q4o_bf16_to_float(uint16_t b) { return u2f((uint32_t)b << 16); }
static inline float bf16_round(float f) {
  return q4o_bf16_to_float(q4o_float_to_bf16(f));
}

/* ------------------------------------------------------------------------ */
/* e2m1 / ue4m3  (include/q4t/quant/format.h)                                 */
/* ------------------------------------------------------------------------ */

/* format.h:41-51 — magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6; bit 3 is the sign. */
float q4o_e2m1_to_float(uint8_t code) {
  static const float mag[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  float v = mag[code & 7];
  return (code & 8) ? -v : v;
}

/* format.h:66-90 — nearest value, ties to the code with an even mantissa
 * bit, saturating at 6.  The seven midpoints alternate between "tie goes
 * down" (0.25, 1.25, 2.5, 5.0) and "tie goes up" (0.75, 1.75, 3.5).  The sign
 * bit is set for every input that compares below zero, including inputs
 * that round to magnitude 0; -0.0 and NaN give an unsigned code.             */
int q4o_float_to_e2m1(float v) {
  static const float mid[7] = {0.25f, 0.75f, 1.25f, 1.75f, 2.5f, 3.5f, 5.0f};
  const float a = v < 0.0f ? -v : v;
  int code = 7;
  for (int i = 0; i < 7; ++i) {
    /* even i: stay below when a <= mid; odd i: stay below when a < mid */
    const int below = (i & 1) ? (a < mid[i]) : (a <= mid[i]);
    if (below) {
      code = i;
      break;
    }
  }
  return (v < 0.0f) ? (code | 8) : code;
}

/* format.h:103-114 — unsigned e4m3: bias 7, subnormal step 2^-9, 0x7F reads
 * as 0.  Bit 7 is ignored.                                                   */
float q4o_e4m3_to_float(uint8_t code) {
  const int ex = code >> 3;
  const int man = code & 7;
  if (ex == 0) return (float)man * 0.001953125f;
  if (ex == 15 && man == 7) return 0.0f;
  return ldexpf(1.0f + (float)man * 0.125f, ex - 7);
}

/* format.h:120-164 — nearest-even encoder for non-negative scales, 448 and
 * above saturate to 0x7E.  Restated with frexpf/rintf (default rounding mode
 * is nearest-even) instead of the reference's normalisation loops.           */
uint8_t q4o_float_to_e4m3(float v) {
  const float a = v < 0.0f ? -v : v;
  if (a == 0.0f) return 0;
  if (a >= 448.0f) return 0x7E;
  if (a < 0.015625f) return (uint8_t)(int)rintf(a * 512.0f); /* 8 = smallest normal */
  int ex;
  const float m = 2.0f * frexpf(a, &ex); /* m in [1,2), a = m * 2^(ex-1) */
  int man = (int)rintf((m - 1.0f) * 8.0f);
  int e = ex - 1 + 7;
  if (man == 8) {
    man = 0;
    ++e;
  }
  if (e > 15 || (e == 15 && man > 6)) return 0x7E;
  return (uint8_t)((e << 3) | man);
}

void q4o_float_to_e4m3_bulk(const float* in, size_t n, uint8_t* out) {
  for (size_t i = 0; i < n; ++i) out[i] = q4o_float_to_e4m3(in[i]);
}
void q4o_float_to_e2m1_bulk(const float* in, size_t n, uint8_t* out) {
  for (size_t i = 0; i < n; ++i) out[i] = (uint8_t)q4o_float_to_e2m1(in[i]);
}

/* ------------------------------------------------------------------------ */
/* scale-factor swizzle  (include/q4t/quant/swizzle.h)                        */
/* ------------------------------------------------------------------------ */

/* swizzle.h:34-44 — 128-row x 4-group atoms of 512 bytes; inside an atom the
 * byte index is (row%32)*16 + ((row%128)/32)*4 + group%4; atoms run along K
 * first, then along rows.                                                    */
size_t q4o_sf_offset(int row, int group, int num_g_tiles) {
  const size_t in_atom =
      (size_t)(row & 31) * 16 + (size_t)((row & 127) >> 5) * 4 + (size_t)(group & 3);
  const size_t atom = (size_t)(row >> 7) * (size_t)num_g_tiles + (size_t)(group >> 2);
  return atom * 512 + in_atom;
}
/* swizzle.h:47-50 */
int q4o_sf_num_gtiles(int K) { return (K / 16 + 3) / 4; }
/* swizzle.h:53-57 */
size_t q4o_sf_buffer_size(int rows, int K) {
  return (size_t)((rows + 127) / 128) * (size_t)q4o_sf_num_gtiles(K) * 512;
}
/* swizzle.h:63-75 */
void q4o_swizzle_sf(const uint8_t* row_major, int rows, int K, uint8_t* out) {
  const int groups = K / 16;
  const int nt = q4o_sf_num_gtiles(K);
  memset(out, 0, q4o_sf_buffer_size(rows, K));
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < groups; ++g)
      out[q4o_sf_offset(r, g, nt)] = row_major[(size_t)r * groups + g];
}

/* ------------------------------------------------------------------------ */
/* quantiser                                                                  */
/* ------------------------------------------------------------------------ */

/* One group of 16 (src/quant/act_quant.cu:62-90, tests/quant_fp4_test.cpp:78-94):
 * block scale = amax/6 (1 when the group is all zero); stored scale =
 * e4m3(block/global); codes are rounded against decode(scale)*global through
 * its reciprocal; low nibble holds the even element.                         */
static inline uint8_t quantize_group(const float* a, float global_scale,
                                     uint8_t* bytes8) {
  float gmax = 0.0f;
  for (int j = 0; j < 16; ++j) gmax = fmaxf(gmax, fabsf(a[j]));
  const float block = gmax > 0.0f ? gmax / 6.0f : 1.0f;
  const uint8_t sf = q4o_float_to_e4m3(block / global_scale);
  const float eff = q4o_e4m3_to_float(sf) * global_scale;
  const float inv = eff > 0.0f ? 1.0f / eff : 0.0f;
  for (int j = 0; j < 8; ++j) {
    const int lo = q4o_float_to_e2m1(a[2 * j] * inv);
    const int hi = q4o_float_to_e2m1(a[2 * j + 1] * inv);
    bytes8[j] = (uint8_t)((hi << 4) | (lo & 0xF));
  }
  return sf;
}

void q4o_quantize_f32(const float* v, int rows, int K, float global_scale,
                      uint8_t* packed, uint8_t* sf_rm) {
  const int groups = K / 16;
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < groups; ++g)
      sf_rm[(size_t)r * groups + g] =
          quantize_group(v + (size_t)r * K + g * 16, global_scale,
                         packed + ((size_t)r * groups + g) * 8);
}

void q4o_quantize_bf16(const uint16_t* x, int rows, int K, float global_scale,
                       uint8_t* packed, uint8_t* sf_swizzled) {
  const int groups = K / 16;
  const int nt = q4o_sf_num_gtiles(K);
  memset(sf_swizzled, 0, q4o_sf_buffer_size(rows, K));
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < groups; ++g) {
      float a[16];
      for (int j = 0; j < 16; ++j)
        a[j] = q4o_bf16_to_float(x[(size_t)r * K + g * 16 + j]);
      sf_swizzled[q4o_sf_offset(r, g, nt)] = quantize_group(
          a, global_scale, packed + ((size_t)r * groups + g) * 8);
    }
}

void q4o_dequant_to_bf16(const uint8_t* packed, const uint8_t* sf_rm, int N,
                         int K, float inv_global, uint16_t* out) {
  const int groups = K / 16;
  for (int r = 0; r < N; ++r)
    for (int g = 0; g < groups; ++g) {
      const float scale =
          q4o_e4m3_to_float(sf_rm[(size_t)r * groups + g]) * inv_global;
      const uint8_t* p = packed + ((size_t)r * groups + g) * 8;
      uint16_t* d = out + (size_t)r * K + g * 16;
      for (int j = 0; j < 8; ++j) {
        d[2 * j] = q4o_float_to_bf16(q4o_e2m1_to_float(p[j] & 0xF) * scale);
        d[2 * j + 1] = q4o_float_to_bf16(q4o_e2m1_to_float(p[j] >> 4) * scale);
      }
    }
}

void q4o_dequant_to_f32(const uint8_t* packed, const uint8_t* sf_rm, int rows,
                        int K, float global_scale, float* out) {
  const int groups = K / 16;
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < groups; ++g) {
      const float gs =
          q4o_e4m3_to_float(sf_rm[(size_t)r * groups + g]) * global_scale;
      const uint8_t* p = packed + ((size_t)r * groups + g) * 8;
      float* d = out + (size_t)r * K + g * 16;
      for (int j = 0; j < 8; ++j) {
        d[2 * j] = q4o_e2m1_to_float(p[j] & 0xF) * gs;
        d[2 * j + 1] = q4o_e2m1_to_float(p[j] >> 4) * gs;
      }
    }
}

/* ------------------------------------------------------------------------ */
/* decoded operands for the two GEMM modes                                    */
/* ------------------------------------------------------------------------ */

/* Exact form of one NVFP4 row: codes as integers (twice the e2m1 value) and
 * each scale as mant * 2^(ex-10) with ex in [1,15] (0x7F and 0 give mant 0). */
typedef struct {
  int8_t* v2;   /* [K] */
  int16_t* sm;  /* [K/16] mantissa 0..15 */
  int8_t* se;   /* [K/16] exponent 1..15 */
} exact_row;

static void decode_exact(const uint8_t* packed_row, const uint8_t* sf,
                         int sf_row, int sf_swizzled, int K, exact_row* o) {
  static const int8_t twice[8] = {0, 1, 2, 3, 4, 6, 8, 12};
  const int groups = K / 16;
  const int nt = q4o_sf_num_gtiles(K);
  for (int i = 0; i < K / 2; ++i) {
    const uint8_t b = packed_row[i];
    const int lo = b & 0xF, hi = b >> 4;
    o->v2[2 * i] = (int8_t)((lo & 8) ? -twice[lo & 7] : twice[lo & 7]);
    o->v2[2 * i + 1] = (int8_t)((hi & 8) ? -twice[hi & 7] : twice[hi & 7]);
  }
  for (int g = 0; g < groups; ++g) {
    const uint8_t c = sf_swizzled ? sf[q4o_sf_offset(sf_row, g, nt)]
                                  : sf[(size_t)sf_row * groups + g];
    const int ex = (c >> 3) & 15, man = c & 7;
    if (ex == 0) {
      o->sm[g] = (int16_t)man;
      o->se[g] = 1;
    } else if (ex == 15 && man == 7) {
      o->sm[g] = 0;
      o->se[g] = 1;
    } else {
      o->sm[g] = (int16_t)(8 + man);
      o->se[g] = (int8_t)ex;
    }
  }
}

/* Exact dot of two decoded rows, in units of 2^-20:
 * sum_g (sum_j a2 w2) * ma mw * 2^(ea+ew-2), a2/w2 being twice the values.  Every term is below 2^47 and
 * there are at most a few hundred groups, so int64 never overflows.          */
static inline double exact_dot(const exact_row* a, const exact_row* w, int K) {
  const int groups = K / 16;
  int64_t acc = 0;
  for (int g = 0; g < groups; ++g) {
    const int8_t* pa = a->v2 + g * 16;
    const int8_t* pw = w->v2 + g * 16;
    int s = 0;
    for (int j = 0; j < 16; ++j) s += (int)pa[j] * (int)pw[j];
    acc += (int64_t)s * (int64_t)(a->sm[g] * w->sm[g]) *
           ((int64_t)1 << (a->se[g] + w->se[g] - 2));
  }
  return ldexp((double)acc, -20);
}

static exact_row alloc_exact(int rows, int K) {
  exact_row r;
  r.v2 = (int8_t*)malloc((size_t)rows * K);
  r.sm = (int16_t*)malloc((size_t)rows * (K / 16) * sizeof(int16_t));
  r.se = (int8_t*)malloc((size_t)rows * (K / 16));
  return r;
}
static void free_exact(exact_row* r) {
  free(r->v2);
  free(r->sm);
  free(r->se);
}
static inline exact_row exact_at(const exact_row* base, int row, int K) {
  exact_row r;
  r.v2 = base->v2 + (size_t)row * K;
  r.sm = base->sm + (size_t)row * (K / 16);
  r.se = base->se + (size_t)row * (K / 16);
  return r;
}

/* Sequential fp32 dot, the order of the reference's host loops.              */
static inline float seq_dot(const float* a, const float* w, int K) {
  float acc = 0.0f;
  for (int c = 0; c < K; ++c) acc += a[c] * w[c];
  return acc;
}

/* Dequantise one weight row with swizzled SF (tests/model_moe_test.cpp:137-151). */
static void dequant_row_swz(const uint8_t* packed, const uint8_t* sf, int row,
                            int K, float global_scale, float* out) {
  const int groups = K / 16;
  const int nt = q4o_sf_num_gtiles(K);
  for (int g = 0; g < groups; ++g) {
    const float gs = q4o_e4m3_to_float(sf[q4o_sf_offset(row, g, nt)]) * global_scale;
    const uint8_t* p = packed + ((size_t)row * groups + g) * 8;
    for (int j = 0; j < 8; ++j) {
      out[g * 16 + 2 * j] = q4o_e2m1_to_float(p[j] & 0xF) * gs;
      out[g * 16 + 2 * j + 1] = q4o_e2m1_to_float(p[j] >> 4) * gs;
    }
  }
}

void q4o_fp4_gemm(const uint8_t* w_packed, const uint8_t* w_sf,
                  const uint8_t* a_packed, const uint8_t* a_sf, float* out,
                  int M, int N, int K, float inv_w_global, float inv_a_global,
                  int mode) {
  if (mode == 0) {
    float* wd = (float*)malloc((size_t)N * K * sizeof(float));
    float* ad = (float*)malloc((size_t)M * K * sizeof(float));
#pragma omp parallel for schedule(static)
    for (int n = 0; n < N; ++n)
      dequant_row_swz(w_packed, w_sf, n, K, inv_w_global, wd + (size_t)n * K);
    for (int m = 0; m < M; ++m)
      dequant_row_swz(a_packed, a_sf, m, K, inv_a_global, ad + (size_t)m * K);
#pragma omp parallel for collapse(2) schedule(static)
    for (int m = 0; m < M; ++m)
      for (int n = 0; n < N; ++n)
        out[(size_t)m * N + n] = seq_dot(ad + (size_t)m * K, wd + (size_t)n * K, K);
    free(wd);
    free(ad);
    return;
  }
  exact_row W = alloc_exact(N, K), A = alloc_exact(M, K);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    exact_row r = exact_at(&W, n, K);
    decode_exact(w_packed + (size_t)n * (K / 2), w_sf, n, 1, K, &r);
  }
  for (int m = 0; m < M; ++m) {
    exact_row r = exact_at(&A, m, K);
    decode_exact(a_packed + (size_t)m * (K / 2), a_sf, m, 1, K, &r);
  }
  const float alpha = inv_w_global * inv_a_global;
#pragma omp parallel for collapse(2) schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      exact_row a = exact_at(&A, m, K), w = exact_at(&W, n, K);
      out[(size_t)m * N + n] = (float)(exact_dot(&a, &w, K) * (double)alpha);
    }
  free_exact(&W);
  free_exact(&A);
}

/* ------------------------------------------------------------------------ */
/* BF16 linear                                                                */
/* ------------------------------------------------------------------------ */

/* src/model/gemv.cu:84-112 — one warp per output: lane l owns the 8-element
 * chunks l, l+32, ...; inside a chunk the four even elements feed one
 * accumulator and the four odd ones another, each by fused multiply-add;
 * the two are added, then lanes are folded by shuffle-down 16,8,4,2,1.      */
static float gemv_order_dot(const uint16_t* x, const uint16_t* w, int K) {
  float lane_sum[32];
  const int k8 = K / 8;
  for (int l = 0; l < 32; ++l) {
    float ax = 0.0f, ay = 0.0f;
    for (int i = l; i < k8; i += 32)
      for (int j = 0; j < 4; ++j) {
        ax = fmaf(q4o_bf16_to_float(x[i * 8 + 2 * j]),
                  q4o_bf16_to_float(w[i * 8 + 2 * j]), ax);
        ay = fmaf(q4o_bf16_to_float(x[i * 8 + 2 * j + 1]),
                  q4o_bf16_to_float(w[i * 8 + 2 * j + 1]), ay);
      }
    float s = ax + ay;
    for (int c = k8 * 8 + l; c < K; c += 32)
      s += q4o_bf16_to_float(x[c]) * q4o_bf16_to_float(w[c]);
    lane_sum[l] = s;
  }
  for (int off = 16; off > 0; off >>= 1)
    for (int l = 0; l < off; ++l) lane_sum[l] += lane_sum[l + off];
  return lane_sum[0];
}

void q4o_bf16_linear(const uint16_t* x, const uint16_t* w, uint16_t* y, int M,
                     int N, int K, int mode) {
  float* xf = NULL;
  float* wf = NULL;
  if (mode == 0) {
    xf = (float*)malloc((size_t)M * K * sizeof(float));
    wf = (float*)malloc((size_t)N * K * sizeof(float));
    for (size_t i = 0; i < (size_t)M * K; ++i) xf[i] = q4o_bf16_to_float(x[i]);
    for (size_t i = 0; i < (size_t)N * K; ++i) wf[i] = q4o_bf16_to_float(w[i]);
  }
#pragma omp parallel for collapse(2) schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float v;
      if (mode == 0)
        v = seq_dot(xf + (size_t)m * K, wf + (size_t)n * K, K);
      else
        v = 1.0f * gemv_order_dot(x + (size_t)m * K, w + (size_t)n * K, K);
      y[(size_t)m * N + n] = q4o_float_to_bf16(v);
    }
  free(xf);
  free(wf);
}

/* ------------------------------------------------------------------------ */
/* router                                                                     */
/* ------------------------------------------------------------------------ */

void q4o_router_topk(const uint16_t* logits, int T, int E, int k, int32_t* ids,
                     float* weights) {
  float* vals = (float*)malloc((size_t)E * sizeof(float));
  for (int t = 0; t < T; ++t) {
    for (int e = 0; e < E; ++e) vals[e] = q4o_bf16_to_float(logits[(size_t)t * E + e]);
    float sel[64];
    for (int i = 0; i < k; ++i) {
      /* src/model/moe.cu:154-192: largest value, lowest id on ties; the
       * scan starts from (-1e30, id 0) and the winner is masked to -1e30.    */
      float best = -1e30f;
      int bi = 0;
      for (int e = 0; e < E; ++e)
        if (vals[e] > best || (vals[e] == best && e < bi)) {
          best = vals[e];
          bi = e;
        }
      sel[i] = best;
      ids[(size_t)t * k + i] = bi;
      vals[bi] = -1e30f;
    }
    /* moe.cu:196-211: softmax over the selected values, in selection order. */
    float mx = sel[0];
    for (int i = 1; i < k; ++i) mx = fmaxf(mx, sel[i]);
    float sum = 0.0f;
    for (int i = 0; i < k; ++i) {
      sel[i] = expf(sel[i] - mx);
      sum += sel[i];
    }
    const float inv = 1.0f / sum;
    for (int i = 0; i < k; ++i) weights[(size_t)t * k + i] = sel[i] * inv;
  }
  free(vals);
}

void q4o_permutation(const int32_t* ids, int T, int k, int E, int32_t* counts,
                     int32_t* offsets, int32_t* row_of_flat,
                     int32_t* flat_of_row) {
  const int R = T * k;
  memset(counts, 0, (size_t)E * sizeof(int32_t));
  for (int f = 0; f < R; ++f)
    if (ids[f] >= 0 && ids[f] < E) counts[ids[f]]++;
  offsets[0] = 0;
  for (int e = 0; e < E; ++e) offsets[e + 1] = offsets[e] + counts[e];
  int32_t* cursor = (int32_t*)malloc((size_t)E * sizeof(int32_t));
  memcpy(cursor, offsets, (size_t)E * sizeof(int32_t));
  for (int r = 0; r < R; ++r) flat_of_row[r] = -1;
  for (int f = 0; f < R; ++f) {
    const int e = ids[f];
    if (e < 0 || e >= E) {
      row_of_flat[f] = -1;
      continue;
    }
    const int r = cursor[e]++;
    row_of_flat[f] = r;
    flat_of_row[r] = f;
  }
  free(cursor);
}

/* ------------------------------------------------------------------------ */
/* routed experts                                                             */
/* ------------------------------------------------------------------------ */

static inline float sigmoid_dev(float g) { return 1.0f / (1.0f + expf(-g)); }

int q4o_routed_forward(const uint16_t* x, const int32_t* ids, const float* rw,
                       float* y, const q4o_layer* L, int T, int k, int mode,
                       q4o_taps* taps) {
  const int E = L->E, hs = L->hs, is = L->moe_is;
  if (T <= 0 || k <= 0 || E <= 0 || hs <= 0 || is <= 0 || hs % 16 || is % 16)
    return -1;
  const int R = T * k;
  int32_t* counts = (int32_t*)malloc((size_t)E * 4);
  int32_t* offsets = (int32_t*)malloc((size_t)(E + 1) * 4);
  int32_t* row_of_flat = (int32_t*)malloc((size_t)R * 4);
  int32_t* flat_of_row = (int32_t*)malloc((size_t)R * 4);
  q4o_permutation(ids, T, k, E, counts, offsets, row_of_flat, flat_of_row);
  const size_t gu_sf_block = q4o_sf_buffer_size(2 * is, hs);
  const size_t dn_sf_block = q4o_sf_buffer_size(hs, is);
  /* per grouped row: down-projection output (fp32 in mode 0, bf16-rounded
   * fp32 in mode 1), consumed by the combine below.                          */
  float* dn_rows = (float*)malloc((size_t)R * hs * sizeof(float));

#pragma omp parallel for schedule(dynamic, 1)
  for (int e = 0; e < E; ++e) {
    const int Me = counts[e];
    if (Me == 0) continue;
    const uint8_t* gu_p = L->gu_packed + (size_t)e * is * hs;
    const uint8_t* gu_s = L->gu_sf + (size_t)e * gu_sf_block;
    const uint8_t* dn_p = L->dn_packed + (size_t)e * hs * (is / 2);
    const uint8_t* dn_s = L->dn_sf + (size_t)e * dn_sf_block;
    const float gu_in = L->gu_input_scale[e], dn_in = L->dn_input_scale[e];
    const float gu_alpha = L->gu_w_scale2[e] * gu_in; /* moe_gemm.cu:536-537 */
    const float dn_alpha = L->dn_w_scale2[e] * dn_in;

    float* wgu_f = NULL;
    float* wdn_f = NULL;
    exact_row wgu_x, wdn_x;
    memset(&wgu_x, 0, sizeof wgu_x);
    memset(&wdn_x, 0, sizeof wdn_x);
    if (mode == 0) {
      /* per-expert dequant cache (tests/model_moe_test.cpp:296-335) */
      wgu_f = (float*)malloc((size_t)2 * is * hs * sizeof(float));
      wdn_f = (float*)malloc((size_t)hs * is * sizeof(float));
      for (int n = 0; n < 2 * is; ++n)
        dequant_row_swz(gu_p, gu_s, n, hs, L->gu_w_scale2[e], wgu_f + (size_t)n * hs);
      for (int n = 0; n < hs; ++n)
        dequant_row_swz(dn_p, dn_s, n, is, L->dn_w_scale2[e], wdn_f + (size_t)n * is);
    } else {
      wgu_x = alloc_exact(2 * is, hs);
      wdn_x = alloc_exact(hs, is);
      for (int n = 0; n < 2 * is; ++n) {
        exact_row r = exact_at(&wgu_x, n, hs);
        decode_exact(gu_p + (size_t)n * (hs / 2), gu_s, n, 1, hs, &r);
      }
      for (int n = 0; n < hs; ++n) {
        exact_row r = exact_at(&wdn_x, n, is);
        decode_exact(dn_p + (size_t)n * (is / 2), dn_s, n, 1, is, &r);
      }
    }
    float* arow = (float*)malloc((size_t)hs * sizeof(float));
    uint8_t* a_p = (uint8_t*)malloc((size_t)hs / 2);
    uint8_t* a_s = (uint8_t*)malloc((size_t)hs / 16);
    float* a_dq = (float*)malloc((size_t)hs * sizeof(float));
    float* h = (float*)malloc((size_t)2 * is * sizeof(float));
    float* inter = (float*)malloc((size_t)is * sizeof(float));
    uint8_t* i_p = (uint8_t*)malloc((size_t)is / 2);
    uint8_t* i_s = (uint8_t*)malloc((size_t)is / 16);
    float* i_dq = (float*)malloc((size_t)is * sizeof(float));
    exact_row a_x = alloc_exact(1, hs), i_x = alloc_exact(1, is);

    for (int j = 0; j < Me; ++j) {
      const int row = offsets[e] + j;
      const int t = flat_of_row[row] / k;
      /* input quantisation with this expert's input scale (moe_gemm.cu:158-196) */
      for (int c = 0; c < hs; ++c) arow[c] = q4o_bf16_to_float(x[(size_t)t * hs + c]);
      q4o_quantize_f32(arow, 1, hs, gu_in, a_p, a_s);
      if (taps && taps->a_packed) memcpy(taps->a_packed + (size_t)row * (hs / 2), a_p, hs / 2);
      if (taps && taps->a_sf) memcpy(taps->a_sf + (size_t)row * (hs / 16), a_s, hs / 16);
      if (mode == 0) {
        q4o_dequant_to_f32(a_p, a_s, 1, hs, gu_in, a_dq);
        for (int n = 0; n < 2 * is; ++n) h[n] = seq_dot(a_dq, wgu_f + (size_t)n * hs, hs);
        /* tests/model_moe_test.cpp:358-361 */
        for (int c = 0; c < is; ++c) {
          const float g = h[c], u = h[is + c];
          inter[c] = (g / (1.0f + expf(-g))) * u;
        }
      } else {
        decode_exact(a_p, a_s, 0, 0, hs, &a_x);
        for (int n = 0; n < 2 * is; ++n) {
          exact_row w = exact_at(&wgu_x, n, hs);
          h[n] = bf16_round((float)(exact_dot(&a_x, &w, hs) * (double)gu_alpha));
        }
        /* moe_gemm.cu:219-224: s = 1/(1+exp(-g)); a = g*s*u, left to right */
        for (int c = 0; c < is; ++c) {
          const float g = h[c], u = h[is + c];
          inter[c] = g * sigmoid_dev(g) * u;
        }
      }
      if (taps && taps->gu_out)
        for (int n = 0; n < 2 * is; ++n)
          taps->gu_out[(size_t)row * 2 * is + n] = q4o_float_to_bf16(h[n]);
      q4o_quantize_f32(inter, 1, is, dn_in, i_p, i_s);
      if (taps && taps->i_packed) memcpy(taps->i_packed + (size_t)row * (is / 2), i_p, is / 2);
      if (taps && taps->i_sf) memcpy(taps->i_sf + (size_t)row * (is / 16), i_s, is / 16);
      float* drow = dn_rows + (size_t)row * hs;
      if (mode == 0) {
        q4o_dequant_to_f32(i_p, i_s, 1, is, dn_in, i_dq);
        for (int c = 0; c < hs; ++c) drow[c] = seq_dot(i_dq, wdn_f + (size_t)c * is, is);
      } else {
        decode_exact(i_p, i_s, 0, 0, is, &i_x);
        for (int c = 0; c < hs; ++c) {
          exact_row w = exact_at(&wdn_x, c, is);
          drow[c] = bf16_round((float)(exact_dot(&i_x, &w, is) * (double)dn_alpha));
        }
      }
      if (taps && taps->dn_out)
        for (int c = 0; c < hs; ++c)
          taps->dn_out[(size_t)row * hs + c] = q4o_float_to_bf16(drow[c]);
    }
    free(arow); free(a_p); free(a_s); free(a_dq); free(h); free(inter);
    free(i_p); free(i_s); free(i_dq);
    free_exact(&a_x); free_exact(&i_x);
    if (mode == 0) { free(wgu_f); free(wdn_f); }
    else { free_exact(&wgu_x); free_exact(&wdn_x); }
  }

  /* combine */
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < hs; ++c) {
      if (mode == 0) {
        /* tests/model_moe_test.cpp:366-370: y += w * acc, slot by slot */
        float acc = y[(size_t)t * hs + c];
        for (int s = 0; s < k; ++s) {
          const int r = row_of_flat[t * k + s];
          if (r >= 0) acc += rw[t * k + s] * dn_rows[(size_t)r * hs + c];
        }
        y[(size_t)t * hs + c] = acc;
      } else {
        /* moe_gemm.cu:273-288 with the compiler's contraction made explicit
         * (tests/mtp_moe_path_test.cpp:242-248): acc = fma(w, d, acc); y += acc */
        float acc = 0.0f;
        for (int s = 0; s < k; ++s) {
          const int r = row_of_flat[t * k + s];
          if (r >= 0) acc = fmaf(rw[t * k + s], dn_rows[(size_t)r * hs + c], acc);
        }
        y[(size_t)t * hs + c] += acc;
      }
    }
  free(counts); free(offsets); free(row_of_flat); free(flat_of_row); free(dn_rows);
  return 0;
}

/* Slot-order combine of bf16 rows addressed through row_of_flat
 * (CombineGroupedKernel, src/quant/moe_gemm.cu:273-288): y += fma chain from 0. */
void q4o_combine_rows(const uint16_t* rows, const int32_t* row_of_flat, const float* rw,
                      int T, int k, int hs, float* y) {
#pragma omp parallel for schedule(static)
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < hs; ++c) {
      float acc = 0.0f;
      for (int s = 0; s < k; ++s) {
        const int r = row_of_flat[t * k + s];
        if (r >= 0) acc = fmaf(rw[t * k + s], q4o_bf16_to_float(rows[(size_t)r * hs + c]), acc);
      }
      y[(size_t)t * hs + c] += acc;
    }
}

/* ------------------------------------------------------------------------ */
/* shared expert + gated combine                                              */
/* ------------------------------------------------------------------------ */

void q4o_shared_combine(const uint16_t* x, const float* routed,
                        const q4o_layer* L, int T, int linear_mode,
                        uint16_t* y) {
  const int hs = L->hs, sis = L->shared_is;
  uint16_t* gu = (uint16_t*)malloc((size_t)T * 2 * sis * 2);
  uint16_t* act = (uint16_t*)malloc((size_t)T * sis * 2);
  uint16_t* down = (uint16_t*)malloc((size_t)T * hs * 2);
  q4o_bf16_linear(x, L->shared_gu, gu, T, 2 * sis, hs, linear_mode);
  /* src/model/moe.cu:276-287 */
  for (int t = 0; t < T; ++t)
    for (int c = 0; c < sis; ++c) {
      const float g = q4o_bf16_to_float(gu[(size_t)t * 2 * sis + c]);
      const float u = q4o_bf16_to_float(gu[(size_t)t * 2 * sis + sis + c]);
      act[(size_t)t * sis + c] = q4o_float_to_bf16((g * sigmoid_dev(g)) * u);
    }
  q4o_bf16_linear(act, L->shared_down, down, T, hs, sis, linear_mode);
  for (int t = 0; t < T; ++t) {
    float dot;
    if (linear_mode == 0) {
      /* tests/model_moe_test.cpp:394-397 */
      dot = 0.0f;
      for (int c = 0; c < hs; ++c)
        dot += q4o_bf16_to_float(x[(size_t)t * hs + c]) *
               q4o_bf16_to_float(L->shared_gate_scalar[c]);
    } else {
      /* src/model/moe.cu:302-311: 256 strided partials by fused multiply-add,
       * then a halving tree in shared memory.                                */
      float part[256];
      for (int i = 0; i < 256; ++i) {
        float a = 0.0f;
        for (int c = i; c < hs; c += 256)
          a = fmaf(q4o_bf16_to_float(x[(size_t)t * hs + c]),
                   q4o_bf16_to_float(L->shared_gate_scalar[c]), a);
        part[i] = a;
      }
      for (int off = 128; off > 0; off >>= 1)
        for (int i = 0; i < off; ++i) part[i] += part[i + off];
      dot = part[0];
    }
    const float gate = sigmoid_dev(dot);
    for (int c = 0; c < hs; ++c) {
      const float sd = q4o_bf16_to_float(down[(size_t)t * hs + c]);
      const float r = routed[(size_t)t * hs + c];
      /* moe.cu:317-318; the device contracts r + gate*sd into one fma */
      const float v = linear_mode == 0 ? r + gate * sd : fmaf(gate, sd, r);
      y[(size_t)t * hs + c] = q4o_float_to_bf16(v);
    }
  }
  free(gu); free(act); free(down);
}

int q4o_moe_forward(const uint16_t* x, const q4o_layer* L, int T, int k,
                    int logits_mode, int routed_mode, int linear_mode,
                    uint16_t* y, uint16_t* logits_out, int32_t* ids_out,
                    float* rw_out, float* routed_out) {
  const int E = L->E, hs = L->hs;
  if (T <= 0) return 0;
  if (k <= 0 || k > 16) return -1; /* src/model/moe.cu:443 */
  uint16_t* logits = (uint16_t*)malloc((size_t)T * E * 2);
  int32_t* ids = (int32_t*)malloc((size_t)T * k * 4);
  float* rw = (float*)malloc((size_t)T * k * 4);
  float* routed = (float*)calloc((size_t)T * hs, 4);
  q4o_bf16_linear(x, L->gate, logits, T, E, hs, logits_mode);
  q4o_router_topk(logits, T, E, k, ids, rw);
  int rc = q4o_routed_forward(x, ids, rw, routed, L, T, k, routed_mode, NULL);
  if (rc == 0) q4o_shared_combine(x, routed, L, T, linear_mode, y);
  if (logits_out) memcpy(logits_out, logits, (size_t)T * E * 2);
  if (ids_out) memcpy(ids_out, ids, (size_t)T * k * 4);
  if (rw_out) memcpy(rw_out, rw, (size_t)T * k * 4);
  if (routed_out) memcpy(routed_out, routed, (size_t)T * hs * 4);
  free(logits); free(ids); free(rw); free(routed);
  return rc;
}

/* RMSNorm of bf16 rows without a learned weight, in the summation order of the reference's
 * GroupedRmsNormKernel (src/model/hyperconnection.cu:55-110): one warp per row, lane l sums
 * the squares of elements [8i, 8i+8) for i = l, l+32, ... (eight fused multiply-adds per
 * group, then one add into the lane's partial), the 32 partials are combined by the xor
 * butterfly 16, 8, 4, 2, 1, and the row is scaled by 1/sqrt(mean + eps).  The device code of
 * the reference uses rsqrtf (approximate, not reproducible on a host); the correctly rounded
 * reciprocal square root stands in for it here and in the CUDA path (at most 2 ulp apart). */
void q4o_rmsnorm_bf16(const uint16_t* x, int T, int hs, float eps, uint16_t* out) {
  const int n8 = hs / 8;
  for (int t = 0; t < T; ++t) {
    const uint16_t* row = x + (size_t)t * hs;
    float part[32];
    for (int l = 0; l < 32; ++l) {
      float acc = 0.0f;
      for (int i = l; i < n8; i += 32) {
        float s = 0.0f;
        for (int j = 0; j < 8; ++j) {
          const float v = q4o_bf16_to_float(row[8 * i + j]);
          s = fmaf(v, v, s);
        }
        acc += s;
      }
      for (int i = n8 * 8 + l; i < hs; i += 32) {
        const float v = q4o_bf16_to_float(row[i]);
        acc = fmaf(v, v, acc);
      }
      part[l] = acc;
    }
    for (int off = 16; off > 0; off >>= 1) {
      float next[32];
      for (int l = 0; l < 32; ++l) next[l] = part[l] + part[l ^ off];
      memcpy(part, next, sizeof(part));
    }
    const float r = 1.0f / sqrtf(part[0] / (float)hs + eps);
    for (int c = 0; c < hs; ++c) out[(size_t)t * hs + c] = q4o_float_to_bf16(q4o_bf16_to_float(row[c]) * r);
  }
}

/* x <- bf16(x + y) (fp32 add, one rounding), then h <- RMSNorm(x): the step between two
 * layers of the decode stack.  y may be NULL (first layer: only the norm). */
void q4o_residual_rmsnorm_bf16(uint16_t* x, const uint16_t* y, int T, int hs, float eps, uint16_t* h) {
  if (y)
    for (size_t i = 0; i < (size_t)T * hs; ++i)
      x[i] = q4o_float_to_bf16(q4o_bf16_to_float(x[i]) + q4o_bf16_to_float(y[i]));
  q4o_rmsnorm_bf16(x, T, hs, eps, h);
}

/* The layer's gated residual write (CombineWithGateKernel, src/model/hyperconnection.cu:286-305;
 * GatedResidualFrame::Write after MoEForward, src/model/decoder_layer.cu:708): out[t, b, c] =
 * bf16(R[t, b, c] + y[t, c] * gate[t, b]), all operands bf16.  The device compiler contracts the
 * multiply-add, so it is one fused multiply-add here. */
void q4o_gated_residual_write(const uint16_t* y, const uint16_t* residual, const uint16_t* gate, int T, int hc, int hs,
                              uint16_t* out) {
  for (int t = 0; t < T; ++t)
    for (int b = 0; b < hc; ++b) {
      const float inj = q4o_bf16_to_float(gate[(size_t)t * hc + b]);
      const size_t at = ((size_t)t * hc + b) * hs;
      for (int c = 0; c < hs; ++c)
        out[at + c] = q4o_float_to_bf16(fmaf(q4o_bf16_to_float(y[(size_t)t * hs + c]), inj,
                                             q4o_bf16_to_float(residual[at + c])));
    }
}

/* The MTP draft layer's BF16 routed experts (src/mtp/moe_bf16.cu:93-131, 340-420): per
 * (token, slot) h = bf16(x . W_gu[e]^T) with fp32 accumulation (sequential here; the
 * reference's library GEMM leaves the order open), inter = bf16((g * (1/(1+expf(-g)))) * u),
 * out = bf16(inter . W_dn[e]^T), y[t] += r * out.  The reference adds with atomicAdd in
 * no fixed order; here the slots are added in order with a fused multiply-add, as the
 * NVFP4 layer does.  gu [E, 2*is, hs], down [E, hs, is] bf16; y fp32 [T, hs] accumulated into. */
void q4o_moe_bf16_routed_forward(const uint16_t* x, const int32_t* ids, const float* rw, const uint16_t* gu,
                                 const uint16_t* down, int T, int k, int E, int hs, int is, float* y) {
#pragma omp parallel for schedule(dynamic)
  for (int t = 0; t < T; ++t) {
    float* h = (float*)malloc(sizeof(float) * (size_t)(2 * is + is + hs));
    float* inter = h + 2 * is;
    float* xf = inter + is;
    for (int c = 0; c < hs; ++c) xf[c] = q4o_bf16_to_float(x[(size_t)t * hs + c]);
    for (int s = 0; s < k; ++s) {
      const int e = ids[t * k + s];
      if (e < 0 || e >= E) continue;
      const uint16_t* wg = gu + (size_t)e * 2 * is * hs;
      for (int n = 0; n < 2 * is; ++n) {
        float acc = 0.0f;
        for (int c = 0; c < hs; ++c) acc += xf[c] * q4o_bf16_to_float(wg[(size_t)n * hs + c]);
        h[n] = q4o_bf16_to_float(q4o_float_to_bf16(acc));
      }
      for (int n = 0; n < is; ++n) {
        const float g = h[n], u = h[is + n];
        const float sg = 1.0f / (1.0f + expf(-g));
        inter[n] = q4o_bf16_to_float(q4o_float_to_bf16((g * sg) * u));
      }
      const uint16_t* wd = down + (size_t)e * hs * is;
      const float w = rw[t * k + s];
      for (int c = 0; c < hs; ++c) {
        float acc = 0.0f;
        for (int n = 0; n < is; ++n) acc += inter[n] * q4o_bf16_to_float(wd[(size_t)c * is + n]);
        const float o = q4o_bf16_to_float(q4o_float_to_bf16(acc));
        y[(size_t)t * hs + c] = fmaf(w, o, y[(size_t)t * hs + c]);
      }
    }
    free(h);
  }
}

/* Sets the number of OpenMP threads of this library (a launcher may have pinned the process
 * to one thread through the environment before the runtime was loaded). */
void q4o_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

int q4o_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
