// Thin extern "C" wrapper over the REFERENCE's own header-only format and
// swizzle primitives, compiled from the reference tree where it lies
// (-I<reference>/include).  The resulting oracle/_ref/libq4t_ref.so is used
// only by tests to pin the oracle's restatement bit-for-bit; it contains no
// code of this repository's product and is never shipped.
//
// Wrapped: include/q4t/quant/format.h (E2m1ToFloat, FloatToE2m1Code,
// E4m3ToFloat, FloatToE4m3) and include/q4t/quant/swizzle.h (SfOffset,
// SfNumGtiles, SfBufferSize, SwizzleSfInto).
#include <cstddef>
#include <cstdint>

#include "q4t/quant/format.h"
#include "q4t/quant/swizzle.h"

extern "C" {
float ref_e2m1_to_float(uint8_t c) { return q4t::quant::E2m1ToFloat(c); }
int ref_float_to_e2m1(float v) { return q4t::quant::FloatToE2m1Code(v); }
float ref_e4m3_to_float(uint8_t c) { return q4t::quant::E4m3ToFloat(c); }
uint8_t ref_float_to_e4m3(float v) { return q4t::quant::FloatToE4m3(v); }
size_t ref_sf_offset(int r, int g, int nt) { return q4t::quant::SfOffset(r, g, nt); }
int ref_sf_num_gtiles(int K) { return q4t::quant::SfNumGtiles(K); }
size_t ref_sf_buffer_size(int rows, int K) { return q4t::quant::SfBufferSize(rows, K); }
void ref_swizzle_sf(const uint8_t* rm, int rows, int K, uint8_t* out) {
  q4t::quant::SwizzleSfInto(rm, rows, K, out);
}
// Bulk forms so that a test can sweep many bit patterns per FFI call.
void ref_float_to_e4m3_bulk(const float* in, size_t n, uint8_t* out) {
  for (size_t i = 0; i < n; ++i) out[i] = q4t::quant::FloatToE4m3(in[i]);
}
void ref_float_to_e2m1_bulk(const float* in, size_t n, uint8_t* out) {
  for (size_t i = 0; i < n; ++i)
    out[i] = static_cast<uint8_t>(q4t::quant::FloatToE2m1Code(in[i]));
}
}
