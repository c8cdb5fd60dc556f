// Scale-factor atom layout helpers with the reference's names
// (include/q4t/quant/swizzle.h:34-83), forwarded to the C ABI.
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

#include "q4t_moe_b200.h"

namespace q4t::quant {
inline std::size_t SfOffset(int row, int group, int num_g_tiles) { return q4t_sf_offset(row, group, num_g_tiles); }
inline int SfNumGtiles(int K) { return q4t_sf_num_gtiles(K); }
inline std::size_t SfBufferSize(int rows, int K) { return q4t_sf_buffer_size(rows, K); }
inline void SwizzleSfInto(const uint8_t* row_major, int rows, int K, uint8_t* out) {
  const int groups = K / 16, nt = SfNumGtiles(K);
  const std::size_t n = SfBufferSize(rows, K);
  for (std::size_t i = 0; i < n; ++i) out[i] = 0;
  for (int r = 0; r < rows; ++r)
    for (int g = 0; g < groups; ++g) out[SfOffset(r, g, nt)] = row_major[static_cast<std::size_t>(r) * groups + g];
}
inline std::vector<uint8_t> SwizzleSf(const uint8_t* row_major, int rows, int K) {
  std::vector<uint8_t> out(SfBufferSize(rows, K));
  SwizzleSfInto(row_major, rows, K, out.data());
  return out;
}
}  // namespace q4t::quant
