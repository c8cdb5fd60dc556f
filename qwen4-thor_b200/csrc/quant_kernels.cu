// NVFP4 quantise / dequantise kernels: the standalone activation quantiser,
// the expert-grouped gather-quantiser that feeds the gate/up GEMM and the
// dequantiser.
#include "kernels.h"
#include "q4t_device.cuh"

namespace q4t {

namespace {

// One thread per group of 16 values; 4 neighbouring threads (the 4 groups of
// one scale atom column block) merge their scale bytes into one 32-bit store.
// ROWMAP: rows are gathered (source row = flat_of_row[r] / k, scale =
// input_scale[expert of r]) and scales go to tile-local atoms; otherwise plain
// row order, one global scale, scales in the standard swizzled buffer.
template <bool ROWMAP>
__global__ void __launch_bounds__(256) quantize_rows_kernel(
    const uint16_t* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_out,
    int rows, int K, float global_scale,
    // ROWMAP only:
    const int32_t* __restrict__ flat_of_row, const int32_t* __restrict__ expert_ids,
    const float* __restrict__ input_scale, const int32_t* __restrict__ row_tile,
    const int32_t* __restrict__ tile_row0, const int32_t* __restrict__ rows_dev, int k, int E) {
  chain_wait();
  const int groups = K >> 4;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  // grouped rows past the device-side count belong to skipped (token,slot) entries
  if (ROWMAP) rows = min(rows, *rows_dev);
  const int64_t total = static_cast<int64_t>(rows) * groups;
  // groups is a multiple of 4, so the 4 lanes of a quad share one row
  const bool live = idx < total;
  const int row = live ? static_cast<int>(idx / groups) : 0;
  const int g = live ? static_cast<int>(idx % groups) : 0;

  int src_row = row;
  float gs = global_scale;
  size_t sf_base = 0;
  uint32_t sf_row = row;
  if constexpr (ROWMAP) {
    if (live) {
      const int flat = flat_of_row[row];
      src_row = flat / k;
      const int e = expert_ids[flat];
      gs = input_scale[e];
      const int t = row_tile[row];
      sf_base = static_cast<size_t>(t) * (static_cast<size_t>((groups + 3) >> 2) * 512u);
      sf_row = static_cast<uint32_t>(row - tile_row0[t]);
    }
  }
  uint32_t sf = 0;
  if (live) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(src_row) * K + g * 16);
    const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float a[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a[2 * j] = bf16x2_lo(w[j]);
      a[2 * j + 1] = bf16x2_hi(w[j]);
    }
    uint32_t lo, hi;
    sf = quantize_group16(a, gs, lo, hi);
    *reinterpret_cast<uint2*>(packed + (static_cast<size_t>(row) * groups + g) * 8) = make_uint2(lo, hi);
  }
  if ((groups & 3) == 0) {
    // merge the quad's scale bytes: groups g..g+3 of one row, g % 4 == 0 at the leader
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t word = sf;
    word |= __shfl_down_sync(0xffffffffu, sf, 1) << 8;
    word |= __shfl_down_sync(0xffffffffu, sf, 2) << 16;
    word |= __shfl_down_sync(0xffffffffu, sf, 3) << 24;
    if (live && (lane & 3u) == 0) {
      size_t off;
      if constexpr (ROWMAP)
        off = sf_base + static_cast<size_t>(g >> 2) * 512u + sf_in_atom(sf_row, 0);
      else
        off = sf_offset(sf_row, g, groups >> 2);
      *reinterpret_cast<uint32_t*>(sf_out + off) = word;
    }
  } else if (live) {
    if constexpr (ROWMAP)
      sf_out[sf_base + static_cast<size_t>(g >> 2) * 512u + sf_in_atom(sf_row, g)] = sf;
    else
      sf_out[sf_offset(sf_row, g, (groups + 3) >> 2)] = sf;
  }
}

// Quantises token rows once and writes codes and scale bytes to several buffers (this
// GPU's and its peers' copies of a rank's token block).  One warp per row; a lane owns
// four neighbouring groups (64 values), so each destination receives the row as 32-byte
// code pieces and 4-byte scale pieces that the warp lays down contiguously: 1 KB of codes
// and 128 scale bytes (row-major, NOT swizzled) per 2048 values.  K a multiple of 64.
__global__ void __launch_bounds__(256) publish_tokens_kernel(const uint16_t* __restrict__ x,
                                                             const __grid_constant__ PublishTargets dst,
                                                             int rows, int K, float global_scale) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int groups = K >> 4;
  for (int g0 = lane * 4; g0 < groups; g0 += 128) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * K + g0 * 16);
    uint32_t codes[8], sfw = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 v0 = __ldg(src + 2 * j), v1 = __ldg(src + 2 * j + 1);
      const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      float a[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        a[2 * i] = bf16x2_lo(w[i]);
        a[2 * i + 1] = bf16x2_hi(w[i]);
      }
      sfw |= quantize_group16(a, global_scale, codes[2 * j], codes[2 * j + 1]) << (8 * j);
    }
    const size_t code_at = static_cast<size_t>(row) * (K >> 1) + static_cast<size_t>(g0) * 8;
    const size_t sf_at = static_cast<size_t>(row) * groups + g0;
    for (int d = 0; d < dst.n; ++d) {
      uint4* c = reinterpret_cast<uint4*>(dst.packed[d] + code_at);
      c[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
      c[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
      *reinterpret_cast<uint32_t*>(dst.sf[d] + sf_at) = sfw;
    }
  }
}

// The same, but a token travels only to the ranks that serve one of its selected experts
// (and always to its own rank).  dst.packed[r] / dst.sf[r] are indexed by RANK here.  The
// owner of expert e: map 0 -> e / (E/world), map 1 -> e % world, map 2 -> owner[e] (a rank,
// or negative for an expert replicated on every rank, which the token's own rank serves).
// One warp per token: lanes 0..k-1 look up the owners, the warp ORs them into a mask.
__global__ void __launch_bounds__(256) publish_selected_kernel(const uint16_t* __restrict__ x,
                                                               const int32_t* __restrict__ ids,
                                                               const __grid_constant__ PublishTargets dst,
                                                               int rows, int K, int k, int E, int map, int self,
                                                               const int32_t* __restrict__ owner,
                                                               float global_scale) {
  chain_wait();
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int world = dst.n;
  uint32_t mine = 0;
  if (lane < k) {
    const int e = ids[row * k + lane];
    if (e >= 0 && e < E) {
      int o;
      if (map == 2) o = owner[e];
      else if (map == 1) o = e % world;
      else o = e / (E / world);
      if (o >= 0 && o < world) mine = 1u << o;
    }
  }
  const uint32_t mask = __reduce_or_sync(0xffffffffu, mine) | (1u << self);
  const int groups = K >> 4;
  for (int g0 = lane * 4; g0 < groups; g0 += 128) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * K + g0 * 16);
    uint32_t codes[8], sfw = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 v0 = __ldg(src + 2 * j), v1 = __ldg(src + 2 * j + 1);
      const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      float a[16];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        a[2 * i] = bf16x2_lo(w[i]);
        a[2 * i + 1] = bf16x2_hi(w[i]);
      }
      sfw |= quantize_group16(a, global_scale, codes[2 * j], codes[2 * j + 1]) << (8 * j);
    }
    const size_t code_at = static_cast<size_t>(row) * (K >> 1) + static_cast<size_t>(g0) * 8;
    const size_t sf_at = static_cast<size_t>(row) * groups + g0;
    for (uint32_t m = mask; m != 0; m &= m - 1) {
      const int d = __ffs(m) - 1;
      uint4* c = reinterpret_cast<uint4*>(dst.packed[d] + code_at);
      c[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
      c[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
      *reinterpret_cast<uint32_t*>(dst.sf[d] + sf_at) = sfw;
    }
  }
}

// Quantises every token once (one input scale for all experts) and writes the codes and
// scale bytes straight to the token's k grouped rows.  One thread per group of 16 values, as
// in the plain quantiser (neighbouring lanes read and write neighbouring 32 / 8 bytes; four
// lanes merge their scale bytes into one word of the destination row's tile-local atom); the
// k destinations of the block's tokens are looked up once into shared memory.  Replaces
// "quantise the tokens, then copy each row k times" (half the memory traffic).
// K a multiple of 64 and at least 128, k <= 16.
constexpr int kScatterMaxTokens = 34;  // tokens one block of 256 groups can touch when K >= 128
__global__ void __launch_bounds__(256) quantize_scatter_kernel(
    const uint16_t* __restrict__ x, uint8_t* __restrict__ packed, uint8_t* __restrict__ sf_tiles, int T, int K,
    float global_scale, const int32_t* __restrict__ row_of_flat, const int32_t* __restrict__ row_tile,
    const int32_t* __restrict__ tile_row0, int k) {
  chain_wait();
  __shared__ int32_t s_row[kScatterMaxTokens * 16], s_tile[kScatterMaxTokens * 16], s_in[kScatterMaxTokens * 16];
  const int groups = K >> 4, ntk = K >> 6;
  const int64_t idx0 = static_cast<int64_t>(blockIdx.x) * 256, total = static_cast<int64_t>(T) * groups;
  const int tok0 = static_cast<int>(idx0 / groups);
  const int tok1 = static_cast<int>(min(total - 1, idx0 + 255) / groups);
  for (int j = threadIdx.x; j < (tok1 - tok0 + 1) * k; j += 256) {
    const int r = row_of_flat[(tok0 + j / k) * k + j % k];
    s_row[j] = r;
    if (r >= 0) {
      const int tile = row_tile[r];
      s_tile[j] = tile;
      s_in[j] = r - tile_row0[tile];
    }
  }
  __syncthreads();
  const int64_t idx = idx0 + threadIdx.x;
  const bool live = idx < total;
  const int token = live ? static_cast<int>(idx / groups) : tok0;
  const int g = live ? static_cast<int>(idx % groups) : 0;
  uint32_t lo = 0, hi = 0, sf = 0;
  if (live) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(token) * K + g * 16);
    const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float a[16];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      a[2 * j] = bf16x2_lo(w[j]);
      a[2 * j + 1] = bf16x2_hi(w[j]);
    }
    sf = quantize_group16(a, global_scale, lo, hi);
  }
  // groups is a multiple of 4, so the four lanes of a quad hold groups g..g+3 of one token
  uint32_t word = sf;
  word |= __shfl_down_sync(0xffffffffu, sf, 1) << 8;
  word |= __shfl_down_sync(0xffffffffu, sf, 2) << 16;
  word |= __shfl_down_sync(0xffffffffu, sf, 3) << 24;
  if (!live) return;
  const bool leader = (threadIdx.x & 3) == 0;
  const int base = (token - tok0) * k;
  for (int s = 0; s < k; ++s) {
    const int r = s_row[base + s];
    if (r < 0) continue;
    *reinterpret_cast<uint2*>(packed + static_cast<size_t>(r) * (K >> 1) + static_cast<size_t>(g) * 8) = make_uint2(lo, hi);
    if (leader)
      *reinterpret_cast<uint32_t*>(sf_tiles + (static_cast<size_t>(s_tile[base + s]) * ntk + (g >> 2)) * 512u +
                                   sf_in_atom(static_cast<uint32_t>(s_in[base + s]), 0)) = word;
  }
}

// One warp per grouped row: copies the row's token codes (quantised once per token by
// its owner rank) from the gathered token buffer of all ranks (token = flat / k over all
// ranks' tokens; scale bytes row-major [tokens, K/16]) and moves the scale bytes into the
// row tile's local atoms, four bytes (one K-tile of one row) at a time.
__global__ void __launch_bounds__(256) gather_codes_rowsf_kernel(
    const uint8_t* __restrict__ xq_packed, const uint8_t* __restrict__ xq_sf, uint8_t* __restrict__ packed,
    uint8_t* __restrict__ sf_tiles, int rows, int K, const int32_t* __restrict__ flat_of_row,
    const int32_t* __restrict__ row_tile, const int32_t* __restrict__ tile_row0,
    const int32_t* __restrict__ rows_dev, int k) {
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= min(rows, *rows_dev)) return;
  const int token = flat_of_row[r] / k;
  const int t = row_tile[r];
  const uint32_t in_tile = static_cast<uint32_t>(r - tile_row0[t]);
  const int row_bytes = K >> 1, ntk = K >> 6;
  const uint4* from = reinterpret_cast<const uint4*>(xq_packed + static_cast<size_t>(token) * row_bytes);
  const uint32_t* from_sf = reinterpret_cast<const uint32_t*>(xq_sf + static_cast<size_t>(token) * (K >> 4));
  uint4* dst = reinterpret_cast<uint4*>(packed + static_cast<size_t>(r) * row_bytes);
  for (int c = lane; c < (row_bytes >> 4); c += 32) dst[c] = __ldg(from + c);
  for (int a = lane; a < ntk; a += 32)
    *reinterpret_cast<uint32_t*>(sf_tiles + (static_cast<size_t>(t) * ntk + a) * 512u + sf_in_atom(in_tile, 0)) =
        __ldg(from_sf + a);
}

__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ packed,
                                                      const uint8_t* __restrict__ group_scale,
                                                      uint16_t* __restrict__ out, float inv_global,
                                                      int N, int K) {
  const int groups = K >> 4;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(N) * groups) return;
  const uint2 c = *reinterpret_cast<const uint2*>(packed + idx * 8);
  // reference order: decode(scale) * inv_global, then code * that, then bf16
  const float scale = e4m3_decode(group_scale[idx]) * inv_global;
  const uint32_t w[2] = {c.x, c.y};
  uint32_t o[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t b = (w[j >> 2] >> (8 * (j & 3))) & 0xffu;
    const uint32_t lo = b & 0xfu, hi = b >> 4;
    // e2m1 magnitude: 0,.5,1,1.5,2,3,4,6
    const float ml = (lo & 6u) ? __uint_as_float((((lo >> 1) & 3u) + 126u) << 23 | (lo & 1u) << 22)
                               : 0.5f * static_cast<float>(lo & 1u);
    const float mh = (hi & 6u) ? __uint_as_float((((hi >> 1) & 3u) + 126u) << 23 | (hi & 1u) << 22)
                               : 0.5f * static_cast<float>(hi & 1u);
    const float vl = ((lo & 8u) ? -ml : ml) * scale;
    const float vh = ((hi & 8u) ? -mh : mh) * scale;
    o[j] = f32x2_to_bf16x2(vl, vh);
  }
  uint4* dst = reinterpret_cast<uint4*>(out + idx * 16);
  dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
  dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
}

// Expert parallelism without collectives: CTA p copies this rank's id block into rank p's
// gathered id buffer (plain stores, possibly over NVLink), makes every earlier write of this
// GPU visible system-wide and then raises this rank's flag in rank p's flag row.  Launched
// after the kernels whose output the flag announces (stream order plus the fence).
__global__ void __launch_bounds__(1024) ep_post_kernel(const int32_t* __restrict__ ids, int n_ids,
                                                       const __grid_constant__ EpPostTargets dst, uint32_t epoch) {
  const int p = blockIdx.x;
  if (ids != nullptr) {
    int32_t* out = dst.ids[p];
    const int n4 = n_ids >> 2;
    const uint4* src4 = reinterpret_cast<const uint4*>(ids);
    uint4* out4 = reinterpret_cast<uint4*>(out);
    for (int i = threadIdx.x; i < n4; i += blockDim.x) out4[i] = src4[i];
    for (int i = (n4 << 2) + threadIdx.x; i < n_ids; i += blockDim.x) out[i] = ids[i];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst.flag[p]), "r"(epoch) : "memory");
  }
}

// Waits until every rank has raised its flag in this rank's flag row to `epoch` (or later).
// Bounded: after about two seconds the lane gives up and raises *status.
__global__ void __launch_bounds__(32) ep_wait_kernel(const uint32_t* flags, int world, uint32_t epoch,
                                                     int32_t* status) {
  const int lane = threadIdx.x;
  if (lane < world) {
    const uint32_t* f = flags + lane;
    const long long start = clock64();
    bool ok = false;
    for (uint32_t i = 0;; ++i) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) {
        ok = true;
        break;
      }
      if ((i & 63u) == 63u && clock64() - start > (1ll << 32)) break;
      __nanosleep(64);
    }
    if (!ok && status) atomicMax(status, 4);
  }
  __threadfence_system();
}

}  // namespace

cudaError_t launch_quantize(const uint16_t* x, uint8_t* packed, uint8_t* sf, int M, int K,
                            float global_scale, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(M) * (K / 16);
  if (total == 0) return cudaSuccess;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  const int32_t* no_table = nullptr;
  const float* no_scale = nullptr;
  return launch_chained(quantize_rows_kernel<false>, dim3(blocks), dim3(256), 0, stream, x, packed, sf, M, K,
                        global_scale, no_table, no_table, no_scale, no_table, no_table, no_table, 1, 0);
}

cudaError_t launch_gather_quantize(const uint16_t* x, uint8_t* packed, uint8_t* sf_tiles, int R,
                                   int K, const int32_t* flat_of_row, const int32_t* expert_ids,
                                   const float* input_scale, const int32_t* row_tile,
                                   const int32_t* tile_row0, const int32_t* rows_dev, int k, int E,
                                   cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(R) * (K / 16);
  if (total == 0) return cudaSuccess;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  return launch_chained(quantize_rows_kernel<true>, dim3(blocks), dim3(256), 0, stream, x, packed, sf_tiles, R, K,
                        0.0f, flat_of_row, expert_ids, input_scale, row_tile, tile_row0, rows_dev, k, E);
}

cudaError_t launch_quantize_scatter(const uint16_t* x, uint8_t* packed, uint8_t* sf_tiles, int T, int K,
                                    float global_scale, const int32_t* row_of_flat, const int32_t* row_tile,
                                    const int32_t* tile_row0, int k, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(T) * (K / 16);
  if (total == 0) return cudaSuccess;
  if (K < 128 || K % 64 || k > 16) return cudaErrorInvalidValue;
  return launch_chained(quantize_scatter_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream,
                        x, packed, sf_tiles, T, K, global_scale, row_of_flat, row_tile, tile_row0, k);
}

cudaError_t launch_gather_codes_rowsf(const uint8_t* xq_packed, const uint8_t* xq_sf, uint8_t* packed,
                                      uint8_t* sf_tiles, int R, int K, const int32_t* flat_of_row,
                                      const int32_t* row_tile, const int32_t* tile_row0, const int32_t* rows_dev,
                                      int k, cudaStream_t stream) {
  if (R == 0) return cudaSuccess;
  gather_codes_rowsf_kernel<<<(R + 7) / 8, 256, 0, stream>>>(xq_packed, xq_sf, packed, sf_tiles, R, K, flat_of_row,
                                                             row_tile, tile_row0, rows_dev, k);
  return cudaGetLastError();
}

cudaError_t launch_publish_tokens(const uint16_t* x, const PublishTargets& dst, int M, int K, float global_scale,
                                  cudaStream_t stream) {
  if (M == 0 || dst.n == 0) return cudaSuccess;
  publish_tokens_kernel<<<(M + 7) / 8, 256, 0, stream>>>(x, dst, M, K, global_scale);
  return cudaGetLastError();
}

cudaError_t launch_publish_selected(const uint16_t* x, const int32_t* ids, const PublishTargets& dst, int M, int K,
                                    int k, int E, int map, int self, const int32_t* owner, float global_scale,
                                    cudaStream_t stream) {
  if (M == 0 || dst.n == 0) return cudaSuccess;
  if (k > 32) return cudaErrorInvalidValue;
  return launch_chained(publish_selected_kernel, dim3((M + 7) / 8), dim3(256), 0, stream, x, ids, dst, M, K, k, E, map,
                        self, owner, global_scale);
}

cudaError_t launch_ep_post(const int32_t* ids, int n_ids, const EpPostTargets& dst, int world, uint32_t epoch,
                           cudaStream_t stream) {
  ep_post_kernel<<<world, 1024, 0, stream>>>(ids, n_ids, dst, epoch);
  return cudaGetLastError();
}

cudaError_t launch_ep_wait(const uint32_t* flags, int world, uint32_t epoch, int32_t* status, cudaStream_t stream) {
  ep_wait_kernel<<<1, 32, 0, stream>>>(flags, world, epoch, status);
  return cudaGetLastError();
}

cudaError_t launch_dequant(const uint8_t* packed, const uint8_t* group_scale, uint16_t* out,
                           float inv_global, int N, int K, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(N) * (K / 16);
  if (total == 0) return cudaSuccess;
  dequant_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(
      packed, group_scale, out, inv_global, N, K);
  return cudaGetLastError();
}

}  // namespace q4t
