// Router, token->expert permutation, SwiGLU and combine kernels.
#include <cstdlib>

#include "kernels.h"
#include "q4t_device.cuh"

namespace q4t {

namespace {

// y[m, n] = bf16(x[m,:] . w[n,:]) for M <= 8 with the accumulation order of
// the reference's warp-per-output GEMV (src/model/gemv.cu:56-119 and the
// small-M kernel it is documented bit-identical to, src/model/small_m_gemm.cu:
// 57-113): lane l owns the 8-element chunks l, l+32, ...; inside a chunk even
// elements feed one accumulator and odd elements another by fused multiply-
// add; the two are added; lanes fold by shuffle-down 16..1; bf16 round.
template <int MAXM>
__global__ void __launch_bounds__(256) small_m_linear_kernel(const uint16_t* __restrict__ x,
                                                             const uint16_t* __restrict__ w,
                                                             uint16_t* __restrict__ y, int M, int N,
                                                             int K) {
  extern __shared__ __align__(16) uint16_t s_x[];  // [M, K], loaded once per block
  const int k8 = K >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  const uint4* wrow = reinterpret_cast<const uint4*>(w + static_cast<size_t>(n < N ? n : 0) * K);
  // The weights do not come from the kernel before this one: the first eight chunks of the
  // row (all of it up to K = 2048) are requested before the wait and the staging of x.
  uint4 wv[8];
#pragma unroll
  for (int u = 0; u < 8; ++u)
    if (n < N && lane + 32 * u < k8) wv[u] = __ldg(wrow + lane + 32 * u);
  chain_wait();
  for (int i = threadIdx.x; i < M * k8; i += 256)
    reinterpret_cast<uint4*>(s_x)[i] = __ldg(reinterpret_cast<const uint4*>(x) + i);
  __syncthreads();
  if (n >= N) return;
  float ax[MAXM], ay[MAXM];
#pragma unroll
  for (int m = 0; m < MAXM; ++m) ax[m] = ay[m] = 0.0f;
  // chunks lane, lane+32, ... in order; the weight loads of eight chunks are
  // issued together so that their latencies overlap
  for (int i0 = lane; i0 < k8; i0 += 32 * 8) {
    if (i0 != lane) {
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (i0 + 32 * u < k8) wv[u] = __ldg(wrow + i0 + 32 * u);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + 32 * u;
      if (i < k8) {
        const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
#pragma unroll
        for (int m = 0; m < MAXM; ++m) {
          if (m < M) {
            const uint4 xv = reinterpret_cast<const uint4*>(s_x + static_cast<size_t>(m) * K)[i];
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              ax[m] = fmaf(bf16x2_lo(xw[j]), bf16x2_lo(ww[j]), ax[m]);
              ay[m] = fmaf(bf16x2_hi(xw[j]), bf16x2_hi(ww[j]), ay[m]);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MAXM; ++m) {
    if (m < M) {
      float s = ax[m] + ay[m];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) s += __shfl_down_sync(0xffffffffu, s, off);
      if (lane == 0) y[static_cast<size_t>(m) * N + n] = f32_to_bf16(1.0f * s);
    }
  }
}

// Top-k + softmax over the selected logits, one warp per token
// (RouterTopkKernel, src/model/moe.cu:134-212): k rounds of arg-max by
// (value desc, id asc) with the winner masked to -1e30; then, in selection
// order, e_i = __expf(v_i - max), sum, w_i = e_i * (1/sum).
__device__ __forceinline__ void topk_token(const uint16_t* __restrict__ row, const int32_t* __restrict__ fixed,
                                           int32_t* ids_out, float* rw_out, int E, int k, int lane) {
  float sel_v = 0.0f;  // lane i < k keeps the i-th selected value
  int sel_i = 0;
  if (fixed != nullptr) {
    if (lane < k) {
      sel_i = fixed[lane];
      sel_v = bf16_to_f32(row[sel_i]);
    }
  } else {
    // Order-preserving 32-bit keys: high half = the bf16 logit mapped to an
    // unsigned order (-0.0 folded into +0.0, which compare equal as floats),
    // low half = 0xFFFF - expert id, so that the maximum key is the largest
    // value and, among equal values, the lowest id.  A selected entry's key
    // becomes 0.  One warp-wide integer max (redux) per round.
    // Register slot i of lane l holds expert (i / 8) * 256 + 8 * l + i % 8: two 16-byte
    // loads per lane when the row is 16-byte aligned (E a multiple of 8), the ids travel
    // inside the keys, so the placement does not matter for the result.
    uint32_t key[16];
    uint32_t lmax = 0;
    const bool vec = (E & 7) == 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int e0 = h * 256 + 8 * lane;
      uint32_t w[4] = {0, 0, 0, 0};
      if (vec && e0 < E) {
        const uint4 v = *reinterpret_cast<const uint4*>(row + e0);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int e = e0 + j;
        uint32_t kv = 0;
        if (e < E) {
          uint32_t b = vec ? ((w[j >> 1] >> (16 * (j & 1))) & 0xffffu) : row[e];
          if (b == 0x8000u) b = 0;
          const uint32_t ord = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
          kv = (ord << 16) | (0xffffu - static_cast<uint32_t>(e));
        }
        key[h * 8 + j] = kv;
        lmax = max(lmax, kv);
      }
    }
    for (int r = 0; r < k; ++r) {
      const uint32_t best = __reduce_max_sync(0xffffffffu, lmax);
      const int mid = static_cast<int>(0xffffu - (best & 0xffffu));
      if (lane == r) {
        const uint32_t ord = best >> 16;
        const uint32_t b = (ord & 0x8000u) ? (ord & 0x7fffu) : (~ord & 0xffffu);
        sel_v = bf16_to_f32(static_cast<uint16_t>(b));
        sel_i = mid;
      }
      if (((mid & 255) >> 3) == lane) {  // the owner drops the winner and refreshes its local maximum
        const int slot = ((mid >> 8) << 3) | (mid & 7);
        lmax = 0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          if (i == slot) key[i] = 0;
          lmax = max(lmax, key[i]);
        }
      }
    }
  }
  // softmax in selection order, evaluated redundantly by every lane
  float mx = __shfl_sync(0xffffffffu, sel_v, 0);
  for (int i = 1; i < k; ++i) mx = fmaxf(mx, __shfl_sync(0xffffffffu, sel_v, i));
  const float ev = __expf(sel_v - mx);
  float sum = 0.0f;
  for (int i = 0; i < k; ++i) sum += __shfl_sync(0xffffffffu, ev, i);
  const float inv = __frcp_rn(sum);  // == 1.0f / sum under IEEE division
  if (lane < k) {
    ids_out[lane] = sel_i;
    rw_out[lane] = ev * inv;
  }
}

__global__ void __launch_bounds__(256) topk_kernel(const uint16_t* __restrict__ logits,
                                                   const int32_t* __restrict__ fixed_ids,
                                                   int32_t* __restrict__ ids, float* __restrict__ rw,
                                                   int T, int E, int k) {
  chain_wait();
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  topk_token(logits + static_cast<size_t>(t) * E, fixed_ids ? fixed_ids + static_cast<size_t>(t) * k : nullptr,
             ids + static_cast<size_t>(t) * k, rw + static_cast<size_t>(t) * k, E, k, lane);
}

// ---- permutation: stable counting sort of the (token,slot) entries by expert.
__global__ void __launch_bounds__(256) plan_hist_kernel(const int32_t* __restrict__ ids, int R, int E,
                                                        int32_t* __restrict__ blk_counts) {
  chain_wait();
  extern __shared__ int32_t hist[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0;
  __syncthreads();
  const int base = blockIdx.x * kPlanChunk;
  for (int i = threadIdx.x; i < kPlanChunk; i += blockDim.x) {
    const int f = base + i;
    if (f < R) {
      const int e = ids[f];
      if (e >= 0 && e < E) atomicAdd(&hist[e], 1);
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) blk_counts[static_cast<size_t>(blockIdx.x) * E + e] = hist[e];
}

// Inclusive scan of two values over the 1024 threads of a block (thread e holds element e):
// shuffles inside each warp, one shared-memory step across the 32 warps.  Results land in
// s_a[e] / s_b[e]; s_a[1023] / s_b[1023] are the totals.  Two barriers instead of twenty.
__device__ __forceinline__ void block_scan_pair(int32_t a, int32_t b, int32_t* s_a, int32_t* s_b) {
  __shared__ int32_t w_a[32], w_b[32];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int32_t ua = __shfl_up_sync(0xffffffffu, a, off), ub = __shfl_up_sync(0xffffffffu, b, off);
    if (lane >= off) {
      a += ua;
      b += ub;
    }
  }
  if (lane == 31) {
    w_a[warp] = a;
    w_b[warp] = b;
  }
  __syncthreads();
  if (warp == 0) {
    int32_t ta = w_a[lane], tb = w_b[lane];
    const int32_t own_a = ta, own_b = tb;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int32_t ua = __shfl_up_sync(0xffffffffu, ta, off), ub = __shfl_up_sync(0xffffffffu, tb, off);
      if (lane >= off) {
        ta += ua;
        tb += ub;
      }
    }
    w_a[lane] = ta - own_a;  // what the warps before this one add up to
    w_b[lane] = tb - own_b;
  }
  __syncthreads();
  s_a[e] = a + w_a[warp];
  s_b[e] = b + w_b[warp];
  __syncthreads();
}

// One block of 1024 threads, E <= 1024.  Turns the per-block counts into
// per-block bases, builds offsets[E+1], the row-tile list and its count.
// even_tiles: an expert with rows gets an even number of row tiles; the extra one is empty
// (zero rows, first row just past the expert's last).
__global__ void __launch_bounds__(1024) plan_scan_kernel(int nblk, int E, int max_tiles, PlanTables p,
                                                         int even_tiles) {
  chain_wait();
  __shared__ int32_t s_rows[1024];
  __shared__ int32_t s_tiles[1024];
  const int e = threadIdx.x;
  int32_t c = 0;
  if (e < E) {
    // sixteen blocks at a time: the loads of a chunk are independent, so the chain is
    // one memory round trip per chunk instead of one per block
    int32_t* col = p.blk_counts + e;
    for (int b0 = 0; b0 < nblk; b0 += 16) {
      int32_t v[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = b0 + i < nblk ? col[static_cast<size_t>(b0 + i) * E] : 0;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        if (b0 + i < nblk) col[static_cast<size_t>(b0 + i) * E] = c;
        c += v[i];
      }
    }
    p.counts[e] = c;
  }
  int32_t tiles = (c + kTileM - 1) / kTileM;
  if (even_tiles) tiles = (tiles + 1) & ~1;
  block_scan_pair(c, tiles, s_rows, s_tiles);  // inclusive scans of rows and row tiles over the experts
  const int32_t row_base = s_rows[e] - c, tile_base = s_tiles[e] - tiles;
  const int32_t total_rows = s_rows[1023], total_tiles = s_tiles[1023];
  __syncthreads();
  s_rows[e] = row_base;   // from here on: first grouped row / first row tile of expert e
  s_tiles[e] = tile_base;
  __syncthreads();
  if (e < E) {
    p.offsets[e] = row_base;
    p.tile_off[e] = tile_base;
  }
  if (e == 0) {
    p.offsets[E] = total_rows;
    p.tile_off[E] = total_tiles;
    p.ntiles[0] = min(total_tiles, max_tiles);
  }
  if (e < 4 && p.status) p.status[e] = 0;
  // The tile list, all threads together (a popular expert owns hundreds of tiles): tile t
  // belongs to the last expert whose first tile is <= t (experts without rows share their
  // successor's first tile and come before it).
  for (int t = e; t < min(total_tiles, max_tiles); t += 1024) {
    int lo = 0, hi = E - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (s_tiles[mid] <= t) lo = mid; else hi = mid - 1;
    }
    const int i = t - s_tiles[lo];
    const int32_t rows_e = (lo + 1 < E ? s_rows[lo + 1] : total_rows) - s_rows[lo];
    p.tile_expert[t] = lo;
    p.tile_row0[t] = s_rows[lo] + i * kTileM;
    p.tile_nrows[t] = max(0, min(kTileM, rows_e - i * kTileM));
  }
}

__global__ void __launch_bounds__(256) plan_scatter_kernel(const int32_t* __restrict__ ids, int R, int E,
                                                           PlanTables p) {
  chain_wait();
  // Each of the 8 warps owns 256 consecutive entries of the block's chunk.  A first pass
  // counts every warp's entries per expert, a scan over the warps turns the counts into
  // each warp's first position, and a second pass places the entries; positions follow the
  // flat order without the warps having to take turns.
  extern __shared__ int32_t sm[];
  int32_t* first_row = sm;             // [E] first grouped row of the expert
  int32_t* first_tile = sm + E;        // [E] its first row tile
  uint16_t* wcnt = reinterpret_cast<uint16_t*>(sm + 2 * E);  // [8][E] per-warp counts, then cursors
  int32_t* wbase = sm + 2 * E + 4 * E;  // [E] block's first grouped row of the expert
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    const int32_t o = p.offsets[e];
    first_row[e] = o;
    first_tile[e] = p.tile_off[e];
    wbase[e] = o + p.blk_counts[static_cast<size_t>(blockIdx.x) * E + e];
  }
  for (int i = threadIdx.x; i < 8 * E; i += blockDim.x) wcnt[i] = 0;
  __syncthreads();
  constexpr int kSeg = kPlanChunk / 8;
  const int f0 = blockIdx.x * kPlanChunk + warp * kSeg;
  uint16_t* mine = wcnt + warp * E;
  int vals[kSeg / 32];
#pragma unroll
  for (int it = 0; it < kSeg / 32; ++it) {
    const int f = f0 + it * 32 + lane;
    const int v = f < R ? ids[f] : -1;
    vals[it] = v;
    const bool valid = v >= 0 && v < E;
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? v : -1 - lane);
    if (valid && __popc(peers & ((1u << lane) - 1u)) == 0) mine[v] += static_cast<uint16_t>(__popc(peers));
    __syncwarp();
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {  // exclusive scan over the warps
    uint32_t c = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const uint32_t v = wcnt[w * E + e];
      wcnt[w * E + e] = static_cast<uint16_t>(c);
      c += v;
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < kSeg / 32; ++it) {
    const int f = f0 + it * 32 + lane;
    const int v = vals[it];
    const bool valid = v >= 0 && v < E;
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? v : -1 - lane);
    if (valid) {
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int row = wbase[v] + mine[v] + rank;
      __syncwarp(peers);
      if (rank == 0) mine[v] += static_cast<uint16_t>(__popc(peers));
      p.row_of_flat[f] = row;
      p.flat_of_row[row] = f;
      p.row_tile[row] = first_tile[v] + (row - first_row[v]) / kTileM;
    } else if (f < R) {
      p.row_of_flat[f] = -1;
    }
    __syncwarp();
  }
}

// Whole permutation in one block for small batches (R <= kPlanSmallMax): the
// 32 warps each own a contiguous segment of the (token,slot) entries.  Per-warp
// expert counts, a per-expert scan over the warps, the block scan that yields
// offsets and the row-tile list, then every warp places its own entries in
// order using its private cursors, so the result is the stable order.
constexpr int kPlanSmallMax = 4096;
// With ROUTE the same block first selects the experts of every token (top-k and
// softmax, one warp per token) and then plans from the ids it just wrote.
template <bool ROUTE>
__global__ void __launch_bounds__(1024) plan_small_kernel(const int32_t* ids, int R, int E, int max_tiles,
                                                          PlanTables p, const uint16_t* __restrict__ logits,
                                                          const int32_t* __restrict__ fixed_ids, int32_t* ids_out,
                                                          float* rw_out, int T, int k, int E_logits,
                                                          int even_tiles) {
  chain_wait();
  extern __shared__ uint16_t s_cnt[];  // [32][E]: counts, later exclusive bases, then cursors
  __shared__ int32_t s_rows[1024];
  __shared__ int32_t s_tiles[1024];
  const int e = threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if constexpr (ROUTE) {
    for (int t = warp; t < T; t += 32)
      topk_token(logits + static_cast<size_t>(t) * E_logits,
                 fixed_ids ? fixed_ids + static_cast<size_t>(t) * k : nullptr,
                 ids_out + static_cast<size_t>(t) * k, rw_out + static_cast<size_t>(t) * k, E_logits, k, lane);
    __threadfence_block();  // the ids are read back below by other warps
    ids = ids_out;
  }
  for (int i = threadIdx.x; i < 32 * E; i += 1024) s_cnt[i] = 0;
  __syncthreads();
  const int seg = (R + 31) / 32;
  const int f0 = warp * seg, f1 = min(R, f0 + seg);
  uint16_t* mine = s_cnt + warp * E;
  for (int fb = f0; fb < f1; fb += 32) {
    const int f = fb + lane;
    const int v = f < f1 ? ids[f] : -1;
    const bool valid = v >= 0 && v < E;
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? v : -1 - lane);
    if (valid && __popc(peers & ((1u << lane) - 1u)) == 0) mine[v] += static_cast<uint16_t>(__popc(peers));
    __syncwarp();
  }
  __syncthreads();
  int32_t c = 0;
  if (e < E) {
    for (int w = 0; w < 32; ++w) {
      const int32_t v = s_cnt[w * E + e];
      s_cnt[w * E + e] = static_cast<uint16_t>(c);
      c += v;
    }
  }
  int32_t tiles = (c + kTileM - 1) / kTileM;
  if (even_tiles) tiles = (tiles + 1) & ~1;
  block_scan_pair(c, tiles, s_rows, s_tiles);  // inclusive scans of rows and row tiles over the experts
  const int32_t row_base = s_rows[e] - c, tile_base = s_tiles[e] - tiles;
  const int32_t total_rows = s_rows[1023], total_tiles = s_tiles[1023];
  __syncthreads();
  s_rows[e] = row_base;   // from here on: first grouped row / first row tile of expert e
  s_tiles[e] = tile_base;
  if (e < E) {
    p.counts[e] = c;
    p.offsets[e] = row_base;
    p.tile_off[e] = tile_base;
    for (int i = 0; i < tiles; ++i) {
      const int t = tile_base + i;
      if (t < max_tiles) {
        p.tile_expert[t] = e;
        p.tile_row0[t] = row_base + i * kTileM;
        p.tile_nrows[t] = max(0, min(kTileM, c - i * kTileM));
      }
    }
  }
  if (e == 0) {
    p.offsets[E] = total_rows;
    p.tile_off[E] = total_tiles;
    p.ntiles[0] = min(total_tiles, max_tiles);
  }
  if (e < 4 && p.status) p.status[e] = 0;
  __syncthreads();
  for (int fb = f0; fb < f1; fb += 32) {
    const int f = fb + lane;
    const int v = f < f1 ? ids[f] : -1;
    const bool valid = v >= 0 && v < E;
    const uint32_t peers = __match_any_sync(0xffffffffu, valid ? v : -1 - lane);
    if (valid) {
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int in_expert = mine[v] + rank;
      const int row = s_rows[v] + in_expert;
      __syncwarp(peers);
      if (rank == 0) mine[v] += static_cast<uint16_t>(__popc(peers));
      p.row_of_flat[f] = row;
      p.flat_of_row[row] = f;
      p.row_tile[row] = s_tiles[v] + in_expert / kTileM;
    } else if (f < f1) {
      p.row_of_flat[f] = -1;
    }
    __syncwarp();
  }
}

// Top-k and the permutation tables for 17..256 tokens in one launch: a cluster of eight CTAs.
// CTA c of the cluster owns the tokens [c*tpc, (c+1)*tpc), tpc = ceil(T/8) <= 32: one warp per
// token selects the experts (as topk_kernel), one thread per (token,slot) entry ranks it among
// the CTA's entries of the same expert, and the CTAs read each other's per-expert counts
// through distributed shared memory, so that every CTA knows where its entries start inside
// each expert's rows.  The stable order (expert ascending, then (token,slot) ascending) falls
// out of the CTA order.  All eight CTAs scan the same totals; CTA 0 writes the tables that do
// not belong to entries.  No global counters, no second launch.
constexpr int kRouteClusterCtas = 8;
__device__ __forceinline__ int32_t ld_cluster_s32(uint32_t cluster_addr) {
  int32_t v;
  asm volatile("ld.shared::cluster.s32 %0, [%1];" : "=r"(v) : "r"(cluster_addr) : "memory");
  return v;
}
__global__ void __launch_bounds__(1024) route_plan_cluster_kernel(const uint16_t* __restrict__ logits,
                                                                  const int32_t* __restrict__ fixed_ids,
                                                                  int32_t* ids_out, float* rw_out, int T, int k, int E,
                                                                  int max_tiles, PlanTables p, int even_tiles) {
  chain_wait();
  extern __shared__ uint16_t s_wcnt[];  // [16][E]: entries per (warp of entries, expert), then exclusive bases
  __shared__ int32_t s_own[1024];       // this CTA's entries per expert; later: entries of earlier CTAs
  __shared__ int32_t s_rows[1024];
  __shared__ int32_t s_tiles[1024];
  const int e = threadIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rank = static_cast<int>(cluster_cta_rank());
  const int tpc = (T + kRouteClusterCtas - 1) / kRouteClusterCtas;
  const int t0 = min(T, rank * tpc);
  const int n_tok = min(T - t0, tpc);
  const int f0 = t0 * k, n_ent = n_tok * k;    // this CTA's (token,slot) entries: [f0, f0 + n_ent), at most 512
  const int n_ew = (n_ent + 31) >> 5;          // warps of entries
  if (warp < n_tok)
    topk_token(logits + static_cast<size_t>(t0 + warp) * E,
               fixed_ids ? fixed_ids + static_cast<size_t>(t0 + warp) * k : nullptr,
               ids_out + static_cast<size_t>(t0 + warp) * k, rw_out + static_cast<size_t>(t0 + warp) * k, E, k, lane);
  for (int i = threadIdx.x; i < n_ew * E; i += 1024) s_wcnt[i] = 0;
  __threadfence_block();  // the ids are read back below by other warps
  __syncthreads();
  // thread i owns entry f0 + i
  const bool have = e < n_ent;
  const int v = have ? ids_out[f0 + e] : -1;
  const bool valid = v >= 0 && v < E;
  uint32_t peers = 0;
  if (warp < n_ew) {
    peers = __match_any_sync(0xffffffffu, valid ? v : -1 - lane);
    if (valid && __popc(peers & ((1u << lane) - 1u)) == 0) s_wcnt[warp * E + v] = static_cast<uint16_t>(__popc(peers));
  }
  __syncthreads();
  int32_t own = 0;
  if (e < E) {
    for (int w = 0; w < n_ew; ++w) {
      const int32_t c = s_wcnt[w * E + e];
      s_wcnt[w * E + e] = static_cast<uint16_t>(own);
      own += c;
    }
  }
  s_own[e] = own;
  cluster_sync();  // every CTA's counts are in its shared memory
  int32_t c = 0, before = 0;
  if (e < E) {
    const uint32_t mine = smem_u32(&s_own[e]);
#pragma unroll
    for (int r = 0; r < kRouteClusterCtas; ++r) {
      const int32_t o = ld_cluster_s32(cluster_map(mine, static_cast<uint32_t>(r)));
      c += o;
      if (r < rank) before += o;
    }
  }
  cluster_sync();  // no CTA reads another's shared memory after this point
  int32_t tiles = (c + kTileM - 1) / kTileM;
  if (even_tiles) tiles = (tiles + 1) & ~1;
  block_scan_pair(c, tiles, s_rows, s_tiles);  // inclusive scans of rows and row tiles over the experts
  const int32_t row_base = s_rows[e] - c, tile_base = s_tiles[e] - tiles;
  const int32_t total_rows = s_rows[1023], total_tiles = s_tiles[1023];
  __syncthreads();
  s_rows[e] = row_base;   // from here on: first grouped row / first row tile of expert e
  s_tiles[e] = tile_base;
  s_own[e] = before;      // entries of expert e that belong to earlier CTAs
  if (rank == 0) {
    if (e < E) {
      p.counts[e] = c;
      p.offsets[e] = row_base;
      p.tile_off[e] = tile_base;
      for (int i = 0; i < tiles; ++i) {
        const int t = tile_base + i;
        if (t < max_tiles) {
          p.tile_expert[t] = e;
          p.tile_row0[t] = row_base + i * kTileM;
          p.tile_nrows[t] = max(0, min(kTileM, c - i * kTileM));
        }
      }
    }
    if (e == 0) {
      p.offsets[E] = total_rows;
      p.tile_off[E] = total_tiles;
      p.ntiles[0] = min(total_tiles, max_tiles);
    }
    if (e < 4 && p.status) p.status[e] = 0;
  }
  __syncthreads();
  if (have) {
    const int f = f0 + e;
    if (valid) {
      const int in_expert = s_own[v] + s_wcnt[warp * E + v] + __popc(peers & ((1u << lane) - 1u));
      const int row = s_rows[v] + in_expert;
      p.row_of_flat[f] = row;
      p.flat_of_row[row] = f;
      p.row_tile[row] = s_tiles[v] + in_expert / kTileM;
    } else {
      p.row_of_flat[f] = -1;
    }
  }
}

// ---- expert-parallel helpers
// dest[f] = owner rank of expert ids[f] (experts are split into contiguous
// blocks of experts_per_rank); local[f] = index of that expert on its owner.
// Ids outside [0, E) map to -1 and are skipped by the planner.
__global__ void __launch_bounds__(256) ep_split_ids_kernel(const int32_t* __restrict__ ids, int R, int E,
                                                           int experts_per_rank, int32_t* __restrict__ dest,
                                                           int32_t* __restrict__ local) {
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= R) return;
  const int e = ids[f];
  const bool ok = e >= 0 && e < E;
  dest[f] = ok ? e / experts_per_rank : -1;
  local[f] = ok ? e % experts_per_rank : -1;
}

__global__ void __launch_bounds__(256) ep_localise_ids_kernel(const int32_t* __restrict__ ids, int R, int E,
                                                              int world, int rank, int map,
                                                              const int32_t* __restrict__ placement,
                                                              int flats_per_rank, int32_t* __restrict__ local) {
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= R) return;
  const int e = ids[f];
  int out = -1;
  if (e >= 0 && e < E) {
    if (map == 2) {
      const int v = placement[e];
      if (v >= 0) {
        const int idx = v & ~(1 << 30);
        // a replicated expert serves only the tokens that live on this rank
        out = (v & (1 << 30)) ? (f / flats_per_rank == rank ? idx : -1) : idx;
      }
    } else {
      const int per = E / world;
      const int owner = map == 1 ? e % world : e / per;
      if (owner == rank) out = map == 1 ? e / world : e - owner * per;
    }
  }
  local[f] = out;
}

// Slot mode: out[f] = slot_of_expert[ids[f]] when the id is a valid expert and the slot a
// valid resident slot, else -1 (the planner skips negative ids).
__global__ void __launch_bounds__(256) remap_ids_kernel(const int32_t* __restrict__ ids,
                                                        const int32_t* __restrict__ slot_of_expert,
                                                        int32_t* __restrict__ out, int R, int E, int slots) {
  chain_wait();
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= R) return;
  const int e = ids[f];
  int v = -1;
  if (e >= 0 && e < E) {
    v = slot_of_expert[e];
    if (v < 0 || v >= slots) v = -1;
  }
  out[f] = v;
}

__global__ void __launch_bounds__(256) ep_flat_rows_kernel(const int32_t* __restrict__ ids, int R, int E,
                                                           int32_t* __restrict__ row_of_flat) {
  const int f = blockIdx.x * blockDim.x + threadIdx.x;
  if (f >= R) return;
  const int e = ids[f];
  row_of_flat[f] = (e >= 0 && e < E) ? f : -1;
}

// out[r, :] = src[index[r] / div, :] for r < *rows_dev (rows of `width` bf16
// values, 16-byte vector copies); optionally aux_out[r] = aux[index[r]].
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint16_t* __restrict__ src,
                                                          const int32_t* __restrict__ index, int div,
                                                          const int32_t* __restrict__ rows_dev, int rows,
                                                          int width, uint16_t* __restrict__ out,
                                                          const int32_t* __restrict__ aux,
                                                          int32_t* __restrict__ aux_out) {
  const int per_row = width >> 3;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (rows_dev) rows = min(rows, *rows_dev);
  if (idx >= static_cast<int64_t>(rows) * per_row) return;
  const int r = static_cast<int>(idx / per_row), c = static_cast<int>(idx % per_row);
  const int i = index[r];
  if (i < 0) return;
  reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * width)[c] =
      __ldg(reinterpret_cast<const uint4*>(src + static_cast<size_t>(i / div) * width) + c);
  if (aux_out && c == 0) aux_out[r] = aux[i];
}

// y[t, c] += sum over slots, in slot order, of w * bf16 row value, accumulated
// by fused multiply-add from 0 (CombineGroupedKernel, src/quant/moe_gemm.cu:
// 273-288).  One thread per 8 columns.
__global__ void __launch_bounds__(256) routed_combine_kernel(const uint16_t* __restrict__ dn_out,
                                                             const int32_t* __restrict__ row_of_flat,
                                                             const float* __restrict__ rw,
                                                             float* __restrict__ y, int T, int k, int hs) {
  chain_wait();
  const int per_row = hs >> 3;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(T) * per_row) return;
  const int t = static_cast<int>(idx / per_row), c8 = static_cast<int>(idx % per_row);
  float acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
  for (int s = 0; s < k; ++s) {
    const int r = row_of_flat[t * k + s];
    if (r < 0) continue;
    const float wgt = rw[t * k + s];
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(dn_out + static_cast<size_t>(r) * hs) + c8);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[2 * j] = fmaf(wgt, bf16x2_lo(w[j]), acc[2 * j]);
      acc[2 * j + 1] = fmaf(wgt, bf16x2_hi(w[j]), acc[2 * j + 1]);
    }
  }
  float4* dst = reinterpret_cast<float4*>(y + static_cast<size_t>(t) * hs) + c8 * 2;
  float4 a = dst[0], b = dst[1];
  a.x += acc[0]; a.y += acc[1]; a.z += acc[2]; a.w += acc[3];
  b.x += acc[4]; b.y += acc[5]; b.z += acc[6]; b.w += acc[7];
  dst[0] = a;
  dst[1] = b;
}

// out[t, c] = bf16((g * sigmoid(g)) * u) (SwiGLUKernel, src/model/moe.cu:276-287).
__global__ void __launch_bounds__(256) swiglu_kernel(const uint16_t* __restrict__ gu,
                                                     uint16_t* __restrict__ out, int T, int inner) {
  chain_wait();
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(T) * inner) return;
  const int t = static_cast<int>(idx / inner), c = static_cast<int>(idx % inner);
  const float g = bf16_to_f32(gu[static_cast<size_t>(t) * 2 * inner + c]);
  const float u = bf16_to_f32(gu[static_cast<size_t>(t) * 2 * inner + inner + c]);
  const float sig = __frcp_rn(1.0f + __expf(-g));
  out[idx] = f32_to_bf16((g * sig) * u);
}

// The step between two layers of a decode stack: x <- bf16(x + y) (y may be null), then
// h <- x * rsqrt(mean(x^2) + eps) in bf16.  One warp per row, the summation order of
// GroupedRmsNormKernel (src/model/hyperconnection.cu:55-110): lane l sums the squares of the
// 8-element groups l, l+32, ... (eight fused multiply-adds per group, one add per group),
// xor butterfly over the lanes; the reciprocal square root is the correctly rounded one
// (the reference's rsqrtf is within 2 ulp of it).  hs a multiple of 8.
__global__ void __launch_bounds__(256) residual_rmsnorm_kernel(uint16_t* __restrict__ x,
                                                               const uint16_t* __restrict__ y,
                                                               uint16_t* __restrict__ h, int T, int hs, float eps) {
  chain_wait();
  const int t = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (t >= T) return;
  const int n8 = hs >> 3;
  uint4* xr = reinterpret_cast<uint4*>(x + static_cast<size_t>(t) * hs);
  const uint4* yr = y ? reinterpret_cast<const uint4*>(y + static_cast<size_t>(t) * hs) : nullptr;
  uint4* hr = reinterpret_cast<uint4*>(h + static_cast<size_t>(t) * hs);
  float acc = 0.0f;
  for (int i = lane; i < n8; i += 32) {
    uint4 v = xr[i];
    if (yr) {
      const uint4 w = yr[i];
      const uint32_t a[4] = {v.x, v.y, v.z, v.w}, b[4] = {w.x, w.y, w.z, w.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        o[j] = f32x2_to_bf16x2(bf16x2_lo(a[j]) + bf16x2_lo(b[j]), bf16x2_hi(a[j]) + bf16x2_hi(b[j]));
      v = make_uint4(o[0], o[1], o[2], o[3]);
      xr[i] = v;
    }
    const uint32_t a[4] = {v.x, v.y, v.z, v.w};
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s = fmaf(bf16x2_lo(a[j]), bf16x2_lo(a[j]), s);
      s = fmaf(bf16x2_hi(a[j]), bf16x2_hi(a[j]), s);
    }
    acc += s;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  const float r = __frsqrt_rn(__fdiv_rn(acc, static_cast<float>(hs)) + eps);
  for (int i = lane; i < n8; i += 32) {  // each lane reads back the groups it has just written
    const uint4 v = xr[i];
    const uint32_t a[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = f32x2_to_bf16x2(bf16x2_lo(a[j]) * r, bf16x2_hi(a[j]) * r);
    hr[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// One block of 256 threads per token: routed sum (slot order), gate =
// sigmoid(x . gate_scalar) with the reference's 256 strided fused partials and
// halving tree, y = bf16(fma(gate, shared_down, routed)) (MoECombineKernel,
// src/model/moe.cu:291-321).  Also leaves the fp32 routed sum in `routed` when that is not null.
// PRELOAD: request all of the token's rows before the first is used (k <= 16), so that the
// slot-order sum costs one memory round trip instead of k: 3 us of a 13 us decode launch; at
// 16 K tokens the extra registers cost more than the latency they hide (254 vs 175 us).
// NORM: the stack's residual + RMSNorm step rides on the kernel (a separate instantiation, so that the
// plain combine, which is at the HBM bound at prefill sizes, keeps its registers and shared memory).
template <bool PRELOAD, bool NORM>
__global__ void __launch_bounds__(256) final_combine_kernel(
    const uint16_t* __restrict__ dn_out, const int32_t* __restrict__ row_of_flat,
    const float* __restrict__ rw, const uint16_t* __restrict__ shared_down,
    const uint16_t* __restrict__ x, const uint16_t* __restrict__ gate_scalar,
    float* __restrict__ routed, uint16_t* __restrict__ y, int T, int k, int hs, const HcWrite hcw,
    const NormWrite nw) {
  chain_wait();
  __shared__ float part[256];
  __shared__ float s_sq[NORM ? kNormWriteMaxHs / 8 : 1];   // per 8-column group: sum of squares of the new residual row
  __shared__ float s_rnorm;
  __shared__ int s_row[16];
  __shared__ float s_w[16];
  const int t = blockIdx.x;
  if (threadIdx.x < k) {
    s_row[threadIdx.x] = row_of_flat[t * k + threadIdx.x];
    s_w[threadIdx.x] = rw[t * k + threadIdx.x];
  }
  __syncthreads();
  // The rows of this thread's first column chunk are requested before the gate's dot product
  // and reduction, so that the two memory round trips of the kernel overlap.
  const int n8 = hs >> 3;
  [[maybe_unused]] uint4 v[16];
  if constexpr (PRELOAD) {
    if (static_cast<int>(threadIdx.x) < n8) {
#pragma unroll
      for (int s = 0; s < 16; ++s)
        if (s < k && s_row[s] >= 0)
          v[s] = __ldg(reinterpret_cast<const uint4*>(dn_out + static_cast<size_t>(s_row[s]) * hs) + threadIdx.x);
    }
  }
  float acc = 0.0f;
  for (int c = threadIdx.x; c < hs; c += 256)
    acc = fmaf(bf16_to_f32(x[static_cast<size_t>(t) * hs + c]), bf16_to_f32(gate_scalar[c]), acc);
  part[threadIdx.x] = acc;
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (threadIdx.x < off) part[threadIdx.x] += part[threadIdx.x + off];
    __syncthreads();
  }
  const float gate = __frcp_rn(1.0f + __expf(-part[0]));
  for (int c8 = threadIdx.x; c8 < n8; c8 += 256) {
    float a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = 0.0f;
    if constexpr (PRELOAD) {
      if (c8 != static_cast<int>(threadIdx.x)) {   // later chunks of wide rows (hs > 2048)
#pragma unroll
        for (int s = 0; s < 16; ++s)
          if (s < k && s_row[s] >= 0)
            v[s] = __ldg(reinterpret_cast<const uint4*>(dn_out + static_cast<size_t>(s_row[s]) * hs) + c8);
      }
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        if (s < k && s_row[s] >= 0) {
          const float wgt = s_w[s];
          const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            a[2 * j] = fmaf(wgt, bf16x2_lo(w[j]), a[2 * j]);
            a[2 * j + 1] = fmaf(wgt, bf16x2_hi(w[j]), a[2 * j + 1]);
          }
        }
      }
    } else {
      for (int s = 0; s < k; ++s) {
        const int r = s_row[s];
        if (r < 0) continue;
        const float wgt = s_w[s];
        const uint4 rv = __ldg(reinterpret_cast<const uint4*>(dn_out + static_cast<size_t>(r) * hs) + c8);
        const uint32_t w[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          a[2 * j] = fmaf(wgt, bf16x2_lo(w[j]), a[2 * j]);
          a[2 * j + 1] = fmaf(wgt, bf16x2_hi(w[j]), a[2 * j + 1]);
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = 0.0f + a[j];  // the reference adds into a zeroed buffer
    if (routed) {  // optional fp32 copy of the routed sum
      float4* rdst = reinterpret_cast<float4*>(routed + static_cast<size_t>(t) * hs) + c8 * 2;
      rdst[0] = make_float4(a[0], a[1], a[2], a[3]);
      rdst[1] = make_float4(a[4], a[5], a[6], a[7]);
    }
    const uint4 sv = __ldg(reinterpret_cast<const uint4*>(shared_down + static_cast<size_t>(t) * hs) + c8);
    const uint32_t sw[4] = {sv.x, sv.y, sv.z, sv.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      o[j] = f32x2_to_bf16x2(fmaf(gate, bf16x2_lo(sw[j]), a[2 * j]),
                             fmaf(gate, bf16x2_hi(sw[j]), a[2 * j + 1]));
    *(reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * hs) + c8) = make_uint4(o[0], o[1], o[2], o[3]);
    // The gated residual write of the layer (GatedResidualFrame::Write, CombineWithGateKernel,
    // src/model/hyperconnection.cu:286-305): out[t, b, c] = bf16(R[t, b, c] + y[t, c] * gate[t, b])
    // with the bf16-rounded y and one fused multiply-add, for every hyper-connection branch b.
    for (int b = 0; b < hcw.hc; ++b) {
      const float inj = bf16_to_f32(hcw.inject_gate[static_cast<size_t>(t) * hcw.hc + b]);
      const size_t at = (static_cast<size_t>(t) * hcw.hc + b) * hs;
      const uint4 rv = __ldg(reinterpret_cast<const uint4*>(hcw.residual + at) + c8);
      const uint32_t r[4] = {rv.x, rv.y, rv.z, rv.w};
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        w[j] = f32x2_to_bf16x2(fmaf(bf16x2_lo(o[j]), inj, bf16x2_lo(r[j])), fmaf(bf16x2_hi(o[j]), inj, bf16x2_hi(r[j])));
      *(reinterpret_cast<uint4*>(hcw.out + at) + c8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    // The step between two layers of a decode stack, x <- bf16(x + y) and h = RMSNorm(x), with
    // the arithmetic of residual_rmsnorm_kernel: the sum from the bf16-rounded y, and a sum of
    // squares per 8-column group that is folded below in that kernel's order.
    if constexpr (NORM) {
      uint4* xr = reinterpret_cast<uint4*>(nw.residual + static_cast<size_t>(t) * hs) + c8;
      const uint4 xv = *xr;
      const uint32_t xa[4] = {xv.x, xv.y, xv.z, xv.w};
      uint32_t xn[4];
      float sq = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xn[j] = f32x2_to_bf16x2(bf16x2_lo(xa[j]) + bf16x2_lo(o[j]), bf16x2_hi(xa[j]) + bf16x2_hi(o[j]));
        sq = fmaf(bf16x2_lo(xn[j]), bf16x2_lo(xn[j]), sq);
        sq = fmaf(bf16x2_hi(xn[j]), bf16x2_hi(xn[j]), sq);
      }
      *xr = make_uint4(xn[0], xn[1], xn[2], xn[3]);
      s_sq[c8] = sq;
    }
  }
  if constexpr (NORM) {
    __syncthreads();
    if (threadIdx.x < 32) {   // residual_rmsnorm_kernel: lane l adds groups l, l+32, ... in order, then a butterfly
      float sum = 0.0f;
      for (int i = threadIdx.x; i < n8; i += 32) sum += s_sq[i];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (threadIdx.x == 0) s_rnorm = __frsqrt_rn(__fdiv_rn(sum, static_cast<float>(hs)) + nw.eps);
    }
    __syncthreads();
    const float r = s_rnorm;
    for (int c8 = threadIdx.x; c8 < n8; c8 += 256) {   // each thread reads back the groups it has just written
      const uint4 xv = *(reinterpret_cast<const uint4*>(nw.residual + static_cast<size_t>(t) * hs) + c8);
      const uint32_t xa[4] = {xv.x, xv.y, xv.z, xv.w};
      uint32_t h[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) h[j] = f32x2_to_bf16x2(bf16x2_lo(xa[j]) * r, bf16x2_hi(xa[j]) * r);
      *(reinterpret_cast<uint4*>(nw.out + static_cast<size_t>(t) * hs) + c8) = make_uint4(h[0], h[1], h[2], h[3]);
    }
  }
}

}  // namespace

cudaError_t routing_set_attributes() {
  cudaError_t e;
  if ((e = cudaFuncSetAttribute(plan_small_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536)) != cudaSuccess)
    return e;
  if ((e = cudaFuncSetAttribute(plan_small_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536)) != cudaSuccess)
    return e;
  if ((e = cudaFuncSetAttribute(small_m_linear_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 98304)) != cudaSuccess)
    return e;
  if ((e = cudaFuncSetAttribute(small_m_linear_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 98304)) != cudaSuccess)
    return e;
  return cudaFuncSetAttribute(small_m_linear_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 98304);
}

bool chaining_enabled() {
  static const bool on = getenv("Q4T_NO_CHAIN") == nullptr;
  return on;
}
namespace {
thread_local bool t_chain_break = true;  // a thread's first launch is an ordinary one
}
void chain_break() { t_chain_break = true; }
bool chain_break_pending() {
  const bool v = t_chain_break;
  t_chain_break = false;
  return v;
}

cudaError_t launch_small_m_linear(const uint16_t* x, const uint16_t* w, uint16_t* y, int M, int N,
                                  int K, cudaStream_t stream) {
  const dim3 blocks(static_cast<unsigned>((N + 7) / 8)), threads(256);
  const size_t smem = static_cast<size_t>(M) * K * sizeof(uint16_t);
  if (M <= 1) return launch_chained(small_m_linear_kernel<1>, blocks, threads, smem, stream, x, w, y, M, N, K);
  if (M <= 4) return launch_chained(small_m_linear_kernel<4>, blocks, threads, smem, stream, x, w, y, M, N, K);
  return launch_chained(small_m_linear_kernel<8>, blocks, threads, smem, stream, x, w, y, M, N, K);
}

cudaError_t launch_topk(const uint16_t* logits, const int32_t* fixed_ids, int32_t* ids, float* rw,
                        int T, int E, int k, cudaStream_t stream) {
  return launch_chained(topk_kernel, dim3(static_cast<unsigned>((T + 7) / 8)), dim3(256), 0, stream, logits, fixed_ids,
                        ids, rw, T, E, k);
}

bool route_and_plan_fits(int T, int k) { return T * k <= kPlanSmallMax && T <= 16; }

cudaError_t launch_route_and_plan(const uint16_t* logits, const int32_t* fixed_ids, int32_t* ids, float* rw, int T,
                                  int E, int k, int max_tiles, const PlanTables& p, cudaStream_t stream) {
  return launch_chained(plan_small_kernel<true>, dim3(1), dim3(1024), 32 * E * sizeof(uint16_t), stream,
                        static_cast<const int32_t*>(nullptr), T * k, E, max_tiles, p, logits, fixed_ids, ids, rw, T, k,
                        E, 0);
}

bool route_plan_cluster_fits(int T, int k, int E) {
  return T > 16 && T <= kRouteClusterCtas * 32 && k >= 1 && k <= 16 && E <= 1024;
}

cudaError_t launch_route_plan_cluster(const uint16_t* logits, const int32_t* fixed_ids, int32_t* ids, float* rw, int T,
                                      int E, int k, int max_tiles, const PlanTables& p, cudaStream_t stream) {
  return launch_chained_cluster(route_plan_cluster_kernel, dim3(kRouteClusterCtas), dim3(1024),
                                16 * static_cast<size_t>(E) * sizeof(uint16_t), stream, kRouteClusterCtas, logits,
                                fixed_ids, ids, rw, T, k, E, max_tiles, p, 0);
}

cudaError_t launch_plan(const int32_t* ids, int R, int E, int max_tiles, const PlanTables& p,
                        cudaStream_t stream, bool even_tiles) {
  const int even = even_tiles ? 1 : 0;
  if (even) max_tiles &= ~1;  // the tile count handed to the GEMMs stays even when it is capped
  if (R <= kPlanSmallMax)
    return launch_chained(plan_small_kernel<false>, dim3(1), dim3(1024), 32 * E * sizeof(uint16_t), stream, ids, R, E,
                          max_tiles, p, static_cast<const uint16_t*>(nullptr), static_cast<const int32_t*>(nullptr),
                          static_cast<int32_t*>(nullptr), static_cast<float*>(nullptr), 0, 0, 0, even);
  const int nblk = (R + kPlanChunk - 1) / kPlanChunk;
  cudaError_t e;
  if ((e = launch_chained(plan_hist_kernel, dim3(nblk), dim3(256), E * sizeof(int32_t), stream, ids, R, E,
                          p.blk_counts)) != cudaSuccess)
    return e;
  if ((e = launch_chained(plan_scan_kernel, dim3(1), dim3(1024), 0, stream, nblk, E, max_tiles, p, even)) != cudaSuccess)
    return e;
  return launch_chained(plan_scatter_kernel, dim3(nblk), dim3(256), 7 * E * sizeof(int32_t), stream, ids, R, E, p);
}

cudaError_t launch_ep_split_ids(const int32_t* ids, int R, int E, int experts_per_rank, int32_t* dest,
                                int32_t* local, cudaStream_t stream) {
  if (R == 0) return cudaSuccess;
  ep_split_ids_kernel<<<(R + 255) / 256, 256, 0, stream>>>(ids, R, E, experts_per_rank, dest, local);
  return cudaGetLastError();
}

cudaError_t launch_ep_localise_ids(const int32_t* ids, int R, int E, int world, int rank, int map,
                                   const int32_t* placement, int flats_per_rank, int32_t* local,
                                   cudaStream_t stream) {
  ep_localise_ids_kernel<<<(R + 255) / 256, 256, 0, stream>>>(ids, R, E, world, rank, map, placement, flats_per_rank,
                                                              local);
  return cudaGetLastError();
}

cudaError_t launch_remap_ids(const int32_t* ids, const int32_t* slot_of_expert, int32_t* out, int R, int E, int slots,
                             cudaStream_t stream) {
  if (R == 0) return cudaSuccess;
  return launch_chained(remap_ids_kernel, dim3((R + 255) / 256), dim3(256), 0, stream, ids, slot_of_expert, out, R, E,
                        slots);
}

cudaError_t launch_ep_flat_rows(const int32_t* ids, int R, int E, int32_t* row_of_flat, cudaStream_t stream) {
  ep_flat_rows_kernel<<<(R + 255) / 256, 256, 0, stream>>>(ids, R, E, row_of_flat);
  return cudaGetLastError();
}

cudaError_t launch_gather_rows(const uint16_t* src, const int32_t* index, int div, const int32_t* rows_dev,
                               int rows, int width, uint16_t* out, const int32_t* aux, int32_t* aux_out,
                               cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(rows) * (width / 8);
  if (total == 0) return cudaSuccess;
  gather_rows_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, stream>>>(src, index, div, rows_dev, rows,
                                                                                     width, out, aux, aux_out);
  return cudaGetLastError();
}

cudaError_t launch_routed_combine(const uint16_t* dn_out, const int32_t* row_of_flat,
                                  const float* rw, float* y, int T, int k, int hs,
                                  cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(T) * (hs / 8);
  return launch_chained(routed_combine_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream,
                        dn_out, row_of_flat, rw, y, T, k, hs);
}

cudaError_t launch_swiglu(const uint16_t* gu, uint16_t* out, int T, int inner, cudaStream_t stream) {
  const int64_t total = static_cast<int64_t>(T) * inner;
  return launch_chained(swiglu_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream, gu, out,
                        T, inner);
}

cudaError_t launch_residual_rmsnorm(uint16_t* x, const uint16_t* y, uint16_t* h, int T, int hs, float eps,
                                    cudaStream_t stream) {
  return launch_chained(residual_rmsnorm_kernel, dim3((T + 7) / 8), dim3(256), 0, stream, x, y, h, T, hs, eps);
}

cudaError_t launch_final_combine(const uint16_t* dn_out, const int32_t* row_of_flat, const float* rw,
                                 const uint16_t* shared_down, const uint16_t* x,
                                 const uint16_t* gate_scalar, float* routed, uint16_t* y, int T,
                                 int k, int hs, cudaStream_t stream, const HcWrite& hcw, const NormWrite& nw) {
  if (nw.residual && (hs > kNormWriteMaxHs || hs % 8 || !nw.out)) return cudaErrorInvalidValue;
  if (nw.residual) {
    if (T <= 1024)
      return launch_chained(final_combine_kernel<true, true>, dim3(T), dim3(256), 0, stream, dn_out, row_of_flat, rw,
                            shared_down, x, gate_scalar, routed, y, T, k, hs, hcw, nw);
    return launch_chained(final_combine_kernel<false, true>, dim3(T), dim3(256), 0, stream, dn_out, row_of_flat, rw,
                          shared_down, x, gate_scalar, routed, y, T, k, hs, hcw, nw);
  }
  if (T <= 1024)
    return launch_chained(final_combine_kernel<true, false>, dim3(T), dim3(256), 0, stream, dn_out, row_of_flat, rw,
                          shared_down, x, gate_scalar, routed, y, T, k, hs, hcw, nw);
  return launch_chained(final_combine_kernel<false, false>, dim3(T), dim3(256), 0, stream, dn_out, row_of_flat, rw,
                        shared_down, x, gate_scalar, routed, y, T, k, hs, hcw, nw);
}

}  // namespace q4t
