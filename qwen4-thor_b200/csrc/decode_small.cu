// The routed experts for decode-sized batches (up to 128 tokens; the entry points send batches of
// up to 64 here by default), the counterpart of the reference's device-routed decode path
// (MoEDeviceDecode / MoEDeviceDecodeMulti, include/q4t/quant/moe_decode.h:8-36,
// src/quant/moe_decode.cu:762-823): no permutation step, no separate quantise step, and tiles
// shaped for streaming weights rather than for arithmetic.
//
// With a handful of tokens every selected expert has one or two rows, so the work is reading
// each selected expert's weights once.  The general grouped GEMM puts the token rows on the
// 128-row side of the tcgen05 instruction and 256 weight rows on the other, which gives 4 (gate
// /up) or 8 (down) tiles per expert: 40 tiles for one token on 148 SMs.  Here the operands trade
// places: a tile is 128 WEIGHT rows (the M side, one full block-scale atom per 64 elements of K)
// against up to 16 token rows (the N side), so an expert gives 2*is/128 gate/up tiles and hs/128
// down tiles, and each CTA streams 128 x K/2 bytes of codes through a ring of TMA stages.
//
// The work is the list of (expert, weight tile) pairs over the experts that have entries, in the
// order of their first (token,slot) entry; an expert with more than 16 entries takes several
// passes over its tiles.  Every CTA derives the same list from the id table (at most 2048
// entries) and takes one contiguous share of it, so that its consecutive tiles mostly belong to
// one expert and reuse the token-side operand; with few tiles that is one tile per CTA, with many
// the CTAs are persistent and the weight ring keeps streaming across tiles while the previous
// tile's rows are stored.  The token-side operand never exists in global memory: four warps build it in
// shared memory, in the 128-byte-swizzled K-major layout and the scale-atom layout that TMA
// would have produced --
//   gate/up: the bf16 token rows quantised with the expert's input scale (the arithmetic of
//            the row quantiser, src/quant/act_quant.cu:62-90 of the reference);
//   down:    SwiGLU of the bf16 gate|up rows the first kernel stored, quantised with the
//            expert's down input scale (src/quant/moe_gemm.cu:173-241) --
// while the weight tiles are already in flight.  Every output element is the same sequence of
// block-scaled tcgen05 MMAs over K as in the general kernel (operands swapped), followed by the
// same alpha multiply and bf16 rounding.  Rows are stored in (token,slot) order: row_of_flat is
// the identity (-1 for skipped entries), which is what the combine kernels consume.
#include "kernels.h"
#include "q4t_device.cuh"

namespace q4t {

namespace {

constexpr int kSmallThreads = 192;                // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: operand + epilogue
constexpr int kWorkers = 128;
constexpr uint32_t kWTileBytes = 128 * 128;       // 128 weight rows x 128 bytes of codes
constexpr uint32_t kWSfBytes = 4 * 512;           // their scale atoms for the four MMAs of a k-block
constexpr uint32_t kSmallStage = kWTileBytes + kWSfBytes;
constexpr uint32_t kOpTileBytes = kSmallN * 128;  // 16 token rows x 128 bytes
// Token-side scale atoms are laid down 256 bytes apart: rows 0-15 of an atom are its first 256
// bytes, and the other half (rows 16-31, never used with 16 token rows) overlaps the next atom.
constexpr uint32_t kOpSfStride = 256;
constexpr int kSmallMaxStages = 10;
constexpr int kSmallSharedStages = 5;             // ring depth when two CTAs share an SM ...
constexpr size_t kSmallSharedBytes = 97 * 1024 + 512;   // ... and the dynamic shared memory each may then use, lists aside,
constexpr size_t kSmallSharedMaxBytes = 112 * 1024;      // ... or at most

struct SmallBars {
  uint64_t full[kSmallMaxStages];
  uint64_t empty[kSmallMaxStages];
  uint64_t operand_ready;   // 128 worker arrivals per operand build
  uint64_t acc_full[2];     // one per accumulator buffer
  uint64_t acc_empty[2];    // 4 worker warps per drain
  uint32_t tmem_base;
  uint32_t abort_flag;
  int n_serving;
  int n_found;                              // members collected for the expert being served
  int scan[kSmallThreads / 32];             // per-warp totals of the compaction
};

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void worker_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory"); }

// MODE 0: gate/up (operand = quantised token rows); MODE 1: down (operand = quantised SwiGLU rows).
template <int MODE>
__global__ void __launch_bounds__(kSmallThreads)
small_batch_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ SmallBatchArgs args) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ SmallBars bars;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stages = args.stages;
  const uint32_t k_bytes = static_cast<uint32_t>(args.K) >> 1;
  const int nkb = static_cast<int>((k_bytes + 127u) >> 7);
  const uint32_t ntk = (static_cast<uint32_t>(args.K) + 63u) >> 6;
  const uint32_t op_base = smem_base + static_cast<uint32_t>(stages) * kSmallStage;   // token-side codes
  const uint32_t opsf_base = op_base + static_cast<uint32_t>(nkb) * kOpTileBytes;      // token-side scale atoms
  // the lists, sized by the number of entries (behind the operand)
  const int r_pad = (args.R + 7) & ~7;
  int16_t* const l_ids = reinterpret_cast<int16_t*>(smem_gen + (opsf_base - smem_base) + ntk * kOpSfStride);   // expert of each entry, -1 = skipped
  int16_t* const l_serving = l_ids + r_pad;      // the experts that have entries, by first entry
  int16_t* const l_members = l_serving + r_pad;  // entries of the expert being served (any order)
  uint8_t* const l_passes = reinterpret_cast<uint8_t*>(l_members + r_pad);   // ceil(entries / 16) of each serving expert
  volatile uint32_t* abort_flag = &bars.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    mbar_init(smem_u32(&bars.operand_ready), kWorkers);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&bars.acc_full[b]), 1);
      mbar_init(smem_u32(&bars.acc_empty[b]), kWorkers / 32);
    }
    bars.abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars.tmem_base), args.tmem_cols);
    tmem_relinquish();
  }
  // Per-expert tables for the work list (entries of each expert, its first entry) live in the
  // weight ring, which no copy has touched yet; they are cleared while the kernel still waits
  // for its predecessor.
  const int R = args.R, E = args.E;
  int32_t* const count_of = reinterpret_cast<int32_t*>(smem_gen);
  int32_t* const first_of = count_of + E;
  for (int e = threadIdx.x; e < E; e += kSmallThreads) {
    count_of[e] = 0;
    first_of[e] = 0x7fffffff;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;
  // The gate/up kernel follows the kernel that selected the experts; the down kernel reads the
  // same ids, which were complete before the gate/up kernel started, and waits later, just
  // before it touches the gate|up rows.
  if (MODE == 0) {
    chain_wait();
    // the down kernel may start now: it fetches its weight tiles (which depend only on the
    // ids) into shared memory while this kernel runs, and waits before it reads our rows
    if (args.release_next) chain_release_next();
  }

  // ---- the work list, the same in every CTA: the experts that have entries, in the order of their first entry,
  // with the number of 16-row passes each needs
  for (int i = threadIdx.x; i < R; i += kSmallThreads) {
    const int e = args.ids[i];
    const bool in_range = e >= 0 && e < E;
    l_ids[i] = static_cast<int16_t>(in_range ? e : -1);
    if (in_range) {
      atomicAdd(&count_of[e], 1);
      atomicMin(&first_of[e], i);
    }
    if (MODE == 0 && blockIdx.x == 0) args.row_of_flat[i] = in_range ? i : -1;
  }
  // the first CTA also clears the status word (it starts long before any bounded wait of this
  // launch could run out)
  if (MODE == 0 && blockIdx.x == 0 && threadIdx.x == 0 && args.status) *args.status = 0;
  __syncthreads();
  {
    // compaction in the order in which the experts first appear: thread t owns entries [t*c, (t+1)*c)
    const int c = (R + kSmallThreads - 1) / kSmallThreads;
    const int i0 = min(R, static_cast<int>(threadIdx.x) * c), i1 = min(R, i0 + c);
    int mine = 0;
    for (int i = i0; i < i1; ++i) {
      const int e = l_ids[i];
      mine += (e >= 0 && first_of[e] == i) ? 1 : 0;
    }
    int incl = mine;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) bars.scan[warp] = incl;
    __syncthreads();
    int pos = incl - mine;
    for (int wq = 0; wq < warp; ++wq) pos += bars.scan[wq];
    for (int i = i0; i < i1; ++i) {
      const int e = l_ids[i];
      if (e >= 0 && first_of[e] == i) {
        l_serving[pos] = static_cast<int16_t>(e);
        l_passes[pos] = static_cast<uint8_t>((count_of[e] + kSmallN - 1) / kSmallN);
        ++pos;
      }
    }
    if (threadIdx.x == kSmallThreads - 1) bars.n_serving = pos;
    fence_async_smem();   // the ring is written by TMA from here on
  }
  __syncthreads();
  // this CTA's share of the (serving entry, weight tile) pairs: contiguous, sizes differ by at most one
  const int total = bars.n_serving * args.n_tiles;
  const int ctas = min(static_cast<int>(gridDim.x), total);
  int t_begin = 0, t_end = 0;
  if (static_cast<int>(blockIdx.x) < ctas) {
    const int base = total / ctas, rem = total - base * ctas, c = blockIdx.x;
    t_begin = c * base + min(c, rem);
    t_end = t_begin + base + (c < rem ? 1 : 0);
  }

  if (warp == 0) {
    // ---------------------------------------------------------- weight tiles by TMA
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = t_begin; t < t_end && ok; ++t) {
        const int u = t / args.n_tiles, nt = t - u * args.n_tiles;
        const int e = l_serving[u];
        const int passes = l_passes[u];
        const int w_row0 = e * args.w_rows_per_expert + nt * 128;
        const uint8_t* w_sf = args.w_sf + static_cast<size_t>(e) * args.w_sf_stride + static_cast<size_t>(nt) * ntk * 512u;
        for (int p = 0; p < passes && ok; ++p) {
          uint32_t k_left = k_bytes;
          const uint8_t* sf = w_sf;
          for (int kb = 0; kb < nkb; ++kb) {
            const uint32_t full = smem_u32(&bars.full[stage]), empty = smem_u32(&bars.empty[stage]);
            if (!mbar_try_wait(empty, phase ^ 1u) && !mbar_wait(empty, phase ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            const uint32_t nm = k_left >= 128u ? 4u : k_left >> 5;
            const uint32_t sa = smem_base + static_cast<uint32_t>(stage) * kSmallStage;
            mbar_expect_tx(full, kWTileBytes + nm * 512u);
            tma_load_2d(sa, &tmap_w, kb * 128, w_row0, full);
            bulk_load(sa + kWTileBytes, sf, nm * 512u, full);
            sf += 2048;
            k_left -= 128u;
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
      if (!ok && args.status) atomicMax(args.status, 1);
    }
    if (MODE == 1) chain_wait();
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (MODE == 1) chain_wait();
    if (lane == 0) {
      // M = 128 weight rows, N = 16 token rows, both operands K-major e2m1, ue4m3 scales
      constexpr uint32_t idesc =
          (1u << 7) | (1u << 10) | ((static_cast<uint32_t>(kSmallN) >> 3) << 17) | ((128u >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint64_t wdesc0 = umma_desc_sw128(smem_base), sfw0 = umma_desc_sf(smem_base + kWTileBytes);
      const uint64_t odesc0 = umma_desc_sw128(op_base), sfo0 = umma_desc_sf(opsf_base);
      const uint32_t bar_full0 = smem_u32(&bars.full[0]), bar_empty0 = smem_u32(&bars.empty[0]);
      uint32_t builds = 0, unit = 0;   // operand builds awaited so far; (tile, pass) units issued so far
      int prev_u = -1;
      for (int t = t_begin; t < t_end && ok; ++t) {
        const int u = t / args.n_tiles;
        const int passes = l_passes[u];
        for (int p = 0; p < passes && ok; ++p, ++unit) {
          if (u != prev_u || passes > 1) {   // a new token-side operand
            if (!mbar_wait(smem_u32(&bars.operand_ready), builds & 1u, abort_flag)) {
              ok = false;
              break;
            }
            ++builds;
          }
          prev_u = u;
          const uint32_t ab = unit & 1u;
          if (!mbar_wait(smem_u32(&bars.acc_empty[ab]), ((unit >> 1) & 1u) ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t acc = tmem + ab * 16u;
          uint32_t k_left = k_bytes;
          for (int kb = 0; kb < nkb; ++kb) {
            const uint32_t full = bar_full0 + static_cast<uint32_t>(stage) * 8u;
            if (!mbar_try_wait(full, phase) && !mbar_wait(full, phase, abort_flag)) {
              ok = false;
              break;
            }
            tc_fence_after();
            // descriptors differ from those of stage 0 / k-block 0 by constants in the 14-bit
            // start-address field (16-byte units), so plain 64-bit adds never carry out of it
            const uint64_t soff = static_cast<uint64_t>(stage) * (kSmallStage >> 4);
            const uint64_t wdesc = wdesc0 + soff, sfw = sfw0 + soff;
            const uint64_t odesc = odesc0 + static_cast<uint64_t>(kb) * (kOpTileBytes >> 4);
            const uint64_t sfo = sfo0 + static_cast<uint64_t>(kb) * (4u * kOpSfStride >> 4);
            const uint32_t tsf = tmem + 32u + static_cast<uint32_t>(stage) * 32u;   // this stage's scale columns
            const uint32_t tso = tsf + 16u;
            const uint32_t first = kb != 0;
            if (k_left >= 128u) {
#pragma unroll
              for (uint32_t kk = 0; kk < 4; ++kk) {
                tc_cp_sf(tsf + kk * 4u, sfw + kk * 32u);
                tc_cp_sf(tso + kk * 4u, sfo + kk * (kOpSfStride >> 4));
              }
#pragma unroll
              for (uint32_t kk = 0; kk < 4; ++kk)
                tc_mma_nvf4(acc, wdesc + kk * 2u, odesc + kk * 2u, idesc, tsf + kk * 4u, tso + kk * 4u,
                            kk == 0 ? first : 1u);
            } else {
              const uint32_t nm = k_left >> 5;
              for (uint32_t kk = 0; kk < nm; ++kk) {
                tc_cp_sf(tsf + kk * 4u, sfw + kk * 32u);
                tc_cp_sf(tso + kk * 4u, sfo + kk * (kOpSfStride >> 4));
              }
              for (uint32_t kk = 0; kk < nm; ++kk)
                tc_mma_nvf4(acc, wdesc + kk * 2u, odesc + kk * 2u, idesc, tsf + kk * 4u, tso + kk * 4u,
                            kk == 0 ? first : 1u);
            }
            tc_commit(bar_empty0 + static_cast<uint32_t>(stage) * 8u);
            k_left -= 128u;
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
          if (ok) tc_commit(smem_u32(&bars.acc_full[ab]));
        }
      }
      if (!ok && args.status) atomicMax(args.status, 2);
    }
  } else {
    // ---------------------------------------------------------- operand builders / epilogue
    // (the down kernel's member lists and scales depend only on the ids: it waits for the
    // gate/up kernel just before the first load of a gate|up row)
    bool waited = MODE == 0;
    const int w = static_cast<int>(threadIdx.x) - 64;
    const int quad = warp & 3;
    const int groups = args.K >> 4;
    bool ok = true;
    uint32_t unit = 0;
    int prev_u = -1;
    int n_members = 0;
    for (int t = t_begin; t < t_end && ok; ++t) {
      const int u = t / args.n_tiles, nt = t - u * args.n_tiles;
      const int e = l_serving[u];
      const bool new_expert = u != prev_u;
      if (new_expert) {
        // the entries that name this expert, in whatever order the threads find them: an
        // output row depends only on its own operand row, not on its position in the pass.
        // (The previous expert's list is no longer needed: its rows were stored before this.)
        worker_sync();
        if (w == 0) bars.n_found = 0;
        worker_sync();
        for (int i = w; i < R; i += kWorkers)
          if (l_ids[i] == e) l_members[atomicAdd(&bars.n_found, 1)] = static_cast<int16_t>(i);
        worker_sync();
        n_members = bars.n_found;
      }
      prev_u = u;
      const float in_scale = args.in_scale[e];
      const float alpha = args.alpha_w[e] * args.alpha_a[e];
      const int n_out = nt * 128 + quad * 32 + lane;   // the output column this thread's TMEM lane holds
      const int passes = (n_members + kSmallN - 1) / kSmallN;
      for (int p = 0; p < passes && ok; ++p, ++unit) {
        const int m0 = p * kSmallN;
        const int rows = min(kSmallN, n_members - m0);
        if (new_expert || passes > 1) {
          // ---- build the token-side operand (the MMAs that read the previous one have
          // completed: their accumulators were awaited below before this point)
          if (!waited) {
            chain_wait();
            waited = true;
          }
          for (int item = w; item < rows * groups; item += kWorkers) {
            const int j = item / groups, g = item - j * groups;
            const int entry = l_members[m0 + j];
            float a[16];
            if (MODE == 0) {
              const uint4* src = reinterpret_cast<const uint4*>(args.src + static_cast<size_t>(entry / args.k) * args.src_ld + g * 16);
              const uint4 v0 = __ldg(src), v1 = __ldg(src + 1);
              const uint32_t wv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                a[2 * i] = bf16x2_lo(wv[i]);
                a[2 * i + 1] = bf16x2_hi(wv[i]);
              }
            } else {
              // written by the previous kernel: plain loads, not the read-only path
              const uint4* gsrc = reinterpret_cast<const uint4*>(args.src + static_cast<size_t>(entry) * args.src_ld + g * 16);
              const uint4* usrc = reinterpret_cast<const uint4*>(args.src + static_cast<size_t>(entry) * args.src_ld + args.K + g * 16);
              const uint4 g0 = gsrc[0], g1 = gsrc[1], u0 = usrc[0], u1 = usrc[1];
              const uint32_t gb[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
              const uint32_t ub[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
              // (g * sigmoid(g)) * u on the bf16 projections, sigmoid through an IEEE reciprocal
              // of 1 + __expf(-g): the general kernel's epilogue arithmetic
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float gl = bf16x2_lo(gb[i]), gh = bf16x2_hi(gb[i]);
                const float dl = 1.0f + __expf(-gl), dh = 1.0f + __expf(-gh);
                const float sl = dl < Q4T_RCP_FAST_MAX ? rcp_rn_ge1(dl) : __frcp_rn(dl);
                const float sh = dh < Q4T_RCP_FAST_MAX ? rcp_rn_ge1(dh) : __frcp_rn(dh);
                a[2 * i] = (gl * sl) * bf16x2_lo(ub[i]);
                a[2 * i + 1] = (gh * sh) * bf16x2_hi(ub[i]);
              }
            }
            uint32_t lo, hi;
            const uint32_t sf = quantize_group16(a, in_scale, lo, hi);
            const uint32_t kb = static_cast<uint32_t>(g) >> 4, gi = static_cast<uint32_t>(g) & 15u;
            const uint32_t off = kb * kOpTileBytes + static_cast<uint32_t>(j) * 128u +
                                 (((gi >> 1) ^ (static_cast<uint32_t>(j) & 7u)) << 4) + (gi & 1u) * 8u;
            *reinterpret_cast<uint2*>(smem_gen + (op_base - smem_base) + off) = make_uint2(lo, hi);
            smem_gen[(opsf_base - smem_base) + (static_cast<uint32_t>(g) >> 2) * kOpSfStride + static_cast<uint32_t>(j) * 16u +
                     (static_cast<uint32_t>(g) & 3u)] = static_cast<uint8_t>(sf);
          }
          fence_async_smem();   // the tensor core reads these bytes through the async proxy
          mbar_arrive(smem_u32(&bars.operand_ready));
        }
        // ---- epilogue of this unit
        const uint32_t ab = unit & 1u;
        if (!mbar_wait(smem_u32(&bars.acc_full[ab]), (unit >> 1) & 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t v[16];
        tmem_ld16(tmem + (static_cast<uint32_t>(quad * 32) << 16) + ab * 16u, v);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty[ab]));
        if (n_out < args.w_rows_per_expert) {
#pragma unroll
          for (int j = 0; j < kSmallN; ++j)
            if (j < rows)
              args.out[static_cast<size_t>(l_members[m0 + j]) * args.ldo + n_out] =
                  f32_to_bf16(alpha * __uint_as_float(v[j]));
        }
      }
    }
    if (!ok && args.status && lane == 0) atomicMax(args.status, 3);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, args.tmem_cols);
  }
}

size_t small_list_bytes(int entries) { return static_cast<size_t>((entries + 7) & ~7) * 7; }

size_t small_smem_bytes(int K, int stages, int entries) {
  const size_t nkb = (static_cast<size_t>(K) / 2 + 127) / 128, ntk = (static_cast<size_t>(K) + 63) / 64;
  return 1024 + static_cast<size_t>(stages) * kSmallStage + nkb * kOpTileBytes + ntk * kOpSfStride +
         small_list_bytes(entries) + 256;
}

}  // namespace

// The ring holds a whole tile (every k-block in flight at once: with a handful of tiles the
// kernel is one memory round trip long) when there are few enough tiles for one CTA per SM;
// otherwise as many stages (at most a tile's worth) as leave room for two CTAs per SM, so that
// one streams while the other builds its operand or stores its rows.  The down projection's
// short tiles (two k-blocks at moe_is 512) give small CTAs, four to an SM, which measured
// faster than fewer CTAs with deeper rings.
int small_batch_stages(int K, int tiles, int entries) {
  const int nkb = (K / 2 + 127) / 128;
  constexpr int kDeepRingTiles = 148;  // one tile per SM of a B200
  int stages;
  if (tiles <= kDeepRingTiles) {
    stages = nkb < kSmallMaxStages ? nkb : kSmallMaxStages;
    while (stages > 2 && small_smem_bytes(K, stages, entries) > 200 * 1024) --stages;
  } else {
    // two CTAs per SM; with few entries they leave some shared memory to the kernels of the
    // shared expert, which run beside this one
    size_t budget = kSmallSharedBytes + small_list_bytes(entries);
    if (budget > kSmallSharedMaxBytes) budget = kSmallSharedMaxBytes;
    stages = nkb < kSmallSharedStages ? nkb : kSmallSharedStages;   // short reductions: more, smaller CTAs per SM
    while (stages > 2 && small_smem_bytes(K, stages, entries) > budget) --stages;
  }
  return small_smem_bytes(K, stages, entries) <= 200 * 1024 ? stages : 0;
}

cudaError_t small_batch_set_attributes() {
  cudaError_t e;
  if ((e = cudaFuncSetAttribute(small_batch_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)) != cudaSuccess)
    return e;
  return cudaFuncSetAttribute(small_batch_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
}

cudaError_t launch_small_batch(int mode, const CUtensorMap& tmap_w, const SmallBatchArgs& a, int num_sms,
                               cudaStream_t stream) {
  if (a.R <= 0 || a.R > kSmallMaxEntries || a.E > kSmallMaxExperts || a.stages <= 0) return cudaErrorInvalidValue;
  size_t smem = small_smem_bytes(a.K, a.stages, a.R);
  // Never more CTAs on an SM than its 512 tensor-memory columns serve: one more would sit in
  // its allocation until a whole neighbour had finished.  Shared memory is the resource that
  // bounds residency, so each CTA asks for more than a (limit+1)-th of the SM's 228 KB.
  const size_t tmem_limit = 512u / a.tmem_cols;
  const size_t min_smem = ((228 * 1024) / (tmem_limit + 1) + 16) & ~static_cast<size_t>(15);
  if (smem < min_smem) smem = min_smem;
  // as many CTAs as can be resident at once (shared memory: 228 KB per SM, 1 KB of it reserved
  // per CTA; tensor-memory columns), but never more than there can be tiles; CTAs beyond the
  // number of tiles that exist leave at once
  int per_sm = static_cast<int>((228 * 1024) / (smem + sizeof(SmallBars) + 64 + 1024));
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 4) per_sm = 4;
  if (static_cast<int>(512u / a.tmem_cols) < per_sm) per_sm = static_cast<int>(512u / a.tmem_cols);
  const int upper = a.R * a.n_tiles, resident = per_sm * num_sms;
  const dim3 grid(static_cast<unsigned>(upper < resident ? upper : resident));
  if (mode == 0) return launch_chained(small_batch_kernel<0>, grid, dim3(kSmallThreads), smem, stream, tmap_w, a);
  return launch_chained(small_batch_kernel<1>, grid, dim3(kSmallThreads), smem, stream, tmap_w, a);
}

}  // namespace q4t
