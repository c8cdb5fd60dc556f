// Tensor-core GEMMs for sm_100a: one persistent, warp-specialised kernel
// template that computes 128-row x 256-column tiles of  A[rows,K] . B[n,K]^T
// with tcgen05.mma, accumulators in TMEM, operands staged by TMA into
// 128-byte-swizzled shared memory.
//
//   NVF4 = true : kind::mxf4nvf4 block-scaled MMA (e2m1 codes, one ue4m3 scale
//                 per 16 elements, scale atoms copied to TMEM by tcgen05.cp);
//                 grouped over experts through a row-tile list.
//   NVF4 = false: kind::f16 MMA on bf16 operands (router logits, shared expert).
//
// Warp roles (576 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 2..17 = epilogue (warp w reads TMEM lanes 32*(w%4)..+31, i.e.
// one output row per thread; the four warps of a quadrant split the columns).
// Stages hand over through mbarriers; every wait is bounded and raises a
// status word instead of spinning forever.
//
// A tile's 256 accumulator columns are either 256 consecutive output columns
// or, for the SwiGLU epilogues, 128 gate columns followed by the 128 matching
// up columns, so that one thread sees g and u of the same output element.
#include "kernels.h"
#include "q4t_device.cuh"

namespace q4t {

namespace {

constexpr int kMaxStages = 4;
// Shared-memory ring depth.  Three 54 KB stages measured faster than four for the
// block-scaled tiles (decode gate/up 101 vs 108 us); the BF16 tiles keep four.
template <bool NVF4>
constexpr int num_stages() {
  return NVF4 ? 3 : 4;
}
constexpr int kEpiWarpsPerQuad = 4;                       // epilogue warps sharing one TMEM lane quadrant
constexpr int kEpiWarps = 4 * kEpiWarpsPerQuad;
constexpr int kFirstEpiWarp = 2;                          // warp 0: producer, warp 1: MMA issuer
constexpr int kThreads = (kFirstEpiWarp + kEpiWarps) * 32;
constexpr uint32_t kABytes = 128 * 128;                   // 128 rows x 128 bytes
constexpr uint32_t kSfaBytes = 4 * 512;                   // 4 atoms (one per MMA of a k-block)
constexpr uint32_t kSfbBytes = 8 * 512;                   // 2 x 4 atoms
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSfTmemBase = 256;                     // scale columns start after the accumulator
constexpr uint32_t kSfTmemPerStage = 48;                  // 16 (A) + 32 (B)

template <bool NVF4, int BN>
constexpr uint32_t stage_bytes() {
  return kABytes + BN * 128 + (NVF4 ? kSfaBytes + kSfbBytes : 0u);
}
// Per-warp staging for the bf16 row stores: 32 rows x 64 bytes, through which a
// warp turns "one row per lane" into "four lanes per row" so that each store
// instruction writes whole 64-byte row segments.
constexpr uint32_t kStoreStageBytes = 32 * 64;

struct Barriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full;
  uint64_t acc_empty;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

#ifdef Q4T_TRACE
// Timestamp slots per tile of CTA 0: [role][tile][slot]; role 0 producer, 1 MMA, 2 epilogue warp of quadrant 0.
#define Q4T_STAMP(role, tile_idx, slot)                                                            \
  do {                                                                                             \
    if (args.trace && blockIdx.x == 0 && (tile_idx) < 64) args.trace[((role) * 64 + (tile_idx)) * 8 + (slot)] = clock64(); \
  } while (0)
#else
#define Q4T_STAMP(role, tile_idx, slot) do {} while (0)
#endif

// BN = accumulator columns of one tile (256, or 64 for the narrow BF16 tiles
// that spread small-T projections over more SMs).
template <bool NVF4, Epilogue EPI, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ GemmArgs args) {
  static_assert(!NVF4 || BN == 256, "block-scaled tiles are 256 columns wide");
  extern __shared__ uint8_t smem_raw[];
  __shared__ Barriers bars;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr uint32_t kBBytes = BN * 128;
  constexpr uint32_t kStage = stage_bytes<NVF4, BN>();
  constexpr int kStages = num_stages<NVF4>();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &bars.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    mbar_init(smem_u32(&bars.acc_full), 1);
    mbar_init(smem_u32(&bars.acc_empty), kEpiWarps);
    bars.abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars.tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;
  // Barriers, tensor memory and descriptors are set up (possibly while the previous kernel
  // of the stream was still draining); from here on the kernel reads what that kernel wrote.
  chain_wait();

  const int m_tiles = args.ntiles_dev ? *args.ntiles_dev : args.ntiles_host;
  const int total_tiles = m_tiles * args.n_tiles;
  constexpr bool kSwiglu = (EPI == Epilogue::kSwigluBf16 || EPI == Epilogue::kSwigluQuant);
  constexpr int kHalf = BN / 2;  // SwiGLU: gate columns [0, kHalf), up columns [kHalf, BN)
  // bytes of K covered by one row: NVF4 packs two elements per byte
  const uint32_t k_bytes = NVF4 ? static_cast<uint32_t>(args.K) >> 1 : static_cast<uint32_t>(args.K) << 1;
  const int nkb = static_cast<int>((k_bytes + 127u) >> 7);
  const uint32_t ntk = (static_cast<uint32_t>(args.K) + 63u) >> 6;  // scale atoms along K

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t bar_full0 = smem_u32(&bars.full[0]), bar_empty0 = smem_u32(&bars.empty[0]);
      // The expert and first row of a tile are fetched one tile ahead: with short tiles (two
      // k-blocks in the down GEMM) a table lookup in front of every tile's first load would
      // leave the ring short of requests for the length of an L2 round trip.
      int next_group = 0, next_row0 = 0;
      if (static_cast<int>(blockIdx.x) < total_tiles) {
        const int mt0 = blockIdx.x / args.n_tiles;
        next_group = args.tile_expert ? args.tile_expert[mt0] : 0;
        next_row0 = args.tile_expert ? args.tile_row0[mt0] : mt0 * kTileM;
      }
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mt = tile / args.n_tiles, nt = tile - mt * args.n_tiles;
        const int group = next_group, row0 = next_row0;
        if (tile + static_cast<int>(gridDim.x) < total_tiles) {
          const int nmt = (tile + static_cast<int>(gridDim.x)) / args.n_tiles;
          next_group = args.tile_expert ? args.tile_expert[nmt] : 0;
          next_row0 = args.tile_expert ? args.tile_row0[nmt] : nmt * kTileM;
        }
        const int brow0 = group * args.b_rows_per_group + nt * args.n_per_tile;
        const int brow1 = brow0 + (kSwiglu ? args.up_row_offset : kHalf);
        // scale atoms of B: row blocks of 128 inside the group's buffer
        const uint32_t rb0 = static_cast<uint32_t>(nt * args.n_per_tile) >> 7;
        const uint32_t rb1 = rb0 + (kSwiglu ? static_cast<uint32_t>(args.up_row_offset) >> 7 : 1u);
        const bool second_half = kSwiglu || (nt * args.n_per_tile + 128 < args.b_rows_valid);
        // per-tile bases; the k loop below only adds constants
        const uint8_t* ga = NVF4 ? args.sfa_tiles + static_cast<size_t>(mt) * ntk * 512u : nullptr;
        const uint8_t* gbase = NVF4 ? args.sfb + static_cast<size_t>(group) * args.sfb_group_stride : nullptr;
        const uint8_t* gb0 = NVF4 ? gbase + static_cast<size_t>(rb0) * ntk * 512u : nullptr;
        const uint8_t* gb1 = NVF4 ? gbase + static_cast<size_t>(rb1) * ntk * 512u : nullptr;
        uint32_t k_left = k_bytes;
        int kc = 0;
        for (int kb = 0; kb < nkb; ++kb) {
          const uint32_t full = bar_full0 + stage * 8u, empty = bar_empty0 + stage * 8u;
          if (!mbar_try_wait(empty, phase ^ 1u) && !mbar_wait(empty, phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t nm = k_left >= 128u ? 4u : k_left >> 5;
          const uint32_t sa = smem_base + stage * kStage, sb = sa + kABytes;
          uint32_t tx = kABytes + kBBytes;
          if (NVF4) tx += nm * 512u * (second_half ? 3u : 2u);
          mbar_expect_tx(full, tx);
          tma_load_2d(sa, &tmap_a, kc, row0, full);
          tma_load_2d(sb, &tmap_b, kc, brow0, full);            // box = kHalf rows
          tma_load_2d(sb + kBBytes / 2, &tmap_b, kc, brow1, full);
          if (NVF4) {
            const uint32_t ssfa = sb + kBBytes, ssfb = ssfa + kSfaBytes;
            bulk_load(ssfa, ga, nm * 512u, full);
            bulk_load(ssfb, gb0, nm * 512u, full);
            if (second_half) bulk_load(ssfb + kSfbBytes / 2, gb1, nm * 512u, full);
            ga += 2048;
            gb0 += 2048;
            gb1 += 2048;
          }
          kc += NVF4 ? 128 : 64;  // inner coordinate in tensor-map elements
          k_left -= 128u;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok && args.status) atomicMax(args.status, 1);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptors (M = 128, N = BN, both operands K-major)
      constexpr uint32_t idesc_nvf4 =
          (1u << 7) | (1u << 10) | ((static_cast<uint32_t>(BN) >> 3) << 17) | ((128u >> 4) << 24);
      constexpr uint32_t idesc_bf16 = (1u << 4) | (1u << 7) | (1u << 10) |
                                      ((static_cast<uint32_t>(BN) >> 3) << 17) | ((128u >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      // descriptors of stage 0; later stages differ by a constant in the
      // 14-bit start-address field, so plain 64-bit adds never carry out of it
      const uint64_t adesc0 = umma_desc_sw128(smem_base), bdesc0 = umma_desc_sw128(smem_base + kABytes);
      const uint64_t sfa0 = umma_desc_sf(smem_base + kABytes + kBBytes);
      const uint64_t sfb0 = umma_desc_sf(smem_base + kABytes + kBBytes + kSfaBytes);
      const uint32_t bar_full0 = smem_u32(&bars.full[0]), bar_empty0 = smem_u32(&bars.empty[0]);
      const uint32_t bar_acc_full = smem_u32(&bars.acc_full), bar_acc_empty = smem_u32(&bars.acc_empty);
      int tcount = 0;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
        Q4T_STAMP(1, tcount, 0);
        if (!mbar_try_wait(bar_acc_empty, acc_phase ^ 1u) && !mbar_wait(bar_acc_empty, acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        Q4T_STAMP(1, tcount, 1);
        uint32_t k_left = k_bytes;
        for (int kb = 0; kb < nkb; ++kb) {
          const uint32_t full = bar_full0 + stage * 8u;
          if (!mbar_try_wait(full, phase) && !mbar_wait(full, phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (kb < 4) Q4T_STAMP(1, tcount, 3 + kb);
          const uint64_t soff = static_cast<uint64_t>(stage * (kStage >> 4));
          const uint64_t adesc = adesc0 + soff, bdesc = bdesc0 + soff;
          const uint32_t first = kb != 0;
          if (NVF4) {
            const uint64_t sfa = sfa0 + soff, sfb = sfb0 + soff;
            const uint32_t tsf = tmem + kSfTmemBase + stage * kSfTmemPerStage;
            if (k_left >= 128u) {
#pragma unroll
              for (uint32_t kk = 0; kk < 4; ++kk) {
                tc_cp_sf(tsf + kk * 4u, sfa + kk * 32u);
                tc_cp_sf(tsf + 16u + kk * 8u, sfb + kk * 32u);
                tc_cp_sf(tsf + 20u + kk * 8u, sfb + (kSfbBytes / 32) + kk * 32u);
              }
#pragma unroll
              for (uint32_t kk = 0; kk < 4; ++kk)
                tc_mma_nvf4(tmem, adesc + kk * 2u, bdesc + kk * 2u, idesc_nvf4, tsf + kk * 4u,
                            tsf + 16u + kk * 8u, kk == 0 ? first : 1u);
            } else {
              const uint32_t nm = k_left >> 5;
              for (uint32_t kk = 0; kk < nm; ++kk) {
                tc_cp_sf(tsf + kk * 4u, sfa + kk * 32u);
                tc_cp_sf(tsf + 16u + kk * 8u, sfb + kk * 32u);
                tc_cp_sf(tsf + 20u + kk * 8u, sfb + (kSfbBytes / 32) + kk * 32u);
              }
              for (uint32_t kk = 0; kk < nm; ++kk)
                tc_mma_nvf4(tmem, adesc + kk * 2u, bdesc + kk * 2u, idesc_nvf4, tsf + kk * 4u,
                            tsf + 16u + kk * 8u, kk == 0 ? first : 1u);
            }
          } else {
            if (k_left >= 128u) {
#pragma unroll
              for (uint32_t kk = 0; kk < 4; ++kk)
                tc_mma_f16(tmem, adesc + kk * 2u, bdesc + kk * 2u, idesc_bf16, kk == 0 ? first : 1u);
            } else {
              const uint32_t nm = k_left >> 5;
              for (uint32_t kk = 0; kk < nm; ++kk)
                tc_mma_f16(tmem, adesc + kk * 2u, bdesc + kk * 2u, idesc_bf16, kk == 0 ? first : 1u);
            }
          }
          tc_commit(bar_empty0 + stage * 8u);  // frees the stage once these MMAs have read it
          k_left -= 128u;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(bar_acc_full);
        Q4T_STAMP(1, tcount, 2);
        acc_phase ^= 1u;
      }
      if (!ok && args.status) atomicMax(args.status, 2);
    }
  } else if (warp >= kFirstEpiWarp) {
    // ------------------------------------------------------------ epilogue
    // Four warps share each TMEM lane quadrant and split the tile's columns
    // into units of 16 (store) or 16 gate + 16 up (SwiGLU).  A warp first
    // drains its units into registers (rounded to bf16 where the result is
    // bf16 anyway), hands the accumulator back, and only then does the math
    // and the stores, so the next tile's MMAs overlap with this work.
    const int quad = warp & 3;
    const int sub = (warp - kFirstEpiWarp) >> 2;  // 0..3 within the quadrant
    const int row = quad * 32 + lane;
    const uint32_t tacc = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    constexpr int kUnitCols = 16;
    constexpr int kUnits = kSwiglu ? kHalf / kUnitCols : BN / kUnitCols;
    constexpr int kUnitsPerWarp = (kUnits + kEpiWarpsPerQuad - 1) / kEpiWarpsPerQuad;
    uint32_t acc_phase = 0;
    bool ok = true;
    int tcount = 0;
    const bool stamp = warp == kFirstEpiWarp + 2 && lane == 0;  // quadrant 0, first of its four warps
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++tcount) {
      const int mt = tile / args.n_tiles, nt = tile - mt * args.n_tiles;
      const int group = args.tile_expert ? args.tile_expert[mt] : 0;
      const int row0 = args.tile_expert ? args.tile_row0[mt] : mt * kTileM;
      if (stamp) Q4T_STAMP(2, tcount, 0);
      const int nrows = args.tile_expert ? args.tile_nrows[mt] : min(kTileM, args.total_rows - row0);
      const float alpha =
          args.alpha_w ? args.alpha_w[group] * args.alpha_a[group] : args.alpha_const;
      // everything the epilogue reads from global memory is fetched before the wait
      [[maybe_unused]] float next_scale = 0.0f;
      if constexpr (EPI == Epilogue::kSwigluQuant) next_scale = args.next_scale[group];
      // Row-segment stores: where this lane's own row goes (its place in the tile's rows,
      // or, scattered, in its owner's buffer), looked up while the accumulator is still
      // being produced; the storing lanes fetch it by shuffle.
      [[maybe_unused]] unsigned long long my_row_ptr = 0;
      if constexpr (EPI == Epilogue::kStoreBf16Rows) {
        if (quad * 32 + lane < nrows) {
          const int r = row0 + quad * 32 + lane;
          if (args.scatter_flat) {
            const int f = args.scatter_flat[r];
            const int owner = f / args.scatter_rows_per_rank;
            my_row_ptr = reinterpret_cast<unsigned long long>(
                args.scatter_base[owner] + static_cast<size_t>(f - owner * args.scatter_rows_per_rank) * args.ldo);
          } else {
            my_row_ptr = reinterpret_cast<unsigned long long>(static_cast<uint16_t*>(args.out) +
                                                              static_cast<size_t>(r) * args.ldo);
          }
        }
      }
      if (!mbar_wait(smem_u32(&bars.acc_full), acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (stamp) Q4T_STAMP(2, tcount, 1);
      const bool valid = row < nrows;
      const bool warp_has_rows = quad * 32 < nrows;  // warp-uniform
      const size_t grow = static_cast<size_t>(row0 + row);
      const int n0 = nt * args.n_per_tile;            // first output column of this tile

      // ---- drain this warp's units into registers, then hand the accumulator
      // back to the MMA warp before doing any arithmetic on them
      // this warp's columns are consecutive: units [sub*kUnitsPerWarp, +kUnitsPerWarp)
      uint32_t ra[kUnitsPerWarp * 16];                 // store: the columns; SwiGLU: the gate columns
      uint32_t rb[kSwiglu ? kUnitsPerWarp * 16 : 16];  // SwiGLU: the matching up columns
      if (warp_has_rows) {
        const uint32_t c_first = static_cast<uint32_t>(sub * kUnitsPerWarp * kUnitCols);
        if constexpr (kUnitsPerWarp == 4) {
          tmem_ld64(tacc + c_first, ra);
        } else if constexpr (kUnitsPerWarp == 2) {
          tmem_ld32(tacc + c_first, ra);
          if constexpr (kSwiglu) tmem_ld32(tacc + kHalf + c_first, rb);
        } else {
#pragma unroll
          for (int j = 0; j < kUnitsPerWarp; ++j) {
            const int unit = sub * kUnitsPerWarp + j;
            if (unit < kUnits) {
              tmem_ld16(tacc + unit * kUnitCols, *reinterpret_cast<uint32_t (*)[16]>(&ra[j * 16]));
              if constexpr (kSwiglu)
                tmem_ld16(tacc + kHalf + unit * kUnitCols, *reinterpret_cast<uint32_t (*)[16]>(&rb[j * 16]));
            }
          }
        }
        tmem_ld_wait();
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty));
      if (stamp) Q4T_STAMP(2, tcount, 2);
      acc_phase ^= 1u;
      if (!warp_has_rows) continue;

      // ---- per unit: convert, compute, store (unit by unit keeps few registers live).
      // Rows past the tile's row count carry stale accumulator bits: they are
      // zeroed so the arithmetic below never meets NaNs or denormals.
      if constexpr (EPI == Epilogue::kStoreBf16Rows) {
        static_assert(kUnitsPerWarp == 4, "row-segment stores cover 64 columns per warp");
        // This warp's 64 columns are 128 bytes of each of its 32 rows.  Round to bf16 in
        // place, then pass the rows through the warp's staging block sixteen at a time
        // (one row per lane, 16-byte chunks XOR-swizzled against bank conflicts) and
        // read them back eight lanes per row, so that every store instruction writes
        // whole 128-byte row segments (full lines in L2, full packets to a peer GPU).
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float lo = valid ? alpha * __uint_as_float(ra[2 * i]) : 0.0f;
          const float hi = valid ? alpha * __uint_as_float(ra[2 * i + 1]) : 0.0f;
          ra[i] = f32x2_to_bf16x2(lo, hi);
        }
        const uint32_t stg = smem_base + kStages * kStage + static_cast<uint32_t>(warp - kFirstEpiWarp) * kStoreStageBytes;
        const uint32_t r16 = static_cast<uint32_t>(lane) & 15u;
        const uint32_t chunk = static_cast<uint32_t>(lane) & 7u;
        const int col = n0 + sub * (kUnitsPerWarp * kUnitCols) + static_cast<int>(chunk) * 8;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if ((lane >> 4) == half) {
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c)
              asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(stg + r16 * 128u + ((c ^ (r16 & 7u)) << 4)),
                           "r"(ra[4 * c]), "r"(ra[4 * c + 1]), "r"(ra[4 * c + 2]), "r"(ra[4 * c + 3]) : "memory");
          }
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t rs = (static_cast<uint32_t>(lane) >> 3) + 4u * i;  // row of the sixteen staged
            uint32_t v0, v1, v2, v3;
            asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                         : "r"(stg + rs * 128u + ((chunk ^ (rs & 7u)) << 4)) : "memory");
            // the lane that owns row rr of the quadrant holds its destination (0 past the tile's rows)
            const unsigned long long dst =
                __shfl_sync(0xffffffffu, my_row_ptr, half * 16 + static_cast<int>(rs));
            if (dst != 0 && col < args.b_rows_valid)
              *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dst) + col) = make_uint4(v0, v1, v2, v3);
          }
          __syncwarp();
        }
      } else {
#pragma unroll
      for (int j = 0; j < kUnitsPerWarp; ++j) {
        const int unit = sub * kUnitsPerWarp + j;
        if (unit >= kUnits) continue;
        const int c0 = unit * kUnitCols;
        if constexpr (EPI == Epilogue::kStoreF32) {
          if (valid && n0 + c0 < args.b_rows_valid) {
            float4* dst = reinterpret_cast<float4*>(static_cast<float*>(args.out) + grow * args.ldo + n0 + c0);
#pragma unroll
            for (int i = 0; i < 4; ++i)
              dst[i] = make_float4(alpha * __uint_as_float(ra[j * 16 + 4 * i]), alpha * __uint_as_float(ra[j * 16 + 4 * i + 1]),
                                   alpha * __uint_as_float(ra[j * 16 + 4 * i + 2]), alpha * __uint_as_float(ra[j * 16 + 4 * i + 3]));
          }
        } else {
          uint32_t gb[8];  // bf16x2 words of the 16 (gate) columns
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float lo = valid ? alpha * __uint_as_float(ra[j * 16 + 2 * i]) : 0.0f;
            const float hi = valid ? alpha * __uint_as_float(ra[j * 16 + 2 * i + 1]) : 0.0f;
            gb[i] = f32x2_to_bf16x2(lo, hi);
          }
          if constexpr (EPI == Epilogue::kStoreBf16) {
            // Two units (32 columns = 64 bytes per row) go through the warp's staging
            // block: written one row per lane (16-byte chunks, XOR-swizzled against bank
            // conflicts), read back four lanes per row, stored as 64-byte row segments.
            const uint32_t stg = smem_base + kStages * kStage + static_cast<uint32_t>(warp - kFirstEpiWarp) * kStoreStageBytes;
            const uint32_t sw = (static_cast<uint32_t>(lane) >> 1) & 3u;
            const uint32_t half = static_cast<uint32_t>(j & 1) * 2u;  // chunk pair of this unit inside the 64 bytes
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(stg + lane * 64u + ((half ^ sw) << 4)), "r"(gb[0]),
                         "r"(gb[1]), "r"(gb[2]), "r"(gb[3]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(stg + lane * 64u + (((half + 1u) ^ sw) << 4)),
                         "r"(gb[4]), "r"(gb[5]), "r"(gb[6]), "r"(gb[7]) : "memory");
            if ((j & 1) == 1 || j == kUnitsPerWarp - 1) {
              __syncwarp();
              const bool pair = (j & 1) == 1;                        // a lone last unit stages 16 columns
              const int cbase = (pair ? unit - 1 : unit) * kUnitCols;  // first column of what is staged
              const uint32_t chunk = static_cast<uint32_t>(lane) & 3u;
              const int ncols = (pair ? 2 : 1) * kUnitCols;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int rr = (lane >> 2) + 8 * i;                  // row of the warp's 32
                const uint32_t rsw = (static_cast<uint32_t>(rr) >> 1) & 3u;
                uint32_t v0, v1, v2, v3;
                asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v0), "=r"(v1), "=r"(v2), "=r"(v3)
                             : "r"(stg + rr * 64u + ((chunk ^ rsw) << 4)) : "memory");
                const int col = n0 + cbase + static_cast<int>(chunk) * 8;
                if (quad * 32 + rr < nrows && static_cast<int>(chunk) * 8 < ncols && col < args.b_rows_valid)
                  *reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) +
                                            static_cast<size_t>(row0 + quad * 32 + rr) * args.ldo + col) =
                      make_uint4(v0, v1, v2, v3);
              }
              __syncwarp();
            }
          } else {
            uint32_t ub[8];  // the 16 matching up columns
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float lo = valid ? alpha * __uint_as_float(rb[j * 16 + 2 * i]) : 0.0f;
              const float hi = valid ? alpha * __uint_as_float(rb[j * 16 + 2 * i + 1]) : 0.0f;
              ub[i] = f32x2_to_bf16x2(lo, hi);
            }
            if (args.gu_dump && valid) {
              uint4* dg = reinterpret_cast<uint4*>(args.gu_dump + grow * args.gu_dump_ld + n0 + c0);
              dg[0] = make_uint4(gb[0], gb[1], gb[2], gb[3]);
              dg[1] = make_uint4(gb[4], gb[5], gb[6], gb[7]);
              uint4* du = reinterpret_cast<uint4*>(args.gu_dump + grow * args.gu_dump_ld + args.up_row_offset + n0 + c0);
              du[0] = make_uint4(ub[0], ub[1], ub[2], ub[3]);
              du[1] = make_uint4(ub[4], ub[5], ub[6], ub[7]);
            }
            // SwiGLU on the bf16-rounded projections: (g * sigmoid(g)) * u
            // sigmoid(g) = 1 / (1 + __expf(-g)) with IEEE division, as the reference
            // computes it.  The denominators are >= 1, so the branch-free reciprocal
            // gives the same bits unless one of them reaches 2^126 (g below about -87),
            // in which case the whole unit takes the IEEE routine.
            float a[16];  // first the sigmoid denominators, then the SwiGLU values
            bool big = false;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              a[2 * i] = 1.0f + __expf(-bf16x2_lo(gb[i]));
              a[2 * i + 1] = 1.0f + __expf(-bf16x2_hi(gb[i]));
              big |= !(a[2 * i] < Q4T_RCP_FAST_MAX) | !(a[2 * i + 1] < Q4T_RCP_FAST_MAX);
            }
            const bool slow = __any_sync(0xffffffffu, big);
#pragma unroll
            for (int h = 0; h < 2; ++h) {  // two halves of eight keep the live set small
#pragma unroll
              for (int i = 4 * h; i < 4 * h + 4; ++i) {
                const float s0 = slow ? __frcp_rn(a[2 * i]) : rcp_rn_ge1(a[2 * i]);
                const float s1 = slow ? __frcp_rn(a[2 * i + 1]) : rcp_rn_ge1(a[2 * i + 1]);
                a[2 * i] = (bf16x2_lo(gb[i]) * s0) * bf16x2_lo(ub[i]);
                a[2 * i + 1] = (bf16x2_hi(gb[i]) * s1) * bf16x2_hi(ub[i]);
              }
            }
            if constexpr (EPI == Epilogue::kSwigluBf16) {
              if (valid) {
                uint32_t o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = f32x2_to_bf16x2(a[2 * i], a[2 * i + 1]);
                uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) + grow * args.ldo + n0 + c0);
                dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
              }
            } else {
              const uint32_t out_ntk = (static_cast<uint32_t>(args.up_row_offset) + 63u) >> 6;
              uint32_t lo, hi;
              const uint32_t sf = quantize_group16(a, next_scale, lo, hi);
              if (valid) {
                *reinterpret_cast<uint2*>(static_cast<uint8_t*>(args.out) + grow * args.ldo + ((n0 + c0) >> 1)) =
                    make_uint2(lo, hi);
                const uint32_t g = static_cast<uint32_t>(n0 + c0) >> 4;  // scale group along the intermediate
                args.out_sf_tiles[(static_cast<size_t>(mt) * out_ntk + (g >> 2)) * 512u + sf_in_atom(row, g)] =
                    static_cast<uint8_t>(sf);
              }
            }
          }
        }
      }
      }  // per-unit epilogues
      if (stamp) Q4T_STAMP(2, tcount, 3);
    }
    if (!ok && args.status && lane == 0) atomicMax(args.status, 3);
    (void)stamp;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <bool NVF4, int BN>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, Epilogue epi,
                   int num_sms, cudaStream_t stream) {
  const size_t smem = num_stages<NVF4>() * stage_bytes<NVF4, BN>() + kEpiWarps * kStoreStageBytes + 1024;
  const int grid = a.ntiles_dev ? num_sms : min(num_sms, a.ntiles_host * a.n_tiles);
  if (grid <= 0) return cudaSuccess;
  switch (epi) {
    case Epilogue::kStoreBf16:
      return launch_chained(gemm_kernel<NVF4, Epilogue::kStoreBf16, BN>, dim3(grid), dim3(kThreads), smem, stream, ta, tb, a);
    case Epilogue::kStoreF32:
      return launch_chained(gemm_kernel<NVF4, Epilogue::kStoreF32, BN>, dim3(grid), dim3(kThreads), smem, stream, ta, tb, a);
    case Epilogue::kSwigluBf16:
      return launch_chained(gemm_kernel<NVF4, Epilogue::kSwigluBf16, BN>, dim3(grid), dim3(kThreads), smem, stream, ta, tb, a);
    case Epilogue::kSwigluQuant:
      if constexpr (NVF4) {
        return launch_chained(gemm_kernel<NVF4, Epilogue::kSwigluQuant, BN>, dim3(grid), dim3(kThreads), smem, stream, ta, tb, a);
      } else {
        return cudaErrorInvalidValue;
      }
    case Epilogue::kStoreBf16Rows:
      if constexpr (NVF4) {
        return launch_chained(gemm_kernel<NVF4, Epilogue::kStoreBf16Rows, BN>, dim3(grid), dim3(kThreads), smem, stream, ta, tb, a);
      } else {
        return cudaErrorInvalidValue;
      }
  }
  return cudaGetLastError();
}

template <bool NVF4, Epilogue E, int BN>
cudaError_t set_attr() {
  return cudaFuncSetAttribute(gemm_kernel<NVF4, E, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(num_stages<NVF4>() * stage_bytes<NVF4, BN>() + kEpiWarps * kStoreStageBytes + 1024));
}

}  // namespace

cudaError_t gemm_set_attributes() {
  cudaError_t e;
  if ((e = set_attr<true, Epilogue::kStoreBf16, 256>()) != cudaSuccess) return e;
  if ((e = set_attr<true, Epilogue::kStoreF32, 256>()) != cudaSuccess) return e;
  if ((e = set_attr<true, Epilogue::kSwigluBf16, 256>()) != cudaSuccess) return e;
  if ((e = set_attr<true, Epilogue::kSwigluQuant, 256>()) != cudaSuccess) return e;
  if ((e = set_attr<true, Epilogue::kStoreBf16Rows, 256>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kStoreBf16, 256>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kStoreF32, 256>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kSwigluBf16, 256>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kStoreBf16, 64>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kStoreF32, 64>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kSwigluBf16, 64>()) != cudaSuccess) return e;
  return cudaSuccess;
}

cudaError_t launch_gemm_nvf4(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a,
                             Epilogue epi, int num_sms, cudaStream_t stream) {
  return launch<true, 256>(ta, tb, a, epi, num_sms, stream);
}

cudaError_t launch_gemm_bf16(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a,
                             Epilogue epi, int num_sms, cudaStream_t stream) {
  if (a.tile_cols == 64) return launch<false, 64>(ta, tb, a, epi, num_sms, stream);
  return launch<false, 256>(ta, tb, a, epi, num_sms, stream);
}

}  // namespace q4t
