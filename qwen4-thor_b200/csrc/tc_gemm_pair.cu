// The CTA-pair form of the tensor-core GEMMs (tcgen05 cta_group::2).
//
// Two CTAs of a cluster (neighbouring SMs) share one 256-row x 256-column tile: each CTA
// loads its own 128 rows of A and HALF of the B tile with its own plain TMA loads (nothing
// is multicast), the leader CTA issues one set of scale copies and 256-row MMAs for both,
// and each CTA drains its own 128 accumulator rows.  Row tiles 2j and 2j+1 of the tile
// list form a pair and must belong to the same expert (the planner pads every expert to an
// even tile count).  Roles, barriers and epilogues are those of the single-CTA kernel in
// tc_gemm.cu; the two differ in who signals whom:
//   full[s]    lives in the leader; both CTAs' TMA loads complete on it;
//   empty[s]   one per CTA, signalled by the leader's tcgen05.commit to both;
//   acc_full   one per CTA, signalled the same way;
//   acc_empty  lives in the leader; the epilogue warps of both CTAs arrive on it.
//
// Measured on B200 (dense 163840 x 1024 x 2048 and the 16 K-token layer): this form is
// 5-10 % SLOWER than one CTA per tile.  The block-scaled mainloop is bound by the per-SM
// tensor pipe (the MMAs plus three scale copies per MMA, which every SM of a pair still
// executes), not by the L2 -> SM operand traffic a pair halves: leaving out half of the B
// loads of the single-CTA kernel gains 5 %, leaving out the scale copies 30 %.  It is
// therefore off unless q4t_set_pair_min_rows() / Q4T_PAIR_MIN_ROWS asks for it.
#include "kernels.h"
#include "q4t_device.cuh"

namespace q4t {

namespace {

constexpr int kMaxStages = 6;
// Shared-memory ring depth.  Three 54 KB stages measured faster than four for the
// block-scaled tiles (decode gate/up 101 vs 108 us); the BF16 tiles keep four.
template <bool NVF4, bool PAIR>
constexpr int num_stages() {
  return PAIR ? (NVF4 ? 5 : 6) : (NVF4 ? 3 : 4);
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

// A pair CTA stages only its half of the B tile.
template <bool NVF4, int BN, bool PAIR>
constexpr uint32_t stage_bytes() {
  return kABytes + (PAIR ? BN * 64 : BN * 128) + (NVF4 ? kSfaBytes + kSfbBytes : 0u);
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
// The kernel parameters are used in place (never through a reference): parameters whose
// address escapes are read with generic loads instead of as constant-bank operands, which
// cost the single-CTA kernel 10-15 % when this body was a function called by two wrappers.
// tmap_sfa / tmap_sfb are only read by the block-scaled CTA-pair form.
template <bool NVF4, Epilogue EPI, int BN, bool PAIR>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a_, const __grid_constant__ CUtensorMap tmap_b_,
            const __grid_constant__ CUtensorMap tmap_sfa_, const __grid_constant__ CUtensorMap tmap_sfb_,
            const __grid_constant__ GemmArgs args) {
  const CUtensorMap* const tmap_a = &tmap_a_;
  const CUtensorMap* const tmap_b = &tmap_b_;
  [[maybe_unused]] const CUtensorMap* const tmap_sfa = &tmap_sfa_;
  [[maybe_unused]] const CUtensorMap* const tmap_sfb = &tmap_sfb_;
  static_assert(!NVF4 || BN == 256, "block-scaled tiles are 256 columns wide");
  static_assert(!PAIR || BN == 256, "pair tiles are 256 columns wide");
  extern __shared__ uint8_t smem_raw[];
  __shared__ Barriers bars;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr uint32_t kBBytes = PAIR ? BN * 64 : BN * 128;  // B bytes this CTA stages per k-block
  constexpr uint32_t kStage = stage_bytes<NVF4, BN, PAIR>();
  constexpr int kStages = num_stages<NVF4, PAIR>();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &bars.abort_flag;
  // pair mode: rank 0 of the cluster issues the MMAs and owns the "full" and "accumulator
  // empty" barriers; rank 1 stages its operand halves and drains its own accumulator rows
  const uint32_t cta_rank = PAIR ? cluster_cta_rank() : 0u;
  const bool leader = cta_rank == 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    mbar_init(smem_u32(&bars.acc_full), 1);
    mbar_init(smem_u32(&bars.acc_empty), PAIR ? 2 * kEpiWarps : kEpiWarps);
    bars.abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(tmap_a);
    prefetch_tmap(tmap_b);
    if constexpr (PAIR && NVF4) {
      prefetch_tmap(tmap_sfa);
      prefetch_tmap(tmap_sfb);
    }
  }
  if (warp == 1) {
    if constexpr (PAIR) {
      tmem_alloc_pair(smem_u32(&bars.tmem_base), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(&bars.tmem_base), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (PAIR) cluster_sync(); else __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;
  // Barriers, tensor memory and descriptors are set up (possibly while the previous kernel
  // of the stream was still draining); from here on the kernel reads what that kernel wrote.
  chain_wait();

  const int m_tiles = args.ntiles_dev ? *args.ntiles_dev : args.ntiles_host;
  // pair mode walks pairs of row tiles: CTA rank r of a pair works on row tile 2j + r
  const int total_tiles = (PAIR ? (m_tiles + 1) >> 1 : m_tiles) * args.n_tiles;
  const int tile_first = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int tile_step = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  // (the helpers below capture copies of what they need: a kernel parameter captured by
  // reference would be read through generic loads)
  const int n_tiles = args.n_tiles;
  const int32_t* const tile_expert = args.tile_expert;
  const int32_t* const tile_row0 = args.tile_row0;
  auto row_tile_of = [=](int tile) { return PAIR ? 2 * (tile / n_tiles) + static_cast<int>(cta_rank) : tile / n_tiles; };
  // a pair's second row tile may lie past the end of a dense problem: it loads zeros and stores nothing
  auto tile_exists = [=](int mt) { return !PAIR || mt < m_tiles; };
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
      // pair mode: both CTAs' loads complete on the leader's "full" barriers
      const uint32_t bar_full_sig0 = PAIR ? cluster_map(bar_full0, 0) : bar_full0;
      // The expert and first row of a tile are fetched one tile ahead: with short tiles (two
      // k-blocks in the down GEMM) a table lookup in front of every tile's first load would
      // leave the ring short of requests for the length of an L2 round trip.
      int next_group = 0, next_row0 = 0;
      if (tile_first < total_tiles) {
        const int mt0 = row_tile_of(tile_first);
        const bool ex = tile_exists(mt0);
        next_group = (args.tile_expert && ex) ? args.tile_expert[mt0] : 0;
        next_row0 = (args.tile_expert && ex) ? args.tile_row0[mt0] : mt0 * kTileM;
      }
      for (int tile = tile_first; tile < total_tiles && ok; tile += tile_step) {
        const int mt = row_tile_of(tile), nt = tile - (tile / args.n_tiles) * args.n_tiles;
        const int group = next_group, row0 = next_row0;
        if (tile + tile_step < total_tiles) {
          const int nmt = row_tile_of(tile + tile_step);
          const bool ex = tile_exists(nmt);
          next_group = (args.tile_expert && ex) ? args.tile_expert[nmt] : 0;
          next_row0 = (args.tile_expert && ex) ? args.tile_row0[nmt] : nmt * kTileM;
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
        // pair mode addresses the scale atoms through tensor maps (atom index = coordinate 1)
        [[maybe_unused]] int atom_a = mt * static_cast<int>(ntk);
        [[maybe_unused]] int atom_b0 = group * args.sfb_group_atoms + static_cast<int>(rb0 * ntk);
        [[maybe_unused]] int atom_b1 = group * args.sfb_group_atoms + static_cast<int>(rb1 * ntk);
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
          if constexpr (PAIR) {
            // Both CTAs stage A (own rows), their half of B, their own A scales and all of
            // the B scales; the leader announces the bytes of both.  Scale boxes are always
            // four atoms (a short last k-block reads atoms it does not use).
            const uint32_t sig = bar_full_sig0 + stage * 8u;
            if (leader) {
              uint32_t tx = kABytes + kBBytes;
              if (NVF4) tx += kSfaBytes + (second_half ? kSfbBytes : kSfbBytes / 2);
              mbar_expect_tx(full, 2u * tx);
            }
            tma_load_2d_pair(sa, tmap_a, kc, row0, sig);
            tma_load_2d_pair(sb, tmap_b, kc, leader ? brow0 : brow1, sig);
            if constexpr (NVF4) {
              const uint32_t ssfa = sb + kBBytes, ssfb = ssfa + kSfaBytes;
              tma_load_2d_pair(ssfa, tmap_sfa, 0, atom_a, sig);
              tma_load_2d_pair(ssfb, tmap_sfb, 0, atom_b0, sig);
              if (second_half) tma_load_2d_pair(ssfb + kSfbBytes / 2, tmap_sfb, 0, atom_b1, sig);
              atom_a += 4;
              atom_b0 += 4;
              atom_b1 += 4;
            }
          } else {
            uint32_t tx = kABytes + kBBytes;
            if (NVF4) tx += nm * 512u * (second_half ? 3u : 2u);
            mbar_expect_tx(full, tx);
            tma_load_2d(sa, tmap_a, kc, row0, full);
            tma_load_2d(sb, tmap_b, kc, brow0, full);            // box = kHalf rows
            tma_load_2d(sb + kBBytes / 2, tmap_b, kc, brow1, full);
            if (NVF4) {
              const uint32_t ssfa = sb + kBBytes, ssfb = ssfa + kSfaBytes;
              bulk_load(ssfa, ga, nm * 512u, full);
              bulk_load(ssfb, gb0, nm * 512u, full);
              if (second_half) bulk_load(ssfb + kSfbBytes / 2, gb1, nm * 512u, full);
              ga += 2048;
              gb0 += 2048;
              gb1 += 2048;
            }
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
    if (lane == 0 && leader) {
      // instruction descriptors (M = 128, or 256 over a CTA pair; N = BN; both operands K-major)
      constexpr uint32_t kM = PAIR ? 256u : 128u;
      constexpr uint32_t idesc_nvf4 =
          (1u << 7) | (1u << 10) | ((static_cast<uint32_t>(BN) >> 3) << 17) | ((kM >> 4) << 24);
      constexpr uint32_t idesc_bf16 = (1u << 4) | (1u << 7) | (1u << 10) |
                                      ((static_cast<uint32_t>(BN) >> 3) << 17) | ((kM >> 4) << 24);
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
      // The single issuing thread must spend next to nothing between tcgen05 instructions, so
      // the pair / single forms are chosen by the preprocessor-like helpers below, not at run time.
#define Q4T_CP_SF(taddr, sdesc)                                            \
  do {                                                                     \
    if constexpr (PAIR) tc_cp_sf_pair(taddr, sdesc); else tc_cp_sf(taddr, sdesc); \
  } while (0)
#define Q4T_MMA_NVF4(ad, bd, sfa_t, sfb_t, acc)                                             \
  do {                                                                                      \
    if constexpr (PAIR) tc_mma_nvf4_pair(tmem, ad, bd, idesc_nvf4, sfa_t, sfb_t, acc);      \
    else tc_mma_nvf4(tmem, ad, bd, idesc_nvf4, sfa_t, sfb_t, acc);                          \
  } while (0)
#define Q4T_MMA_F16(ad, bd, acc)                                         \
  do {                                                                   \
    if constexpr (PAIR) tc_mma_f16_pair(tmem, ad, bd, idesc_bf16, acc);  \
    else tc_mma_f16(tmem, ad, bd, idesc_bf16, acc);                      \
  } while (0)
  // in pair mode the completion is signalled to the same barrier of both CTAs
#define Q4T_COMMIT(bar)                                            \
  do {                                                             \
    if constexpr (PAIR) tc_commit_pair(bar, 3); else tc_commit(bar); \
  } while (0)
      int tcount = 0;
      for (int tile = tile_first; tile < total_tiles && ok; tile += tile_step, ++tcount) {
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
                Q4T_CP_SF(tsf + kk * 4u, sfa + kk * 32u);
                Q4T_CP_SF(tsf + 16u + kk * 8u, sfb + kk * 32u);
                Q4T_CP_SF(tsf + 20u + kk * 8u, sfb + (kSfbBytes / 32) + kk * 32u);
              }
#pragma unroll
              for (uint32_t kk = 0; kk < 4; ++kk)
                Q4T_MMA_NVF4(adesc + kk * 2u, bdesc + kk * 2u, tsf + kk * 4u, tsf + 16u + kk * 8u, kk == 0 ? first : 1u);
            } else {
              const uint32_t nm = k_left >> 5;
              for (uint32_t kk = 0; kk < nm; ++kk) {
                Q4T_CP_SF(tsf + kk * 4u, sfa + kk * 32u);
                Q4T_CP_SF(tsf + 16u + kk * 8u, sfb + kk * 32u);
                Q4T_CP_SF(tsf + 20u + kk * 8u, sfb + (kSfbBytes / 32) + kk * 32u);
              }
              for (uint32_t kk = 0; kk < nm; ++kk)
                Q4T_MMA_NVF4(adesc + kk * 2u, bdesc + kk * 2u, tsf + kk * 4u, tsf + 16u + kk * 8u, kk == 0 ? first : 1u);
            }
          } else {
            if (k_left >= 128u) {
#pragma unroll
              for (uint32_t kk = 0; kk < 4; ++kk) Q4T_MMA_F16(adesc + kk * 2u, bdesc + kk * 2u, kk == 0 ? first : 1u);
            } else {
              const uint32_t nm = k_left >> 5;
              for (uint32_t kk = 0; kk < nm; ++kk) Q4T_MMA_F16(adesc + kk * 2u, bdesc + kk * 2u, kk == 0 ? first : 1u);
            }
          }
          Q4T_COMMIT(bar_empty0 + stage * 8u);  // frees the stage once these MMAs have read it
          k_left -= 128u;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) Q4T_COMMIT(bar_acc_full);
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
    // pair mode: the leader's MMA thread waits for the epilogue warps of both CTAs
    const uint32_t bar_acc_empty_sig = PAIR ? cluster_map(smem_u32(&bars.acc_empty), 0) : smem_u32(&bars.acc_empty);
    for (int tile = tile_first; tile < total_tiles && ok; tile += tile_step, ++tcount) {
      const int mt = row_tile_of(tile), nt = tile - (tile / n_tiles) * n_tiles;
      const bool exists = tile_exists(mt);
      const int group = (args.tile_expert && exists) ? args.tile_expert[mt] : 0;
      const int row0 = (args.tile_expert && exists) ? args.tile_row0[mt] : mt * kTileM;
      if (stamp) Q4T_STAMP(2, tcount, 0);
      const int nrows = !exists ? 0 : args.tile_expert ? args.tile_nrows[mt] : min(kTileM, args.total_rows - row0);
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
      if (lane == 0) {
        if constexpr (PAIR) mbar_arrive_cluster(bar_acc_empty_sig); else mbar_arrive(bar_acc_empty_sig);
      }
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
  // pair mode: neither CTA may release its tensor memory (or exit, taking its shared
  // memory and barriers with it) while the other can still touch them
  if constexpr (PAIR) cluster_sync(); else __syncthreads();
  if (warp == 1) {
    __syncwarp();
    if constexpr (PAIR) tmem_dealloc_pair(tmem, kTmemCols); else tmem_dealloc(tmem, kTmemCols);
  }
}

template <bool NVF4, int BN>
constexpr size_t smem_bytes(bool pair) {
  return (pair ? num_stages<NVF4, true>() * stage_bytes<NVF4, BN, true>()
               : num_stages<NVF4, false>() * stage_bytes<NVF4, BN, false>()) +
         kEpiWarps * kStoreStageBytes + 1024;
}

// CTA pairs that can be resident at once (set by gemm_pair_set_attributes; clusters of two need
// both SMs of a pair free, so this may be less than half the SM count).
int g_max_pairs[16] = {};

template <bool NVF4>
cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                        const GemmArgs& a, Epilogue epi, int num_sms, cudaStream_t stream) {
  const size_t smem = smem_bytes<NVF4, 256>(true);
  int dev = 0;
  cudaGetDevice(&dev);
  int pairs = num_sms / 2;
  if (dev >= 0 && dev < 16 && g_max_pairs[dev] > 0) pairs = min(pairs, g_max_pairs[dev]);
  if (!a.ntiles_dev) pairs = min(pairs, ((a.ntiles_host + 1) / 2) * a.n_tiles);
  if (pairs <= 0) return cudaSuccess;
  const dim3 grid(2 * pairs), block(kThreads);
  switch (epi) {
    case Epilogue::kStoreBf16:
      return launch_chained_cluster(gemm_pair_kernel<NVF4, Epilogue::kStoreBf16, 256, true>, grid, block, smem, stream, 2, ta, tb, tsa, tsb, a);
    case Epilogue::kStoreF32:
      return launch_chained_cluster(gemm_pair_kernel<NVF4, Epilogue::kStoreF32, 256, true>, grid, block, smem, stream, 2, ta, tb, tsa, tsb, a);
    case Epilogue::kSwigluBf16:
      if constexpr (!NVF4) {
        return launch_chained_cluster(gemm_pair_kernel<NVF4, Epilogue::kSwigluBf16, 256, true>, grid, block, smem, stream, 2, ta, tb, tsa, tsb, a);
      } else {
        return cudaErrorInvalidValue;
      }
    case Epilogue::kSwigluQuant:
      if constexpr (NVF4) {
        return launch_chained_cluster(gemm_pair_kernel<NVF4, Epilogue::kSwigluQuant, 256, true>, grid, block, smem, stream, 2, ta, tb, tsa, tsb, a);
      } else {
        return cudaErrorInvalidValue;
      }
    case Epilogue::kStoreBf16Rows:
      if constexpr (NVF4) {
        return launch_chained_cluster(gemm_pair_kernel<NVF4, Epilogue::kStoreBf16Rows, 256, true>, grid, block, smem, stream, 2, ta, tb, tsa, tsb, a);
      } else {
        return cudaErrorInvalidValue;
      }
  }
  return cudaGetLastError();
}

template <bool NVF4, Epilogue E>
cudaError_t set_attr_pair() {
  return cudaFuncSetAttribute(gemm_pair_kernel<NVF4, E, 256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(smem_bytes<NVF4, 256>(true)));
}

}  // namespace

cudaError_t gemm_pair_set_attributes() {
  cudaError_t e;
  if ((e = set_attr_pair<true, Epilogue::kStoreBf16>()) != cudaSuccess) return e;
  if ((e = set_attr_pair<true, Epilogue::kStoreF32>()) != cudaSuccess) return e;
  if ((e = set_attr_pair<true, Epilogue::kSwigluQuant>()) != cudaSuccess) return e;
  if ((e = set_attr_pair<true, Epilogue::kStoreBf16Rows>()) != cudaSuccess) return e;
  if ((e = set_attr_pair<false, Epilogue::kStoreBf16>()) != cudaSuccess) return e;
  if ((e = set_attr_pair<false, Epilogue::kStoreF32>()) != cudaSuccess) return e;
  if ((e = set_attr_pair<false, Epilogue::kSwigluBf16>()) != cudaSuccess) return e;
  // how many CTA pairs fit on the device at once
  int dev = 0;
  if ((e = cudaGetDevice(&dev)) != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(2);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem_bytes<true, 256>(true);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<true, Epilogue::kSwigluQuant, 256, true>, &cfg) == cudaSuccess &&
      clusters > 0 && dev >= 0 && dev < 16)
    g_max_pairs[dev] = clusters;
  else
    cudaGetLastError();  // the query is advisory: fall back to half the SM count
  return cudaSuccess;
}

cudaError_t launch_gemm_nvf4_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa,
                                  const CUtensorMap& tsb, const GemmArgs& a, Epilogue epi, int num_sms,
                                  cudaStream_t stream) {
  return launch_pair<true>(ta, tb, tsa, tsb, a, epi, num_sms, stream);
}

cudaError_t launch_gemm_bf16_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, Epilogue epi,
                                  int num_sms, cudaStream_t stream) {
  return launch_pair<false>(ta, tb, ta, tb, a, epi, num_sms, stream);  // the scale maps are not read
}

}  // namespace q4t
