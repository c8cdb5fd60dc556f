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
// Warp roles (256 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM
// owner, warps 4..7 = epilogue (warp w reads TMEM lanes 32*(w%4)..+31, i.e.
// one output row per thread).  Stages hand over through mbarriers; every wait
// is bounded and raises a status word instead of spinning forever.
//
// A tile's 256 accumulator columns are either 256 consecutive output columns
// or, for the SwiGLU epilogues, 128 gate columns followed by the 128 matching
// up columns, so that one thread sees g and u of the same output element.
#include "kernels.h"
#include "q4t_device.cuh"

namespace q4t {

namespace {

constexpr int kStages = 4;
constexpr int kThreads = 256;
constexpr uint32_t kABytes = 128 * 128;       // 128 rows x 128 bytes
constexpr uint32_t kBBytes = 256 * 128;       // 256 rows x 128 bytes
constexpr uint32_t kSfaBytes = 4 * 512;       // 4 atoms (one per MMA of a k-block)
constexpr uint32_t kSfbBytes = 8 * 512;       // 2 x 4 atoms
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSfTmemBase = 256;         // scale columns start after the accumulator
constexpr uint32_t kSfTmemPerStage = 48;      // 16 (A) + 32 (B)

template <bool NVF4>
constexpr uint32_t stage_bytes() {
  return kABytes + kBBytes + (NVF4 ? kSfaBytes + kSfbBytes : 0u);
}

struct Barriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t acc_full;
  uint64_t acc_empty;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

__device__ __forceinline__ float sigmoid_ref(float g) { return __frcp_rn(1.0f + __expf(-g)); }

template <bool NVF4, Epilogue EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ Barriers bars;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  constexpr uint32_t kStage = stage_bytes<NVF4>();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &bars.abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    mbar_init(smem_u32(&bars.acc_full), 1);
    mbar_init(smem_u32(&bars.acc_empty), 4);
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

  const int m_tiles = args.ntiles_dev ? *args.ntiles_dev : args.ntiles_host;
  const int total_tiles = m_tiles * args.n_tiles;
  constexpr bool kSwiglu = (EPI == Epilogue::kSwigluBf16 || EPI == Epilogue::kSwigluQuant);
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
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mt = tile / args.n_tiles, nt = tile - mt * args.n_tiles;
        const int group = args.tile_expert ? args.tile_expert[mt] : 0;
        const int row0 = args.tile_expert ? args.tile_row0[mt] : mt * kTileM;
        const int brow0 = group * args.b_rows_per_group + nt * args.n_per_tile;
        const int brow1 = brow0 + (kSwiglu ? args.up_row_offset : 128);
        // scale atoms of B: row blocks of 128 inside the group's buffer
        const uint32_t rb0 = static_cast<uint32_t>(nt * args.n_per_tile) >> 7;
        const uint32_t rb1 = rb0 + (kSwiglu ? static_cast<uint32_t>(args.up_row_offset) >> 7 : 1u);
        const bool second_half = kSwiglu || (nt * args.n_per_tile + 128 < args.b_rows_valid);
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(smem_u32(&bars.empty[stage]), phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t nm = min(4u, (k_bytes - static_cast<uint32_t>(kb) * 128u) >> 5);
          const uint32_t sa = smem_base + stage * kStage, sb = sa + kABytes;
          const uint32_t full = smem_u32(&bars.full[stage]);
          uint32_t tx = kABytes + kBBytes;
          if (NVF4) tx += nm * 512u * (second_half ? 3u : 2u);
          mbar_expect_tx(full, tx);
          const int kc = kb * (NVF4 ? 128 : 64);  // inner coordinate in tensor-map elements
          tma_load_2d(sa, &tmap_a, kc, row0, full);
          tma_load_2d(sb, &tmap_b, kc, brow0, full);
          tma_load_2d(sb + kBBytes / 2, &tmap_b, kc, brow1, full);
          if (NVF4) {
            const uint32_t ssfa = sb + kBBytes, ssfb = ssfa + kSfaBytes;
            const uint8_t* ga = args.sfa_tiles + (static_cast<size_t>(mt) * ntk + kb * 4u) * 512u;
            const uint8_t* gb = args.sfb + static_cast<size_t>(group) * args.sfb_group_stride;
            bulk_load(ssfa, ga, nm * 512u, full);
            bulk_load(ssfb, gb + (static_cast<size_t>(rb0) * ntk + kb * 4u) * 512u, nm * 512u, full);
            if (second_half)
              bulk_load(ssfb + kSfbBytes / 2, gb + (static_cast<size_t>(rb1) * ntk + kb * 4u) * 512u,
                        nm * 512u, full);
          }
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
      // instruction descriptors (M = 128, N = 256, both operands K-major)
      constexpr uint32_t idesc_nvf4 = (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
      constexpr uint32_t idesc_bf16 =
          (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(smem_u32(&bars.acc_empty), acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < nkb; ++kb) {
          if (!mbar_wait(smem_u32(&bars.full[stage]), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t nm = min(4u, (k_bytes - static_cast<uint32_t>(kb) * 128u) >> 5);
          const uint32_t sa = smem_base + stage * kStage, sb = sa + kABytes;
          const uint64_t adesc = umma_desc_sw128(sa), bdesc = umma_desc_sw128(sb);
          if (NVF4) {
            const uint32_t ssfa = sb + kBBytes, ssfb = ssfa + kSfaBytes;
            const uint32_t tsf = tmem + kSfTmemBase + stage * kSfTmemPerStage;
            for (uint32_t kk = 0; kk < nm; ++kk) {
              tc_cp_sf(tsf + kk * 4u, umma_desc_sf(ssfa + kk * 512u));
              tc_cp_sf(tsf + 16u + kk * 8u, umma_desc_sf(ssfb + kk * 512u));
              tc_cp_sf(tsf + 16u + kk * 8u + 4u, umma_desc_sf(ssfb + kSfbBytes / 2 + kk * 512u));
            }
            for (uint32_t kk = 0; kk < nm; ++kk)
              tc_mma_nvf4(tmem, adesc + kk * 2u, bdesc + kk * 2u, idesc_nvf4, tsf + kk * 4u,
                          tsf + 16u + kk * 8u, (kb | static_cast<int>(kk)) != 0);
          } else {
            for (uint32_t kk = 0; kk < nm; ++kk)
              tc_mma_f16(tmem, adesc + kk * 2u, bdesc + kk * 2u, idesc_bf16,
                         (kb | static_cast<int>(kk)) != 0);
          }
          tc_commit(smem_u32(&bars.empty[stage]));  // frees the stage once these MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(smem_u32(&bars.acc_full));
        acc_phase ^= 1u;
      }
      if (!ok && args.status) atomicMax(args.status, 2);
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t tacc = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const int mt = tile / args.n_tiles, nt = tile - mt * args.n_tiles;
      const int group = args.tile_expert ? args.tile_expert[mt] : 0;
      const int row0 = args.tile_expert ? args.tile_row0[mt] : mt * kTileM;
      const int nrows = args.tile_expert ? args.tile_nrows[mt] : min(kTileM, args.total_rows - row0);
      const float alpha =
          args.alpha_w ? args.alpha_w[group] * args.alpha_a[group] : args.alpha_const;
      if (!mbar_wait(smem_u32(&bars.acc_full), acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const bool valid = row < nrows;
      const size_t grow = static_cast<size_t>(row0 + row);
      if (quad * 32 < nrows) {  // warp-uniform: skip quadrants without rows
        if constexpr (!kSwiglu) {
          const int n0 = nt * 256;
#pragma unroll 1
          for (int c0 = 0; c0 < 256; c0 += 16) {
            if (n0 + c0 >= args.b_rows_valid) break;  // uniform
            uint32_t r[16];
            tmem_ld16(tacc + c0, r);
            tmem_ld_wait();
            if (valid) {
              if constexpr (EPI == Epilogue::kStoreBf16) {
                uint32_t o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  o[j] = f32x2_to_bf16x2(alpha * __uint_as_float(r[2 * j]),
                                         alpha * __uint_as_float(r[2 * j + 1]));
                uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) +
                                                      grow * args.ldo + n0 + c0);
                dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
              } else {
                float4* dst = reinterpret_cast<float4*>(static_cast<float*>(args.out) +
                                                        grow * args.ldo + n0 + c0);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  dst[j] = make_float4(alpha * __uint_as_float(r[4 * j]),
                                       alpha * __uint_as_float(r[4 * j + 1]),
                                       alpha * __uint_as_float(r[4 * j + 2]),
                                       alpha * __uint_as_float(r[4 * j + 3]));
              }
            }
          }
        } else {
          const int n0 = nt * 128;  // first intermediate column of this tile
          float next_scale = 1.0f;
          if constexpr (EPI == Epilogue::kSwigluQuant) next_scale = args.next_scale[group];
          const uint32_t out_ntk = (static_cast<uint32_t>(args.up_row_offset) + 63u) >> 6;
          uint32_t sf_word = 0;
#pragma unroll 1
          for (int c0 = 0; c0 < 128; c0 += 16) {
            uint32_t rg[16], ru[16];
            tmem_ld16(tacc + c0, rg);
            tmem_ld16(tacc + 128 + c0, ru);
            tmem_ld_wait();
            // the reference rounds the projection output to bf16 before SwiGLU
            uint32_t gb[8], ub[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              gb[j] = f32x2_to_bf16x2(alpha * __uint_as_float(rg[2 * j]),
                                      alpha * __uint_as_float(rg[2 * j + 1]));
              ub[j] = f32x2_to_bf16x2(alpha * __uint_as_float(ru[2 * j]),
                                      alpha * __uint_as_float(ru[2 * j + 1]));
            }
            if (args.gu_dump && valid) {
              uint4* dg = reinterpret_cast<uint4*>(args.gu_dump + grow * args.gu_dump_ld + n0 + c0);
              dg[0] = make_uint4(gb[0], gb[1], gb[2], gb[3]);
              dg[1] = make_uint4(gb[4], gb[5], gb[6], gb[7]);
              uint4* du = reinterpret_cast<uint4*>(args.gu_dump + grow * args.gu_dump_ld +
                                                   args.up_row_offset + n0 + c0);
              du[0] = make_uint4(ub[0], ub[1], ub[2], ub[3]);
              du[1] = make_uint4(ub[4], ub[5], ub[6], ub[7]);
            }
            float a[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float g0 = bf16x2_lo(gb[j]), g1 = bf16x2_hi(gb[j]);
              const float u0 = bf16x2_lo(ub[j]), u1 = bf16x2_hi(ub[j]);
              a[2 * j] = (g0 * sigmoid_ref(g0)) * u0;
              a[2 * j + 1] = (g1 * sigmoid_ref(g1)) * u1;
            }
            if constexpr (EPI == Epilogue::kSwigluBf16) {
              if (valid) {
                uint32_t o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = f32x2_to_bf16x2(a[2 * j], a[2 * j + 1]);
                uint4* dst = reinterpret_cast<uint4*>(static_cast<uint16_t*>(args.out) +
                                                      grow * args.ldo + n0 + c0);
                dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
                dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
              }
            } else {
              uint32_t lo, hi;
              const uint32_t sf = quantize_group16(a, next_scale, lo, hi);
              sf_word |= sf << (8 * ((c0 >> 4) & 3));
              if (valid) {
                *reinterpret_cast<uint2*>(static_cast<uint8_t*>(args.out) + grow * args.ldo +
                                          ((n0 + c0) >> 1)) = make_uint2(lo, hi);
                if (((c0 >> 4) & 3) == 3) {
                  uint8_t* dst = args.out_sf_tiles +
                                 (static_cast<size_t>(mt) * out_ntk + ((n0 + c0) >> 6)) * 512u +
                                 sf_in_atom(row, 0);
                  *reinterpret_cast<uint32_t*>(dst) = sf_word;
                }
              }
              if (((c0 >> 4) & 3) == 3) sf_word = 0;
            }
          }
        }
      }
      // hand the accumulator back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty));
      acc_phase ^= 1u;
    }
    if (!ok && args.status && lane == 0) atomicMax(args.status, 3);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, kTmemCols);
  }
}

template <bool NVF4>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a, Epilogue epi,
                   int num_sms, cudaStream_t stream) {
  const size_t smem = kStages * stage_bytes<NVF4>() + 1024;
  const int m_tiles_bound = a.ntiles_dev ? num_sms : a.ntiles_host;
  int grid = a.ntiles_dev ? num_sms : min(num_sms, m_tiles_bound * a.n_tiles);
  if (grid <= 0) return cudaSuccess;
#define Q4T_LAUNCH(E)                                                                          \
  gemm_kernel<NVF4, E><<<grid, kThreads, smem, stream>>>(ta, tb, a);                           \
  break
  switch (epi) {
    case Epilogue::kStoreBf16: Q4T_LAUNCH(Epilogue::kStoreBf16);
    case Epilogue::kStoreF32: Q4T_LAUNCH(Epilogue::kStoreF32);
    case Epilogue::kSwigluBf16: Q4T_LAUNCH(Epilogue::kSwigluBf16);
    case Epilogue::kSwigluQuant: Q4T_LAUNCH(Epilogue::kSwigluQuant);
  }
#undef Q4T_LAUNCH
  return cudaGetLastError();
}

template <bool NVF4, Epilogue E>
cudaError_t set_attr() {
  return cudaFuncSetAttribute(gemm_kernel<NVF4, E>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(kStages * stage_bytes<NVF4>() + 1024));
}

}  // namespace

cudaError_t gemm_set_attributes() {
  cudaError_t e;
  if ((e = set_attr<true, Epilogue::kStoreBf16>()) != cudaSuccess) return e;
  if ((e = set_attr<true, Epilogue::kStoreF32>()) != cudaSuccess) return e;
  if ((e = set_attr<true, Epilogue::kSwigluBf16>()) != cudaSuccess) return e;
  if ((e = set_attr<true, Epilogue::kSwigluQuant>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kStoreBf16>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kStoreF32>()) != cudaSuccess) return e;
  if ((e = set_attr<false, Epilogue::kSwigluBf16>()) != cudaSuccess) return e;
  return cudaSuccess;
}

cudaError_t launch_gemm_nvf4(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a,
                             Epilogue epi, int num_sms, cudaStream_t stream) {
  return launch<true>(ta, tb, a, epi, num_sms, stream);
}

cudaError_t launch_gemm_bf16(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& a,
                             Epilogue epi, int num_sms, cudaStream_t stream) {
  if (epi == Epilogue::kSwigluQuant) return cudaErrorInvalidValue;
  return launch<false>(ta, tb, a, epi, num_sms, stream);
}

}  // namespace q4t
