// y[M, N] = bf16(x[M, K] . w[N, K]^T) for ONE tile of token rows (M <= 128): the router logits
// (src/model/moe.cu:433-441 of the reference, a bf16 linear over the gate matrix) and the shared
// expert's down projection (src/model/moe.cu:955-969) of mid-size batches.
//
// With a single row tile the work is N/64 column tiles of K/16 tcgen05 steps each, and a
// handful of CTAs have to stream the whole weight matrix.  What bounds such a CTA is not
// bandwidth but how fast one thread can issue TMA loads: a cp.async.bulk.tensor with its
// expect_tx costs that thread about 280 clocks whatever the size of the box (measured: 4 KB,
// 16 KB and 64 KB boxes alike), so loading k-block by k-block (three loads per 64 elements of K)
// took 13 us for K = 2048.  Here the operands are seen through 3-D tensor maps (64 elements x
// rows x K/64) and one load brings four k-blocks, 64 KB of token rows or 32 KB of weight rows;
// the k-blocks land in shared memory one after the other, each in the 128-byte-swizzled K-major
// layout the MMA descriptors expect.  Every output element is the same sequence of kind::f16
// MMAs over K (16 elements per step, fp32 accumulation in tensor memory) as in the general GEMM
// kernel, so the bits do not depend on which of the two kernels ran.
//
// SWIGLU = true is the shared expert's gate/up projection: a CTA takes 32 gate rows and the 32
// matching up rows of the weight (accumulator columns 0-31 and 32-63) and stores
// bf16((g * sigmoid(g)) * u) of the bf16-rounded projections, the arithmetic of the general
// kernel's SwiGLU epilogue (src/model/moe.cu:955-969 of the reference).
#include "kernels.h"
#include "q4t_device.cuh"

namespace q4t {

namespace {

constexpr int kSmThreads = 192;                      // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
constexpr int kSmBN = 64;                            // output columns per CTA
constexpr int kSmDepth = 4;                          // k-blocks (64 bf16 = 128 bytes per row) per load
constexpr uint32_t kSmBSub = kSmBN * 128;            // one k-block of 64 weight rows
constexpr uint32_t kSmBSlot = kSmDepth * kSmBSub;    // 32 KB
constexpr int kSmMaxStages = 6;                      // ring depth, each stage: four k-blocks of the token rows (a_rows x 512 bytes), then the weights
constexpr uint32_t kSmTmemCols = 64;

struct SmBars {
  uint64_t full[kSmMaxStages];
  uint64_t empty[kSmMaxStages];
  uint64_t acc_full;
  uint64_t acc_empty;   // the four epilogue warps have read the accumulator (tiles of several passes)
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// Raised when a bounded wait of this kernel ran out (read and cleared by small_m_gemm_timed_out).
__device__ int g_small_m_gemm_timeout;

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, int32_t c0, int32_t c1, int32_t c2,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, int32_t c0, int32_t c1, int32_t c2, int32_t c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}

// a_rows: rows of the token operand's box (a multiple of 8).  The MMA always reads 128 rows:
// the rows past the box are whatever follows in shared memory (the next k-blocks, the weight
// slot: always inside this stage) and only feed output rows that are never stored.
// SWIGLU: N is the width of the output (a group's weight has 2*N rows, up rows N rows after the
// gate rows); gu_dump (optional) receives the bf16 projections [rows, 2*N].
// Grouped form (g.tile_expert != null; the BF16 experts of the MTP draft layer, src/mtp/
// moe_bf16.cu of the reference): blockIdx.y is a row tile of the permutation tables (the rows of
// one expert, consecutive in x), the weights are that expert's, N and the weight rows count per
// group.  A tile with more rows than the box takes several passes over its weights.
struct SmGroups {
  const int32_t* tile_expert;
  const int32_t* tile_row0;
  const int32_t* tile_nrows;
  const int32_t* ntiles;
  int w_rows_per_group;
};

template <bool SWIGLU>
__global__ void __launch_bounds__(kSmThreads)
bf16_small_m_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    uint16_t* __restrict__ y, int M, int N, int K, int a_rows, int stages,
                    uint16_t* __restrict__ gu_dump, const SmGroups g) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ SmBars bars;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &bars.abort_flag;
  const int nkb = K >> 6;                                  // k-blocks of 64 elements
  const int ngroups = (nkb + kSmDepth - 1) / kSmDepth;      // loads per operand; a short last one reads zeros
  const uint32_t a_sub = static_cast<uint32_t>(a_rows) * 128u;
  const uint32_t a_slot = kSmDepth * a_sub, stage_bytes = a_slot + kSmBSlot;
  constexpr int kOutCols = SWIGLU ? kSmBN / 2 : kSmBN;   // output columns per CTA
  const int n0 = blockIdx.x * kOutCols;

  // x (and the permutation tables) come from the kernels before this one: the grouped form reads
  // the tables first (a CTA without a tile leaves before it has set anything up), the plain form
  // sets up while it may still be waiting
  const bool grouped = g.tile_expert != nullptr;
  int row0 = 0, nrows = M, w_row0 = n0;
  if (grouped) {
    chain_wait();
    const int mt = blockIdx.y;
    if (mt >= *g.ntiles) return;   // the whole CTA: nothing has been set up yet
    row0 = g.tile_row0[mt];
    nrows = g.tile_nrows[mt];
    w_row0 = g.tile_expert[mt] * g.w_rows_per_group + n0;
  }
  const int passes = (nrows + a_rows - 1) / a_rows;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&bars.full[s]), 1);
      mbar_init(smem_u32(&bars.empty[s]), 1);
    }
    mbar_init(smem_u32(&bars.acc_full), 1);
    mbar_init(smem_u32(&bars.acc_empty), (kSmThreads - 64) / 32);
    bars.abort_flag = 0;
    mbar_fence_init();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&bars.tmem_base), kSmTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars.tmem_base;
  if (!grouped) chain_wait();

  if (warp == 0) {
    if (lane == 0) {
      bool ok = true;
      int stage = 0;
      uint32_t phase = 0;
      for (int p = 0; p < passes && ok; ++p) {
        for (int kg = 0; kg < ngroups && ok; ++kg) {
          const uint32_t full = smem_u32(&bars.full[stage]), empty = smem_u32(&bars.empty[stage]);
          if (!mbar_wait(empty, phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + static_cast<uint32_t>(stage) * stage_bytes, sb = sa + a_slot;
          mbar_expect_tx(full, stage_bytes);
          tma_load_3d(sa, &tmap_x, 0, row0 + p * a_rows, kg * kSmDepth, full);
          if (SWIGLU) {   // 4-D box: per k-block 32 gate rows followed by the 32 matching up rows
            tma_load_4d(sb, &tmap_w, 0, w_row0, 0, kg * kSmDepth, full);
          } else {
            tma_load_3d(sb, &tmap_w, 0, w_row0, kg * kSmDepth, full);
          }
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) atomicExch(&g_small_m_gemm_timeout, 1);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // M = 128, N = 64, both operands K-major bf16, fp32 accumulation
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((static_cast<uint32_t>(kSmBN) >> 3) << 17) |
                                 ((128u >> 4) << 24);
      bool ok = true;
      int stage = 0;
      uint32_t phase = 0;
      for (int p = 0; p < passes && ok; ++p) {
        // the epilogue of the previous pass has read the accumulator
        if (p > 0 && !mbar_wait(smem_u32(&bars.acc_empty), (p - 1) & 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        uint32_t accumulate = 0;
        for (int kg = 0; kg < ngroups && ok; ++kg) {
          if (!mbar_wait(smem_u32(&bars.full[stage]), phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + static_cast<uint32_t>(stage) * stage_bytes, sb = sa + a_slot;
          const int left = nkb - kg * kSmDepth;
          for (int j = 0; j < kSmDepth && j < left; ++j) {
            const uint64_t adesc = umma_desc_sw128(sa + static_cast<uint32_t>(j) * a_sub);
            const uint64_t bdesc = umma_desc_sw128(sb + static_cast<uint32_t>(j) * kSmBSub);
#pragma unroll
            for (uint32_t u = 0; u < 4; ++u) {   // 16 elements (32 bytes) of K per instruction
              tc_mma_f16(tmem, adesc + 2u * u, bdesc + 2u * u, idesc, accumulate);
              accumulate = 1;
            }
          }
          tc_commit(smem_u32(&bars.empty[stage]));
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) tc_commit(smem_u32(&bars.acc_full));
      }
      if (!ok) atomicExch(&g_small_m_gemm_timeout, 1);
    }
  } else {
    // epilogue: warp w may touch the tensor-memory lanes of quadrant w % 4; lane = row of the pass
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    for (int p = 0; p < passes; ++p) {
      if (!mbar_wait(smem_u32(&bars.acc_full), p & 1u, abort_flag)) {
        if (lane == 0) atomicExch(&g_small_m_gemm_timeout, 1);
        break;
      }
      tc_fence_after();
      uint32_t v[4][16];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld16(tmem + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(c) * 16u, v[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars.acc_empty));
      const int r = p * a_rows + row;             // row inside the tile
      if (row < a_rows && r < nrows) {
        const size_t orow = static_cast<size_t>(row0 + r);
        if constexpr (!SWIGLU) {
          uint4* dst = reinterpret_cast<uint4*>(y + orow * N + n0);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o[j] = f32x2_to_bf16x2(1.0f * __uint_as_float(v[c][2 * j]), 1.0f * __uint_as_float(v[c][2 * j + 1]));
            dst[2 * c] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[2 * c + 1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        } else {
          // columns 0-31: gate, 32-63: the matching up columns; 16 outputs per round
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t gb[8], ub[8], o[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              gb[j] = f32x2_to_bf16x2(1.0f * __uint_as_float(v[c][2 * j]), 1.0f * __uint_as_float(v[c][2 * j + 1]));
              ub[j] = f32x2_to_bf16x2(1.0f * __uint_as_float(v[c + 2][2 * j]), 1.0f * __uint_as_float(v[c + 2][2 * j + 1]));
            }
            if (gu_dump) {
              uint4* dg = reinterpret_cast<uint4*>(gu_dump + orow * 2 * N + n0 + c * 16);
              dg[0] = make_uint4(gb[0], gb[1], gb[2], gb[3]);
              dg[1] = make_uint4(gb[4], gb[5], gb[6], gb[7]);
              uint4* du = reinterpret_cast<uint4*>(gu_dump + orow * 2 * N + N + n0 + c * 16);
              du[0] = make_uint4(ub[0], ub[1], ub[2], ub[3]);
              du[1] = make_uint4(ub[4], ub[5], ub[6], ub[7]);
            }
            // (g * sigmoid(g)) * u on the bf16 projections, sigmoid through an IEEE reciprocal of
            // 1 + __expf(-g): the general kernel's epilogue arithmetic
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float gl = bf16x2_lo(gb[j]), gh = bf16x2_hi(gb[j]);
              const float dl = 1.0f + __expf(-gl), dh = 1.0f + __expf(-gh);
              const float sl = dl < Q4T_RCP_FAST_MAX ? rcp_rn_ge1(dl) : __frcp_rn(dl);
              const float sh = dh < Q4T_RCP_FAST_MAX ? rcp_rn_ge1(dh) : __frcp_rn(dh);
              o[j] = f32x2_to_bf16x2((gl * sl) * bf16x2_lo(ub[j]), (gh * sh) * bf16x2_hi(ub[j]));
            }
            uint4* dst = reinterpret_cast<uint4*>(y + orow * N + n0 + c * 16);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, kSmTmemCols);
  }
}

size_t small_m_stage_bytes(int a_rows) { return static_cast<size_t>(kSmDepth) * a_rows * 128 + kSmBSlot; }
size_t small_m_smem_bytes(int a_rows, int stages) { return 1024 + static_cast<size_t>(stages) * small_m_stage_bytes(a_rows); }

// As many stages as fit beside the other CTAs that share the SM when the whole grid is resident
// at once: a CTA is bound by the round trips of its own ring (two loads in flight gave 21 GB/s per
// CTA), so few CTAs take deep rings and many CTAs shallow ones.
int small_m_stages(int a_rows, int ctas, int num_sms, bool beside_others = false) {
  if (beside_others) return 2;   // leave the SM's shared memory to the kernels of the other stream
  int per_sm = (ctas + num_sms - 1) / num_sms;
  if (per_sm < 1) per_sm = 1;
  if (per_sm > 3) per_sm = 3;
  const size_t budget = (227 * 1024) / per_sm - 2048;
  int stages = static_cast<int>((budget - 1024) / small_m_stage_bytes(a_rows));
  return stages < 2 ? 2 : (stages > kSmMaxStages ? kSmMaxStages : stages);
}

}  // namespace

cudaError_t bf16_small_m_set_attributes() {
  cudaError_t e = cudaFuncSetAttribute(bf16_small_m_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(bf16_small_m_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 226 * 1024);
}

bool bf16_small_m_fits(int M, int N, int K) { return M >= 1 && M <= 128 && N >= kSmBN && N % kSmBN == 0 && K >= 64 && K % 64 == 0; }
bool bf16_small_m_swiglu_fits(int M, int N, int K) { return M >= 1 && M <= 128 && N >= 32 && N % 32 == 0 && K >= 64 && K % 64 == 0; }

int bf16_small_m_box_rows(int M) { return (M + 7) & ~7; }

cudaError_t launch_bf16_small_m(const CUtensorMap& tmap_x, const CUtensorMap& tmap_w, uint16_t* y, int M, int N, int K,
                                int num_sms, bool beside_others, cudaStream_t stream) {
  if (!bf16_small_m_fits(M, N, K)) return cudaErrorInvalidValue;
  const int a_rows = bf16_small_m_box_rows(M), ctas = N / kSmBN;
  const int stages = small_m_stages(a_rows, ctas, num_sms, beside_others);
  return launch_chained(bf16_small_m_kernel<false>, dim3(static_cast<unsigned>(ctas)), dim3(kSmThreads),
                        small_m_smem_bytes(a_rows, stages), stream, tmap_x, tmap_w, y, M, N, K, a_rows, stages,
                        static_cast<uint16_t*>(nullptr), SmGroups{});
}

cudaError_t launch_bf16_small_m_swiglu(const CUtensorMap& tmap_x, const CUtensorMap& tmap_w, uint16_t* act, int M, int N,
                                       int K, uint16_t* gu_dump, int num_sms, cudaStream_t stream) {
  if (!bf16_small_m_swiglu_fits(M, N, K)) return cudaErrorInvalidValue;
  const int a_rows = bf16_small_m_box_rows(M), ctas = N / (kSmBN / 2), stages = small_m_stages(a_rows, ctas, num_sms, true);
  return launch_chained(bf16_small_m_kernel<true>, dim3(static_cast<unsigned>(ctas)), dim3(kSmThreads),
                        small_m_smem_bytes(a_rows, stages), stream, tmap_x, tmap_w, act, M, N, K, a_rows, stages, gu_dump,
                        SmGroups{});
}

cudaError_t launch_bf16_small_m_grouped(const CUtensorMap& tmap_x, const CUtensorMap& tmap_w, uint16_t* y, bool swiglu,
                                        int box_rows, int max_row_tiles, int N, int K, const int32_t* tile_expert,
                                        const int32_t* tile_row0, const int32_t* tile_nrows, const int32_t* ntiles,
                                        int w_rows_per_group, int num_sms, cudaStream_t stream) {
  if (box_rows < 8 || box_rows > 128 || box_rows % 8 || max_row_tiles < 1 || max_row_tiles > 65535 || K < 64 || K % 64 ||
      N % (swiglu ? 32 : 64) || !tile_expert)
    return cudaErrorInvalidValue;
  const SmGroups g{tile_expert, tile_row0, tile_nrows, ntiles, w_rows_per_group};
  const dim3 grid(static_cast<unsigned>(N / (swiglu ? kSmBN / 2 : kSmBN)), static_cast<unsigned>(max_row_tiles));
  const int stages = small_m_stages(box_rows, static_cast<int>(grid.x * grid.y), num_sms);
  const size_t smem = small_m_smem_bytes(box_rows, stages);
  if (swiglu)
    return launch_chained(bf16_small_m_kernel<true>, grid, dim3(kSmThreads), smem, stream, tmap_x, tmap_w, y, 0, N, K,
                          box_rows, stages, static_cast<uint16_t*>(nullptr), g);
  return launch_chained(bf16_small_m_kernel<false>, grid, dim3(kSmThreads), smem, stream, tmap_x, tmap_w, y, 0, N, K,
                        box_rows, stages, static_cast<uint16_t*>(nullptr), g);
}

// True once after a launch of the kernels above gave up on a bounded wait.
bool small_m_gemm_timed_out() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_small_m_gemm_timeout, sizeof(v)) != cudaSuccess) return false;
  if (v) {
    const int zero = 0;
    cudaMemcpyToSymbol(g_small_m_gemm_timeout, &zero, sizeof(zero));
  }
  return v != 0;
}

}  // namespace q4t
