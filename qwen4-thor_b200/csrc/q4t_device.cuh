// Device-side building blocks shared by all kernels of libq4t_moe_b200:
// bf16 conversion, the NVFP4 number formats (hardware converters plus a
// compare-chain form used to cross-check them), the block-scale atom layout
// and thin wrappers over the sm_100a PTX used by the tensor-core kernels
// (mbarrier, TMA, tcgen05).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace q4t {

// ---------------------------------------------------------------- bf16
__device__ __forceinline__ float bf16_to_f32(uint16_t b) {
  return __uint_as_float(static_cast<uint32_t>(b) << 16);
}
__device__ __forceinline__ uint16_t f32_to_bf16(float f) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
// Two floats -> packed bf16x2 (lo in bits 0-15), round to nearest even.
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float bf16x2_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16x2_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// ---------------------------------------------------------------- formats
// Compare-chain e2m1 encoder: nearest, ties to the even code, saturating,
// sign set for inputs below zero (also when the magnitude rounds to 0);
// -0.0 and NaN give an unsigned code.  Follows FloatToE2m1Code
// (include/q4t/quant/format.h:66-90 of the reference).
__device__ __forceinline__ uint32_t e2m1_encode_sw(float v) {
  const float a = fabsf(v);
  uint32_t c = 7;
  if (a <= 0.25f) c = 0;
  else if (a < 0.75f) c = 1;
  else if (a <= 1.25f) c = 2;
  else if (a < 1.75f) c = 3;
  else if (a <= 2.5f) c = 4;
  else if (a < 3.5f) c = 5;
  else if (a <= 5.0f) c = 6;
  return v < 0.0f ? (c | 8u) : c;
}
// Hardware form: one cvt for two values; byte = code(hi) << 4 | code(lo).
// Adding +0.0f first turns -0.0 into +0.0 so that the sign nibble agrees
// with the compare-chain form for zero inputs.
__device__ __forceinline__ uint32_t e2m1x2_encode_hw(float lo, float hi) {
  uint32_t r;
  const float l = lo + 0.0f, h = hi + 0.0f;
  asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }"
      : "=r"(r)
      : "f"(h), "f"(l));
  return r;
}
// Unsigned e4m3 decode (bias 7, 2^-9 subnormal step, 0x7F reads as 0), after
// E4m3ToFloat (format.h:103-114).
__device__ __forceinline__ float e4m3_decode(uint32_t code) {
  const uint32_t ex = (code >> 3) & 15u, man = code & 7u;
  if (ex == 0) return static_cast<float>(man) * 0.001953125f;
  if (ex == 15 && man == 7) return 0.0f;
  // (8 + man) * 2^(ex - 10), built directly as a float: exponent ex+117+3
  return __uint_as_float(((ex + 120u) << 23) | (man << 20));
}
// Compare/normalise e4m3 encoder for non-negative inputs: nearest even,
// >= 448 saturates to 0x7E; after FloatToE4m3 (format.h:120-164).
__device__ __forceinline__ uint32_t e4m3_encode_sw(float v) {
  const float a = fabsf(v);
  if (a == 0.0f) return 0;
  if (a >= 448.0f) return 0x7E;
  if (a < 0.015625f) return static_cast<uint32_t>(__float2int_rn(a * 512.0f));
  const uint32_t u = __float_as_uint(a);
  int e = static_cast<int>(u >> 23) - 127;                     // floor(log2 a), a is normal here
  const float frac = __uint_as_float((u & 0x007fffffu) | 0x3f800000u);  // [1,2)
  int man = __float2int_rn((frac - 1.0f) * 8.0f);
  int ex = e + 7;
  if (man == 8) { man = 0; ++ex; }
  if (ex > 15 || (ex == 15 && man > 6)) return 0x7E;
  return static_cast<uint32_t>((ex << 3) | man);
}
// Hardware form (round to nearest even, saturate to the largest finite).
__device__ __forceinline__ uint32_t e4m3_encode_hw(float v) {
  uint32_t r;
  asm("{ .reg .b16 t; cvt.rn.satfinite.e4m3x2.f32 t, %1, %2; cvt.u32.u16 %0, t; }"
      : "=r"(r)
      : "f"(0.0f), "f"(v));
  return r & 0xffu;
}

// Correctly rounded reciprocal without the special-case branches of the IEEE
// routine: hardware approximation plus one Newton step in fused arithmetic.
// Equal to 1.0f / x (round to nearest) for every x in [1, 2^126); the encoder
// self-check sweeps that whole range against the IEEE routine.  Branch-free,
// so sixteen of them interleave freely in the epilogue.
__device__ __forceinline__ float rcp_rn_ge1(float x) {
  float r0;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(x));
  const float e = fmaf(-x, r0, 1.0f);
  return fmaf(r0, e, r0);
}
// Upper end of the range where rcp_rn_ge1 is exact (results stay normal).
#define Q4T_RCP_FAST_MAX 8.5070592e37f  /* 2^126 */

// Quantise 16 consecutive values against one global scale
// (src/quant/act_quant.cu:62-90, src/quant/moe_gemm.cu:173-195 of the
// reference): block = amax/6 (1 for an all-zero group), scale byte =
// e4m3(block/global), codes rounded against decode(scale)*global through its
// IEEE reciprocal.  Returns the scale byte; the 8 code bytes go to lo/hi.
__device__ __forceinline__ uint32_t quantize_group16(const float (&a)[16], float global_scale,
                                                     uint32_t& lo, uint32_t& hi) {
  float gmax = 0.0f;
#pragma unroll
  for (int j = 0; j < 16; ++j) gmax = fmaxf(gmax, fabsf(a[j]));
  const float block = gmax > 0.0f ? __fdiv_rn(gmax, 6.0f) : 1.0f;
  const uint32_t sf = e4m3_encode_hw(__fdiv_rn(block, global_scale));
  const float eff = e4m3_decode(sf) * global_scale;
  const float inv = eff > 0.0f ? __frcp_rn(eff) : 0.0f;
  lo = 0;
  hi = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    lo |= e2m1x2_encode_hw(a[2 * j] * inv, a[2 * j + 1] * inv) << (8 * j);
    hi |= e2m1x2_encode_hw(a[8 + 2 * j] * inv, a[8 + 2 * j + 1] * inv) << (8 * j);
  }
  return sf;
}

// ---------------------------------------------------------------- SF atoms
// Byte offset inside one 512-byte atom of (row within its 128-row block,
// group within its 4-group tile).
__device__ __host__ __forceinline__ uint32_t sf_in_atom(uint32_t row, uint32_t group) {
  return (row & 31u) * 16u + ((row & 127u) >> 5) * 4u + (group & 3u);
}
__device__ __host__ __forceinline__ size_t sf_offset(uint32_t row, uint32_t group,
                                                     uint32_t num_g_tiles) {
  return static_cast<size_t>((row >> 7) * num_g_tiles + (group >> 2)) * 512u + sf_in_atom(row, group);
}

// ---------------------------------------------------------------- PTX: sync
// ---- programmatic dependent launch: a kernel launched with launch_chained() may become
// resident as soon as the blocks of the kernel before it in the stream have exited, before
// that kernel's memory is flushed and its completion is processed; it must execute
// chain_wait() before its first access to global memory (the wait returns once the earlier
// kernel has completed and its writes are visible).  With griddepcontrol.launch_dependents
// issued BEFORE the kernel's own wait, a chain of three kernels produced wrong results on B200
// (the third no longer waited for the first); issued after the wait it is correct, and it only
// pays where the next kernel has work to do before its own wait (chain_release_next below).
// A no-op in a kernel launched the ordinary way.
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets the next kernel of the chain become resident now instead of when this kernel's blocks
// have exited.  Only ever issued AFTER this kernel's own chain_wait() (see above), and only by
// a kernel whose successor has useful work to do before its own wait (prefetching operands
// that do not depend on this kernel).
__device__ __forceinline__ void chain_release_next() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{ .reg .pred p; elect.sync _|p, 0xffffffff; selp.u32 %0, 1, 0, p; }" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after about two seconds of polling, or as soon as
// another role of the CTA has raised *abort_flag (shared memory); returns
// false in both cases and raises the flag itself on a time-out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile uint32_t* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 0) {
      if (*abort_flag) return false;
      if (clock64() - start > (1ll << 32)) break;
    }
  }
  *abort_flag = 1;
  return false;
}

// ---------------------------------------------------------------- PTX: TMA
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int32_t c0, int32_t c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------- PTX: tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// Copies one 512-byte scale atom (32 rows x 16 bytes in shared memory) into
// 4 TMEM columns, replicated over the four 32-lane quadrants.
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p; }"
      ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// 16 consecutive fp32 columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// Wider forms: one instruction for 32 / 64 consecutive columns (draining an
// accumulator costs roughly per instruction, not per column).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
      "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,"
      "%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
        "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
        "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
        "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
        "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---------------------------------------------------------------- PTX: CTA pairs
// Two CTAs of one cluster (ranks 0 and 1, neighbouring SMs) work on one 256-row tile with
// tcgen05 cta_group::2: rank 0 (the leader) issues the MMAs, which read both CTAs' shared
// memory at the same offsets and write both CTAs' tensor memory; each CTA loads its own
// operand halves and its TMA completions land on the LEADER's mbarrier.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// All threads of all CTAs of the cluster; also orders shared-memory and mbarrier set-up
// before any remote access.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrive on an mbarrier of another CTA of the cluster (address from cluster_map).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes are counted on an mbarrier that may live in the pair's
// other CTA (`bar` is a cluster address).  Plain load: one CTA's own shared memory is the
// destination, nothing is multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* tmap, int32_t c0, int32_t c1,
                                                 uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// Tensor-memory allocation of a CTA pair: the same warp of BOTH CTAs executes it, with
// the same shared-memory destination offset.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// Arrives, once the pair's earlier tcgen05 operations of this thread have completed, on the
// mbarrier at this shared-memory offset in every CTA of `cta_mask`.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}
// Scale atom copy in both CTAs: each CTA's shared memory to its own tensor memory.
__device__ __forceinline__ void tc_cp_sf_pair(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4_pair(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %6, 0;\n"
      "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%4], [%5], p; }"
      ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_mma_f16_pair(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile whose rows are
// 128 bytes wide and 128-byte swizzled (what a TMA box of 128 bytes x rows
// with SWIZZLE_128B leaves in shared memory): 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);       // start address
  d |= static_cast<uint64_t>(1024u >> 4) << 32;                   // stride between 8-row groups
  d |= 1ull << 46;                                                // descriptor version (sm_100)
  d |= 2ull << 61;                                                // 128-byte swizzle
  return d;
}
// Descriptor of one scale atom in shared memory: no swizzle, 8-row x 16-byte
// core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sf(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffffu) >> 4);
  d |= static_cast<uint64_t>(128u >> 4) << 32;
  d |= 1ull << 46;
  return d;
}

}  // namespace q4t
