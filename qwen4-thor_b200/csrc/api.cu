// C ABI of libq4t_moe_b200 (include/q4t_moe_b200.h): argument checking,
// workspace carving, TMA descriptor construction and kernel sequencing.  All
// device work goes to the caller's stream; nothing here synchronises except
// the self-check and status helpers that say so.
#include "../../include/q4t_moe_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <atomic>
#include <mutex>
#include <string>

#include "kernels.h"

namespace {

thread_local std::string g_error;

int fail(int code, const std::string& msg) {
  g_error = msg;
  return code;
}
int fail_cuda(const char* what, cudaError_t e) {
  g_error = std::string(what) + ": " + cudaGetErrorString(e);
  return Q4T_ERR_CUDA;
}

}  // namespace

// Lets the library's other translation units record an error for the calling thread.
int q4t_internal_fail(int code, const char* msg) { return fail(code, msg ? msg : ""); }

namespace {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready = false;
  int num_sms = 0;
  EncodeFn encode = nullptr;
  // The shared expert depends only on x, so q4t_moe_forward runs it on this
  // library-owned stream beside the router / permutation / quantise chain and
  // joins before the combine (fork and join by events, no host involvement).
  // One stream and one set of events per HOST THREAD and device (see ThreadLanes):
  // callers on different threads never meet on them.
  cudaStream_t side_stream = nullptr;
  cudaEvent_t fork_event = nullptr, join_event = nullptr, mid_event = nullptr;
};
constexpr int kMaxDevices = 16;
DeviceState g_dev[kMaxDevices];   // per device: facts shared by all threads (no stream, no events)
std::mutex g_dev_mutex;

// What device_state() hands out: the calling thread's own copy of the device's facts plus
// its own side stream and events, created on the thread's first call for that device and
// released when the thread ends.
struct ThreadLanes {
  DeviceState dev[kMaxDevices];
  ~ThreadLanes() {
    for (DeviceState& d : dev) {
      if (!d.ready) continue;
      // at process exit the runtime may already be gone: failures are of no consequence
      cudaEventDestroy(d.fork_event);
      cudaEventDestroy(d.join_event);
      cudaEventDestroy(d.mid_event);
      cudaStreamDestroy(d.side_stream);
    }
  }
};
thread_local ThreadLanes t_lanes;

// Per-device one-time set-up: architecture check, driver entry point for the
// tensor-map encoder, shared-memory attribute of the GEMM kernels.
int device_state(const DeviceState** out) {
  // every compute entry point passes here first: its first kernel follows the caller's
  // own stream work and is launched the ordinary way
  q4t::chain_break();
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(Q4T_ERR_DEVICE, std::string("no CUDA device: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(Q4T_ERR_DEVICE, "device index out of range");
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  DeviceState& s = g_dev[dev];
  if (!s.ready) {
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) return fail_cuda("cudaGetDeviceProperties", e);
    if (prop.major != 10)
      return fail(Q4T_ERR_DEVICE, "libq4t_moe_b200 needs an sm_100 device (found sm_" +
                                      std::to_string(prop.major) + std::to_string(prop.minor) + ")");
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess)
      return fail(Q4T_ERR_DEVICE, "cuTensorMapEncodeTiled entry point unavailable");
    if ((e = q4t::gemm_set_attributes()) != cudaSuccess) return fail_cuda("cudaFuncSetAttribute", e);
    if ((e = q4t::gemm_pair_set_attributes()) != cudaSuccess) return fail_cuda("cudaFuncSetAttribute", e);
    if ((e = q4t::routing_set_attributes()) != cudaSuccess) return fail_cuda("cudaFuncSetAttribute", e);
    if ((e = q4t::small_batch_set_attributes()) != cudaSuccess) return fail_cuda("cudaFuncSetAttribute", e);
    if ((e = q4t::bf16_small_m_set_attributes()) != cudaSuccess) return fail_cuda("cudaFuncSetAttribute", e);
    s.encode = reinterpret_cast<EncodeFn>(fn);
    s.num_sms = prop.multiProcessorCount;
    s.ready = true;
  }
  DeviceState& mine = t_lanes.dev[dev];
  if (!mine.ready) {
    DeviceState fresh = s;
    if ((e = cudaStreamCreateWithFlags(&fresh.side_stream, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&fresh.fork_event, cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&fresh.join_event, cudaEventDisableTiming)) != cudaSuccess ||
        (e = cudaEventCreateWithFlags(&fresh.mid_event, cudaEventDisableTiming)) != cudaSuccess)
      return fail_cuda("side stream set-up", e);
    mine = fresh;
  }
  *out = &mine;
  return Q4T_OK;
}

// 2-D K-major tensor map whose box is 128 bytes x box_rows rows, 128-byte swizzled.
int make_tmap(const DeviceState* ds, CUtensorMap* tm, bool bf16, const void* base, uint64_t inner_elems,
              uint64_t rows, uint64_t pitch_bytes, uint32_t box_rows = 128) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || (pitch_bytes & 15u))
    return fail(Q4T_ERR_INVALID, "operand base and row pitch must be 16-byte aligned");
  cuuint64_t dims[2] = {inner_elems, rows};
  cuuint64_t strides[1] = {pitch_bytes};
  cuuint32_t box[2] = {bf16 ? 64u : 128u, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = ds->encode(tm, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                          const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(Q4T_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return Q4T_OK;
}

// 3-D view of a K-major bf16 matrix, 64 elements x rows x K/64, whose box brings `depth`
// consecutive k-blocks of `box_rows` rows with one load (bf16_small_m.cu); each k-block lands
// 128-byte swizzled like a box of make_tmap.
int make_tmap_kblocks(const DeviceState* ds, CUtensorMap* tm, const void* base, uint64_t K, uint64_t rows,
                      uint32_t box_rows, uint32_t depth) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((K * 2) & 15u) || K % 64)
    return fail(Q4T_ERR_INVALID, "operand base and row pitch must be 16-byte aligned");
  cuuint64_t dims[3] = {64, rows, K / 64};
  cuuint64_t strides[2] = {K * 2, 128};
  cuuint32_t box[3] = {64, box_rows, depth};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = ds->encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(Q4T_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return Q4T_OK;
}

// The same for a gate|up weight [2*N, K]: 64 elements x N rows x 2 halves x K/64, box 64 x 32 x 2 x depth,
// so that every k-block lands as 32 gate rows followed by the 32 matching up rows.
int make_tmap_kblocks_gate_up(const DeviceState* ds, CUtensorMap* tm, const void* base, uint64_t K, uint64_t N,
                              uint32_t depth, uint64_t first_half_rows = 0) {
  if ((reinterpret_cast<uintptr_t>(base) & 15u) || ((K * 2) & 15u) || K % 64)
    return fail(Q4T_ERR_INVALID, "operand base and row pitch must be 16-byte aligned");
  // first_half_rows: rows a box may start at (a stack of [2*N, K] weights: all rows but the last N)
  cuuint64_t dims[4] = {64, first_half_rows ? first_half_rows : N, 2, K / 64};
  cuuint64_t strides[3] = {K * 2, N * K * 2, 128};
  cuuint32_t box[4] = {64, 32, 2, depth};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = ds->encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(Q4T_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return Q4T_OK;
}

// [atoms, 512 bytes] view of a buffer of block-scale atoms for the CTA-pair GEMMs: rows of
// 128 uint32, a box of four atoms (the four k-steps of one 256-element k-block), no swizzle.
// Atoms past the end read as zeros.
int make_sf_tmap(const DeviceState* ds, CUtensorMap* tm, const void* base, uint64_t atoms) {
  if (reinterpret_cast<uintptr_t>(base) & 15u) return fail(Q4T_ERR_INVALID, "scale buffers must be 16-byte aligned");
  cuuint64_t dims[2] = {128, atoms ? atoms : 1};
  cuuint64_t strides[1] = {512};
  cuuint32_t box[2] = {128, 4};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = ds->encode(tm, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(Q4T_ERR_CUDA, "cuTensorMapEncodeTiled failed (" + std::to_string(int(r)) + ")");
  return Q4T_OK;
}

// GEMMs with at least this many A rows run as CTA pairs (tc_gemm_pair.cu).  Off by default:
// on B200 the pair form measured 5-10 % slower than one CTA per tile, because the block-scaled
// mainloop is bound by each SM's tensor pipe, not by the operand traffic a pair halves.
// q4t_set_pair_min_rows() or the environment variable Q4T_PAIR_MIN_ROWS turn it on.
constexpr int64_t kPairNever = static_cast<int64_t>(1) << 62;
std::atomic<int64_t> g_pair_min_rows{-1};
int64_t pair_min_rows() {
  int64_t v = g_pair_min_rows.load(std::memory_order_relaxed);
  if (v < 0) {
    const char* e = std::getenv("Q4T_PAIR_MIN_ROWS");
    const long long n = e ? std::atoll(e) : 0;
    v = n <= 0 ? kPairNever : static_cast<int64_t>(n);
    g_pair_min_rows.store(v, std::memory_order_relaxed);
  }
  return v;
}

// Optional event marks between stages (off by default).
struct StageTimer {
  bool enabled = false;
  cudaEvent_t ev[Q4T_NUM_STAGES + 1] = {};
  bool marked[Q4T_NUM_STAGES + 1] = {};
};
thread_local StageTimer g_timer;
void stage_begin(cudaStream_t st) {
  if (!g_timer.enabled) return;
  for (bool& m : g_timer.marked) m = false;
  cudaEventRecord(g_timer.ev[0], st);
  g_timer.marked[0] = true;
}
// Marks the end of stage `i` (its event is ev[i + 1]).
void stage_end(int i, cudaStream_t st) {
  if (!g_timer.enabled) return;
  cudaEventRecord(g_timer.ev[i + 1], st);
  g_timer.marked[i + 1] = true;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
size_t sf_buffer_size(int rows, int K) {
  return static_cast<size_t>((rows + 127) / 128) * static_cast<size_t>((K / 16 + 3) / 4) * 512;
}

void routed_layout(int M, int k, int hs, int is, int E, q4t_routed_ws_layout* L) {
  const size_t R = static_cast<size_t>(M) * k;
  // every expert with rows ends in one partial row tile; batches that run as CTA pairs pad
  // each such expert to an even tile count
  const size_t active = R < static_cast<size_t>(E) ? R : static_cast<size_t>(E);
  const size_t max_tiles = static_cast<int64_t>(R) >= pair_min_rows() ? ((R / 128 + 2 * active + 2) & ~static_cast<size_t>(1))
                                                                      : R / 128 + active + 1;
  const size_t nblk = (R + q4t::kPlanChunk - 1) / q4t::kPlanChunk;
  size_t off = 0;
  auto take = [&](size_t bytes, size_t align = 256) {
    off = align_up(off, align);
    const size_t at = off;
    off += bytes;
    return at;
  };
  // reference regions, packed back to back as in MoEWorkspace::Init
  L->a_packed = take(R * (hs / 2), 1);
  L->a_sf = take(sf_buffer_size(static_cast<int>(R), hs), 1);
  L->gu_out = take(R * 2 * is * 2, 1);
  L->dn_out = take(R * hs * 2, 1);
  L->counts = take(static_cast<size_t>(E) * 4);
  L->offsets = take(static_cast<size_t>(E + 1) * 4);
  L->row_of_flat = take(R * 4);
  L->flat_of_row = take(R * 4);
  L->row_tile = take(R * 4);
  L->ntiles = take(256);
  L->tile_expert = take(max_tiles * 4);
  L->tile_row0 = take(max_tiles * 4);
  L->tile_nrows = take(max_tiles * 4);
  L->a_sf_tiles = take(max_tiles * static_cast<size_t>((hs + 63) / 64) * 512);
  L->xq_packed = take(static_cast<size_t>(M) * (hs / 2));
  L->xq_sf = take(sf_buffer_size(M, hs));
  L->inter_packed = take(R * (is / 2));
  L->inter_sf_tiles = take(max_tiles * static_cast<size_t>((is + 63) / 64) * 512);
  L->status = take(256);
  // planning scratch that callers never read: tile_off [E+1], blk_counts [nblk, E]
  take(static_cast<size_t>(E + 1) * 4);
  take(nblk * static_cast<size_t>(E) * 4);
  L->max_tiles = max_tiles;
  L->total = align_up(off, 256);
}

void forward_layout(int T, int k, int hs, int is, int sis, int E, q4t_forward_ws_layout* F) {
  q4t_routed_ws_layout R;
  routed_layout(T, k, hs, is, E, &R);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    off = align_up(off, 256);
    const size_t at = off;
    off += bytes;
    return at;
  };
  F->routed_ws = take(R.total);
  F->logits = take(static_cast<size_t>(T) * E * 2);
  F->expert_ids = take(static_cast<size_t>(T) * k * 4);
  F->router_w = take(static_cast<size_t>(T) * k * 4);
  F->routed = take(static_cast<size_t>(T) * hs * 4);
  F->shared_gu = take(static_cast<size_t>(T) * 2 * sis * 2);
  F->shared_act = take(static_cast<size_t>(T) * sis * 2);
  F->shared_down = take(static_cast<size_t>(T) * hs * 2);
  F->slot_ids = take(static_cast<size_t>(T) * k * 4);
  F->total = align_up(off, 256);
}

bool routed_dims_ok(int E, int hs, int is) {
  // hs and 2*is multiples of 128 (per-expert scale blocks), is a multiple of
  // 128 (gate and up rows of one tile come from whole scale atoms), E within
  // the planning kernel's single-block scan.
  return E > 0 && E <= 1024 && hs > 0 && is > 0 && hs % 128 == 0 && is % 128 == 0;
}

struct RoutedPtrs {
  q4t_routed_ws_layout L;
  uint8_t* base;
  template <typename T>
  T* at(size_t off) const { return reinterpret_cast<T*>(base + off); }
};

// Steps shared by the routed entry point and the full layer: permutation,
// gather-quantise, gate/up GEMM with fused SwiGLU + requantisation, down GEMM.
q4t::PlanTables plan_tables(const RoutedPtrs& P, int E) {
  const q4t_routed_ws_layout& L = P.L;
  q4t::PlanTables pt;
  pt.counts = P.at<int32_t>(L.counts);
  pt.offsets = P.at<int32_t>(L.offsets);
  pt.row_of_flat = P.at<int32_t>(L.row_of_flat);
  pt.flat_of_row = P.at<int32_t>(L.flat_of_row);
  pt.row_tile = P.at<int32_t>(L.row_tile);
  pt.ntiles = P.at<int32_t>(L.ntiles);
  pt.tile_expert = P.at<int32_t>(L.tile_expert);
  pt.tile_row0 = P.at<int32_t>(L.tile_row0);
  pt.tile_nrows = P.at<int32_t>(L.tile_nrows);
  pt.tile_off = P.at<int32_t>(align_up(L.status + 256, 256));
  pt.blk_counts = P.at<int32_t>(align_up(align_up(L.status + 256, 256) + static_cast<size_t>(E + 1) * 4, 256));
  pt.status = P.at<int32_t>(L.status);
  return pt;
}

// plan_done: the permutation tables of P were already produced (fused with the router).
// peer (optional): the token rows come quantised from the gathered per-rank blocks and
// the down-projection rows go straight to their owners' landing buffers.
struct PeerRoute {
  const uint8_t* xq_packed;  // [world*tokens_per_rank, hs/2]
  const uint8_t* xq_sf;      // [world*tokens_per_rank, hs/16] row-major scale bytes
  uint16_t* dn_rows[q4t::kMaxPeers];
  int rows_per_rank;  // tokens_per_rank * k
};
// Tensor-memory columns of the decode-sized kernels: the accumulator (32) and one slot of
// scale atoms per ring stage (16 weight-side + 16 token-side columns); at most 10 stages.
uint32_t small_tmem_cols(int stages) {
  const uint32_t need = 32u + 32u * static_cast<uint32_t>(stages);
  uint32_t c = 32;
  while (c < need) c <<= 1;
  return c;
}

// Decode-sized batches (decode_small.cu) unless the caller asks for the general path
// (flags bit 2) or the reduction lengths do not fit its shared-memory operand.
bool small_batch_applies(int M, int k, int E, int hs, int is, uint32_t flags) {
  static const bool off = std::getenv("Q4T_NO_SMALL_BATCH") != nullptr;
  // measured on a B200 at hs 2048 / 512 experts / top-10: this path is 8 us faster than the
  // grouped kernels at 32 and 64 tokens, level with them at 96 and 128
  static const int max_tokens = [] {
    const char* v = std::getenv("Q4T_SMALL_MAX_TOKENS");
    const int n = v ? std::atoi(v) : 64;
    return n < q4t::kSmallMaxTokens ? n : q4t::kSmallMaxTokens;
  }();
  const int limit = (flags & 8u) ? q4t::kSmallMaxTokens : max_tokens;
  return !off && !(flags & 4u) && M <= limit && M * k <= q4t::kSmallMaxEntries && E <= q4t::kSmallMaxExperts &&
         q4t::small_batch_stages(hs, 1 << 20, M * k) > 0 && q4t::small_batch_stages(is, 1 << 20, M * k) > 0;
}

// Gate/up and down for a decode-sized batch: two launches, rows in (token,slot) order.
int run_routed_small(const DeviceState* ds, const uint16_t* x, const int32_t* ids, const q4t_routed_weights* w,
                     const RoutedPtrs& P, int M, int k, cudaStream_t st) {
  const int E = w->E, hs = w->hs, is = w->moe_is, R = M * k;
  const q4t_routed_ws_layout& L = P.L;
  stage_end(2, st);
  stage_end(3, st);
  CUtensorMap tm;
  int rc;
  if ((rc = make_tmap(ds, &tm, false, w->gu_packed, hs / 2, static_cast<uint64_t>(E) * 2 * is, hs / 2)) != Q4T_OK)
    return rc;
  q4t::SmallBatchArgs g{};
  g.ids = ids;
  g.R = R;
  g.k = k;
  g.E = E;
  g.K = hs;
  g.n_tiles = 2 * is / 128;
  g.w_rows_per_expert = 2 * is;
  g.w_sf = w->gu_sf;
  g.w_sf_stride = sf_buffer_size(2 * is, hs);
  g.alpha_w = w->gu_w_scale2;
  g.alpha_a = w->gu_input_scale;
  g.in_scale = w->gu_input_scale;
  g.src = x;
  g.src_ld = hs;
  g.out = P.at<uint16_t>(L.gu_out);
  g.ldo = 2 * is;
  g.row_of_flat = P.at<int32_t>(L.row_of_flat);
  g.status = P.at<int32_t>(L.status);
  g.stages = q4t::small_batch_stages(hs, R * g.n_tiles, R);
  g.tmem_cols = small_tmem_cols(g.stages);
  {
    static const int rel = [] { const char* v = std::getenv("Q4T_SMALL_RELEASE"); return v ? std::atoi(v) : 1; }();
    g.release_next = rel;
  }
  cudaError_t e = q4t::launch_small_batch(0, tm, g, ds->num_sms, st);
  if (e != cudaSuccess) return fail_cuda("decode gate/up launch", e);
  stage_end(4, st);
  if ((rc = make_tmap(ds, &tm, false, w->dn_packed, is / 2, static_cast<uint64_t>(E) * hs, is / 2)) != Q4T_OK) return rc;
  q4t::SmallBatchArgs d{};
  d.ids = ids;
  d.R = R;
  d.k = k;
  d.E = E;
  d.K = is;
  d.n_tiles = hs / 128;
  d.w_rows_per_expert = hs;
  d.w_sf = w->dn_sf;
  d.w_sf_stride = sf_buffer_size(hs, is);
  d.alpha_w = w->dn_w_scale2;
  d.alpha_a = w->dn_input_scale;
  d.in_scale = w->dn_input_scale;
  d.src = P.at<uint16_t>(L.gu_out);
  d.src_ld = 2 * is;
  d.out = P.at<uint16_t>(L.dn_out);
  d.ldo = hs;
  d.row_of_flat = nullptr;
  d.status = P.at<int32_t>(L.status);
  d.stages = q4t::small_batch_stages(is, R * d.n_tiles, R);
  d.tmem_cols = small_tmem_cols(d.stages);
  if ((e = q4t::launch_small_batch(1, tm, d, ds->num_sms, st)) != cudaSuccess) return fail_cuda("decode down launch", e);
  stage_end(5, st);
  return Q4T_OK;
}

int run_routed_core(const DeviceState* ds, const uint16_t* x, const int32_t* ids,
                    const q4t_routed_weights* w, const RoutedPtrs& P, int M, int k, uint32_t flags,
                    cudaStream_t st, bool plan_done = false, const PeerRoute* peer = nullptr) {
  const int E = w->E, hs = w->hs, is = w->moe_is;
  const int R = M * k;
  const q4t_routed_ws_layout& L = P.L;
  if (!plan_done && !peer && small_batch_applies(M, k, E, hs, is, flags)) return run_routed_small(ds, x, ids, w, P, M, k, st);
  cudaError_t e;
  const q4t::PlanTables pt = plan_tables(P, E);  // the planner also clears the status words
  // large batches: CTA-pair GEMMs over pairs of row tiles of one expert
  const bool pair = !plan_done && static_cast<int64_t>(R) >= pair_min_rows();
  if (!plan_done) {
    if ((e = q4t::launch_plan(ids, R, E, static_cast<int>(L.max_tiles), pt, st, pair)) != cudaSuccess)
      return fail_cuda("plan launch", e);
  }
  stage_end(2, st);

  uint8_t* a_packed = P.at<uint8_t>(L.a_packed);
  uint8_t* a_sf_tiles = P.at<uint8_t>(L.a_sf_tiles);
  // With one input scale for all experts and a large batch, quantise each token
  // once and copy its codes to its k rows; otherwise quantise every grouped row.
  if (peer) {
    if ((e = q4t::launch_gather_codes_rowsf(peer->xq_packed, peer->xq_sf, a_packed, a_sf_tiles, R, hs,
                                            pt.flat_of_row, pt.row_tile, pt.tile_row0, pt.offsets + E, k, st)) !=
        cudaSuccess)
      return fail_cuda("block code gather launch", e);
  } else if (w->gu_input_scale_uniform > 0.0f && k > 1 && k <= 16 && hs >= 128 && R >= 8192) {
    if ((e = q4t::launch_quantize_scatter(x, a_packed, a_sf_tiles, M, hs, w->gu_input_scale_uniform, pt.row_of_flat,
                                          pt.row_tile, pt.tile_row0, k, st)) != cudaSuccess)
      return fail_cuda("quantise-scatter launch", e);
  } else if ((e = q4t::launch_gather_quantize(x, a_packed, a_sf_tiles, R, hs, pt.flat_of_row, ids,
                                              w->gu_input_scale, pt.row_tile, pt.tile_row0, pt.offsets + E, k, E,
                                              st)) != cudaSuccess) {
    return fail_cuda("gather-quantise launch", e);
  }
  stage_end(3, st);

  CUtensorMap tm_a, tm_b;
  int rc;
  // gate/up: A = grouped input codes [R, hs/2], B = all experts' gate|up rows
  if ((rc = make_tmap(ds, &tm_a, false, a_packed, hs / 2, R, hs / 2)) != Q4T_OK) return rc;
  if ((rc = make_tmap(ds, &tm_b, false, w->gu_packed, hs / 2, static_cast<uint64_t>(E) * 2 * is, hs / 2)) != Q4T_OK)
    return rc;
  q4t::GemmArgs g{};
  g.K = hs;
  g.n_tiles = is / 128;
  g.n_per_tile = 128;
  g.up_row_offset = is;
  g.b_rows_per_group = 2 * is;
  g.b_rows_valid = is;
  g.ntiles_dev = pt.ntiles;
  g.tile_expert = pt.tile_expert;
  g.tile_row0 = pt.tile_row0;
  g.tile_nrows = pt.tile_nrows;
  g.total_rows = R;
  g.sfa_tiles = a_sf_tiles;
  g.sfb = w->gu_sf;
  g.sfb_group_stride = sf_buffer_size(2 * is, hs);
  g.out = P.at<uint8_t>(L.inter_packed);
  g.ldo = is / 2;
  g.alpha_w = w->gu_w_scale2;
  g.alpha_a = w->gu_input_scale;
  g.next_scale = w->dn_input_scale;
  g.out_sf_tiles = P.at<uint8_t>(L.inter_sf_tiles);
  g.gu_dump = (flags & 1u) ? P.at<uint16_t>(L.gu_out) : nullptr;
  g.gu_dump_ld = 2 * is;
  g.status = P.at<int32_t>(L.status);
  if (pair) {
    CUtensorMap tm_sfa, tm_sfb;
    g.sfb_group_atoms = static_cast<int>(g.sfb_group_stride / 512);
    if ((rc = make_sf_tmap(ds, &tm_sfa, a_sf_tiles, L.max_tiles * static_cast<uint64_t>((hs + 63) / 64))) != Q4T_OK) return rc;
    if ((rc = make_sf_tmap(ds, &tm_sfb, w->gu_sf, static_cast<uint64_t>(E) * g.sfb_group_atoms)) != Q4T_OK) return rc;
    e = q4t::launch_gemm_nvf4_pair(tm_a, tm_b, tm_sfa, tm_sfb, g, q4t::Epilogue::kSwigluQuant, ds->num_sms, st);
  } else {
    e = q4t::launch_gemm_nvf4(tm_a, tm_b, g, q4t::Epilogue::kSwigluQuant, ds->num_sms, st);
  }
  if (e != cudaSuccess) return fail_cuda("gate/up GEMM launch", e);
  stage_end(4, st);

  // down: A = intermediate codes [R, is/2], B = all experts' down rows
  if ((rc = make_tmap(ds, &tm_a, false, P.at<uint8_t>(L.inter_packed), is / 2, R, is / 2)) != Q4T_OK) return rc;
  if ((rc = make_tmap(ds, &tm_b, false, w->dn_packed, is / 2, static_cast<uint64_t>(E) * hs, is / 2)) != Q4T_OK)
    return rc;
  q4t::GemmArgs d{};
  d.K = is;
  d.n_tiles = (hs + 255) / 256;
  d.n_per_tile = 256;
  d.b_rows_per_group = hs;
  d.b_rows_valid = hs;
  d.ntiles_dev = pt.ntiles;
  d.tile_expert = pt.tile_expert;
  d.tile_row0 = pt.tile_row0;
  d.tile_nrows = pt.tile_nrows;
  d.total_rows = R;
  d.sfa_tiles = P.at<uint8_t>(L.inter_sf_tiles);
  d.sfb = w->dn_sf;
  d.sfb_group_stride = sf_buffer_size(hs, is);
  d.out = P.at<uint16_t>(L.dn_out);
  d.ldo = hs;
  d.alpha_w = w->dn_w_scale2;
  d.alpha_a = w->dn_input_scale;
  d.status = P.at<int32_t>(L.status);
  if (peer) {
    d.scatter_flat = pt.flat_of_row;
    d.scatter_rows_per_rank = peer->rows_per_rank;
    for (int i = 0; i < q4t::kMaxPeers; ++i) d.scatter_base[i] = peer->dn_rows[i];
  }
  const q4t::Epilogue dn_epi = peer ? q4t::Epilogue::kStoreBf16Rows : q4t::Epilogue::kStoreBf16;
  if (pair) {
    CUtensorMap tm_sfa, tm_sfb;
    d.sfb_group_atoms = static_cast<int>(d.sfb_group_stride / 512);
    if ((rc = make_sf_tmap(ds, &tm_sfa, d.sfa_tiles, L.max_tiles * static_cast<uint64_t>((is + 63) / 64))) != Q4T_OK) return rc;
    if ((rc = make_sf_tmap(ds, &tm_sfb, w->dn_sf, static_cast<uint64_t>(E) * d.sfb_group_atoms)) != Q4T_OK) return rc;
    e = q4t::launch_gemm_nvf4_pair(tm_a, tm_b, tm_sfa, tm_sfb, d, dn_epi, ds->num_sms, st);
  } else {
    e = q4t::launch_gemm_nvf4(tm_a, tm_b, d, dn_epi, ds->num_sms, st);
  }
  if (e != cudaSuccess) return fail_cuda("down GEMM launch", e);
  stage_end(5, st);
  return Q4T_OK;
}

// The routed experts with BF16 weights (the MTP draft layer's MoE, src/mtp/moe_bf16.cu:
// 300-420): gather the token rows in expert order, gate/up GEMM with the SwiGLU epilogue
// (bf16 projections, bf16((g*sigmoid(g))*u)), down GEMM to bf16 rows.  `compact` is the
// [M*k, hs] bf16 row buffer; the intermediate reuses the gu_out region, the result dn_out.
// Q4T_NO_SMALL_M_GEMM: the general GEMM kernel for every BF16 projection (A/B measurements).
bool no_small_m_gemm() {
  static const bool off = std::getenv("Q4T_NO_SMALL_M_GEMM") != nullptr;
  return off;
}

int run_routed_core_bf16(const DeviceState* ds, const uint16_t* x, const int32_t* ids,
                         const q4t_bf16_expert_weights* w, const RoutedPtrs& P, uint16_t* compact, int M, int k,
                         cudaStream_t st, bool plan_done) {
  const int E = w->E, hs = w->hs, is = w->moe_is;
  const int R = M * k;
  const q4t_routed_ws_layout& L = P.L;
  cudaError_t e;
  const q4t::PlanTables pt = plan_tables(P, E);
  if (!plan_done && (e = q4t::launch_plan(ids, R, E, static_cast<int>(L.max_tiles), pt, st)) != cudaSuccess)
    return fail_cuda("plan launch", e);
  stage_end(2, st);
  if ((e = q4t::launch_gather_rows(x, pt.flat_of_row, k, pt.offsets + E, R, hs, compact, nullptr, nullptr, st)) !=
      cudaSuccess)
    return fail_cuda("row gather launch", e);
  stage_end(3, st);
  uint16_t* inter = P.at<uint16_t>(L.gu_out);
  CUtensorMap tm_a, tm_b;
  int rc;
  // draft-sized batches: every expert has at most M rows, so a tile is a handful of rows against
  // 64 weight rows, loaded four k-blocks at a time (bf16_small_m.cu)
  if (!no_small_m_gemm() && M <= 16 && hs % 64 == 0 && is % 64 == 0) {
    const int box_rows = q4t::bf16_small_m_box_rows(M);
    // one row tile per expert with rows, one more for every 128 rows an expert has beyond that
    const int max_row_tiles = (R < E ? R : E) + R / 128;
    if ((rc = make_tmap_kblocks(ds, &tm_a, compact, hs, R, box_rows, 4)) != Q4T_OK) return rc;
    if ((rc = make_tmap_kblocks_gate_up(ds, &tm_b, w->gu, hs, is, 4, static_cast<uint64_t>(E) * 2 * is - is)) != Q4T_OK)
      return rc;
    if ((e = q4t::launch_bf16_small_m_grouped(tm_a, tm_b, inter, true, box_rows, max_row_tiles, is, hs, pt.tile_expert,
                                              pt.tile_row0, pt.tile_nrows, pt.ntiles, 2 * is, ds->num_sms, st)) != cudaSuccess)
      return fail_cuda("bf16 gate/up launch", e);
    stage_end(4, st);
    if ((rc = make_tmap_kblocks(ds, &tm_a, inter, is, R, box_rows, 4)) != Q4T_OK) return rc;
    if ((rc = make_tmap_kblocks(ds, &tm_b, w->down, is, static_cast<uint64_t>(E) * hs, 64, 4)) != Q4T_OK) return rc;
    if ((e = q4t::launch_bf16_small_m_grouped(tm_a, tm_b, P.at<uint16_t>(L.dn_out), false, box_rows, max_row_tiles, hs, is,
                                              pt.tile_expert, pt.tile_row0, pt.tile_nrows, pt.ntiles, hs, ds->num_sms, st)) != cudaSuccess)
      return fail_cuda("bf16 down launch", e);
    stage_end(5, st);
    return Q4T_OK;
  }
  if ((rc = make_tmap(ds, &tm_a, true, compact, hs, R, static_cast<uint64_t>(hs) * 2)) != Q4T_OK) return rc;
  if ((rc = make_tmap(ds, &tm_b, true, w->gu, hs, static_cast<uint64_t>(E) * 2 * is, static_cast<uint64_t>(hs) * 2)) !=
      Q4T_OK)
    return rc;
  q4t::GemmArgs g{};
  g.K = hs;
  g.tile_cols = 256;
  g.n_tiles = is / 128;
  g.n_per_tile = 128;
  g.up_row_offset = is;
  g.b_rows_per_group = 2 * is;
  g.b_rows_valid = is;
  g.ntiles_dev = pt.ntiles;
  g.tile_expert = pt.tile_expert;
  g.tile_row0 = pt.tile_row0;
  g.tile_nrows = pt.tile_nrows;
  g.total_rows = R;
  g.out = inter;
  g.ldo = is;
  g.alpha_const = 1.0f;
  g.status = P.at<int32_t>(L.status);
  if ((e = q4t::launch_gemm_bf16(tm_a, tm_b, g, q4t::Epilogue::kSwigluBf16, ds->num_sms, st)) != cudaSuccess)
    return fail_cuda("bf16 gate/up GEMM launch", e);
  stage_end(4, st);
  if ((rc = make_tmap(ds, &tm_a, true, inter, is, R, static_cast<uint64_t>(is) * 2)) != Q4T_OK) return rc;
  if ((rc = make_tmap(ds, &tm_b, true, w->down, is, static_cast<uint64_t>(E) * hs, static_cast<uint64_t>(is) * 2)) !=
      Q4T_OK)
    return rc;
  q4t::GemmArgs d{};
  d.K = is;
  d.tile_cols = 256;
  d.n_tiles = (hs + 255) / 256;
  d.n_per_tile = 256;
  d.b_rows_per_group = hs;
  d.b_rows_valid = hs;
  d.ntiles_dev = pt.ntiles;
  d.tile_expert = pt.tile_expert;
  d.tile_row0 = pt.tile_row0;
  d.tile_nrows = pt.tile_nrows;
  d.total_rows = R;
  d.out = P.at<uint16_t>(L.dn_out);
  d.ldo = hs;
  d.alpha_const = 1.0f;
  d.status = P.at<int32_t>(L.status);
  if ((e = q4t::launch_gemm_bf16(tm_a, tm_b, d, q4t::Epilogue::kStoreBf16, ds->num_sms, st)) != cudaSuccess)
    return fail_cuda("bf16 down GEMM launch", e);
  stage_end(5, st);
  return Q4T_OK;
}

// y[M,N] = bf16(x . w^T): exact-order warp GEMV for M <= 8, tensor cores above.
int run_bf16_linear(const DeviceState* ds, const uint16_t* x, const uint16_t* w, uint16_t* y, int M, int N,
                    int K, cudaStream_t st, bool beside_others = false) {
  cudaError_t e;
  // the exact-order GEMV keeps the M rows of x in shared memory (at most 96 KB); beyond
  // that, shapes the tensor-core kernel accepts fall through to it
  const bool gemv_fits = K % 8 == 0 && static_cast<size_t>(M) * K * 2 <= 98304;
  if (M <= 8 && (gemv_fits || K % 16 || N % 16)) {
    if (!gemv_fits) return fail(Q4T_ERR_INVALID, "K must be a multiple of 8 and M*K at most 49152");
    if ((e = q4t::launch_small_m_linear(x, w, y, M, N, K, st)) != cudaSuccess) return fail_cuda("linear launch", e);
    return Q4T_OK;
  }
  if (K % 16 || N % 16) return fail(Q4T_ERR_INVALID, "K and N must be multiples of 16");
  // one tile of token rows: a kernel that loads four k-blocks at a time (a handful of CTAs are
  // bound by how fast one thread issues TMA loads, not by bandwidth)
  if (!no_small_m_gemm() && q4t::bf16_small_m_fits(M, N, K)) {
    CUtensorMap tx, tw;
    int rc3;
    if ((rc3 = make_tmap_kblocks(ds, &tx, x, K, M, q4t::bf16_small_m_box_rows(M), 4)) != Q4T_OK) return rc3;
    if ((rc3 = make_tmap_kblocks(ds, &tw, w, K, N, 64, 4)) != Q4T_OK) return rc3;
    if ((e = q4t::launch_bf16_small_m(tx, tw, y, M, N, K, ds->num_sms, beside_others, st)) != cudaSuccess) return fail_cuda("bf16 small-M GEMM launch", e);
    return Q4T_OK;
  }
  // few wide tiles would leave most SMs idle: use 64-column tiles then
  const int m_tiles = (M + 127) / 128;
  const bool narrow = m_tiles * ((N + 255) / 256) < ds->num_sms / 2 && N % 64 == 0;
  const int cols = narrow ? 64 : 256;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap(ds, &ta, true, x, K, M, static_cast<uint64_t>(K) * 2)) != Q4T_OK) return rc;
  if ((rc = make_tmap(ds, &tb, true, w, K, N, static_cast<uint64_t>(K) * 2, cols / 2)) != Q4T_OK) return rc;
  q4t::GemmArgs g{};
  g.K = K;
  g.tile_cols = cols;
  g.n_tiles = (N + cols - 1) / cols;
  g.n_per_tile = cols;
  g.b_rows_valid = N;
  g.ntiles_host = m_tiles;
  g.total_rows = M;
  g.out = y;
  g.ldo = N;
  g.alpha_const = 1.0f;
  e = (!narrow && M >= pair_min_rows()) ? q4t::launch_gemm_bf16_pair(ta, tb, g, q4t::Epilogue::kStoreBf16, ds->num_sms, st)
                                        : q4t::launch_gemm_bf16(ta, tb, g, q4t::Epilogue::kStoreBf16, ds->num_sms, st);
  if (e != cudaSuccess) return fail_cuda("bf16 GEMM launch", e);
  return Q4T_OK;
}

// Shared expert: act = bf16((g*sigmoid(g))*u) of bf16(x.Wgu^T), down = bf16(act.Wd^T)
// (src/model/moe.cu:955-969).  T <= 8 uses the reference-order GEMV, larger T the tensor cores.
int run_shared_expert(const DeviceState* ds, const uint16_t* x, const q4t_extra_weights* extra, uint16_t* sgu,
                      uint16_t* sact, uint16_t* sdown, int T, uint32_t flags, cudaStream_t st) {
  const int hs = extra->hs, sis = extra->shared_is;
  cudaError_t e;
  int rc;
  if (T <= 8) {
    if ((rc = run_bf16_linear(ds, x, extra->shared_gu, sgu, T, 2 * sis, hs, st)) != Q4T_OK) return rc;
    if ((e = q4t::launch_swiglu(sgu, sact, T, sis, st)) != cudaSuccess) return fail_cuda("swiglu launch", e);
  } else if (!no_small_m_gemm() && q4t::bf16_small_m_swiglu_fits(T, sis, hs)) {
    // one tile of token rows: the kernel that loads four k-blocks per TMA operation
    CUtensorMap tx, tw;
    if ((rc = make_tmap_kblocks(ds, &tx, x, hs, T, q4t::bf16_small_m_box_rows(T), 4)) != Q4T_OK) return rc;
    if ((rc = make_tmap_kblocks_gate_up(ds, &tw, extra->shared_gu, hs, sis, 4)) != Q4T_OK) return rc;
    if ((e = q4t::launch_bf16_small_m_swiglu(tx, tw, sact, T, sis, hs, (flags & 1u) ? sgu : nullptr, ds->num_sms, st)) != cudaSuccess)
      return fail_cuda("shared gate/up launch", e);
  } else {
    const int m_tiles = (T + 127) / 128;
    const bool narrow = m_tiles * (sis / 128) < ds->num_sms / 2;
    const int cols = narrow ? 64 : 256;
    CUtensorMap ta, tb;
    if ((rc = make_tmap(ds, &ta, true, x, hs, T, static_cast<uint64_t>(hs) * 2)) != Q4T_OK) return rc;
    if ((rc = make_tmap(ds, &tb, true, extra->shared_gu, hs, 2 * sis, static_cast<uint64_t>(hs) * 2, cols / 2)) !=
        Q4T_OK)
      return rc;
    q4t::GemmArgs g{};
    g.K = hs;
    g.tile_cols = cols;
    g.n_tiles = sis / (cols / 2);
    g.n_per_tile = cols / 2;
    g.up_row_offset = sis;
    g.b_rows_valid = sis;
    g.ntiles_host = m_tiles;
    g.total_rows = T;
    g.out = sact;
    g.ldo = sis;
    g.alpha_const = 1.0f;
    g.gu_dump = (flags & 1u) ? sgu : nullptr;
    g.gu_dump_ld = 2 * sis;
    e = (!narrow && T >= pair_min_rows()) ? q4t::launch_gemm_bf16_pair(ta, tb, g, q4t::Epilogue::kSwigluBf16, ds->num_sms, st)
                                          : q4t::launch_gemm_bf16(ta, tb, g, q4t::Epilogue::kSwigluBf16, ds->num_sms, st);
    if (e != cudaSuccess) return fail_cuda("shared gate/up GEMM launch", e);
  }
  return run_bf16_linear(ds, sact, extra->shared_down, sdown, T, hs, sis, st, true);
}

}  // namespace

extern "C" {

const char* q4t_last_error(void) { return g_error.c_str(); }
const char* q4t_version(void) { return "q4t-moe-b200 0.1 (sm_100a)"; }

int32_t q4t_set_pair_min_rows(int64_t rows) {
  g_pair_min_rows.store(rows <= 0 ? kPairNever : rows, std::memory_order_relaxed);
  return Q4T_OK;
}

int32_t q4t_sf_num_gtiles(int32_t K) { return (K / 16 + 3) / 4; }
size_t q4t_sf_buffer_size(int32_t rows, int32_t K) { return sf_buffer_size(rows, K); }
size_t q4t_sf_offset(int32_t row, int32_t group, int32_t num_g_tiles) {
  return static_cast<size_t>(row % 32) * 16 + static_cast<size_t>((row % 128) / 32) * 4 + group % 4 +
         static_cast<size_t>(group / 4) * 512 + static_cast<size_t>(row / 128) * num_g_tiles * 512;
}

int32_t q4t_pack_expert_host(const uint8_t* gate_w, const uint8_t* up_w, const uint8_t* down_w,
                             const uint8_t* gate_s, const uint8_t* up_s, const uint8_t* down_s,
                             int32_t hs, int32_t moe_is, uint8_t* gu_packed_e, uint8_t* gu_sf_e,
                             uint8_t* dn_packed_e, uint8_t* dn_sf_e) {
  if (hs <= 0 || moe_is <= 0) return fail(Q4T_ERR_INVALID, "invalid MoE dims");
  if (hs % 32 || moe_is % 32) return fail(Q4T_ERR_INVALID, "hs and moe_is must be multiples of 32 (FP4 GEMM)");
  if ((2 * moe_is) % 128 || hs % 128)
    return fail(Q4T_ERR_INVALID, "2*moe_is and hs must be multiples of 128 (per-expert SF blocks)");
  if (!gate_w || !up_w || !down_w || !gate_s || !up_s || !down_s || !gu_packed_e || !gu_sf_e || !dn_packed_e ||
      !dn_sf_e)
    return fail(Q4T_ERR_INVALID, "null tensor pointer");
  const size_t gw = static_cast<size_t>(moe_is) * (hs / 2);
  std::memcpy(gu_packed_e, gate_w, gw);
  std::memcpy(gu_packed_e + gw, up_w, gw);
  std::memcpy(dn_packed_e, down_w, static_cast<size_t>(hs) * (moe_is / 2));
  const int ggu = hs / 16, gdn = moe_is / 16;
  const int ntgu = (ggu + 3) / 4, ntdn = (gdn + 3) / 4;
  std::memset(gu_sf_e, 0, sf_buffer_size(2 * moe_is, hs));
  std::memset(dn_sf_e, 0, sf_buffer_size(hs, moe_is));
  for (int r = 0; r < 2 * moe_is; ++r) {
    const uint8_t* src = r < moe_is ? gate_s + static_cast<size_t>(r) * ggu
                                    : up_s + static_cast<size_t>(r - moe_is) * ggu;
    for (int g = 0; g < ggu; ++g) gu_sf_e[q4t_sf_offset(r, g, ntgu)] = src[g];
  }
  for (int r = 0; r < hs; ++r)
    for (int g = 0; g < gdn; ++g) dn_sf_e[q4t_sf_offset(r, g, ntdn)] = down_s[static_cast<size_t>(r) * gdn + g];
  return Q4T_OK;
}

int32_t q4t_quantize_activation_fp4(const uint16_t* bf16, uint8_t* packed_out, uint8_t* sf_out, int32_t M,
                                    int32_t K, float global_scale, void* stream) {
  if (M < 0 || K <= 0 || K % 16) return fail(Q4T_ERR_INVALID, "K must be a positive multiple of 16");
  if (M == 0) return Q4T_OK;
  if (!bf16 || !packed_out || !sf_out) return fail(Q4T_ERR_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(bf16) & 15u) return fail(Q4T_ERR_INVALID, "input must be 16-byte aligned");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  cudaError_t e = q4t::launch_quantize(bf16, packed_out, sf_out, M, K, global_scale, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("quantise launch", e);
}

int32_t q4t_dequant_fp4_to_bf16(const uint8_t* packed, const uint8_t* group_scale, uint16_t* bf16_out,
                                float inv_global_scale, int32_t N, int32_t K, void* stream) {
  if (N < 0 || K <= 0 || K % 16) return fail(Q4T_ERR_INVALID, "K must be a positive multiple of 16");
  if (N == 0) return Q4T_OK;
  if (!packed || !group_scale || !bf16_out) return fail(Q4T_ERR_INVALID, "null pointer");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  cudaError_t e = q4t::launch_dequant(packed, group_scale, bf16_out, inv_global_scale, N, K,
                                      static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("dequant launch", e);
}

int32_t q4t_fp4_gemm(const uint8_t* w_packed, const uint8_t* w_sf, const uint8_t* a_packed,
                     const uint8_t* a_sf, void* out, int32_t out_is_bf16, int32_t M, int32_t N, int32_t K,
                     float inv_w_global, float inv_a_global, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(Q4T_ERR_INVALID, "invalid GEMM dims");
  if (K % 64 || N % 16) return fail(Q4T_ERR_INVALID, "K must be a multiple of 64 and N of 16");
  if (!w_packed || !w_sf || !a_packed || !a_sf || !out) return fail(Q4T_ERR_INVALID, "null pointer");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  CUtensorMap ta, tb;
  if ((rc = make_tmap(ds, &ta, false, a_packed, K / 2, M, K / 2)) != Q4T_OK) return rc;
  if ((rc = make_tmap(ds, &tb, false, w_packed, K / 2, N, K / 2)) != Q4T_OK) return rc;
  q4t::GemmArgs g{};
  g.K = K;
  g.n_tiles = (N + 255) / 256;
  g.n_per_tile = 256;
  g.b_rows_valid = N;
  g.ntiles_host = (M + 127) / 128;
  g.total_rows = M;
  g.sfa_tiles = a_sf;
  g.sfb = w_sf;
  g.out = out;
  g.ldo = N;
  g.alpha_const = inv_w_global * inv_a_global;  // include/q4t/quant/fp4_gemm.h:205
#ifdef Q4T_TRACE
  if (const char* t = std::getenv("Q4T_TRACE_PTR")) g.trace = reinterpret_cast<long long*>(std::strtoull(t, nullptr, 0));
#endif
  const q4t::Epilogue epi = out_is_bf16 ? q4t::Epilogue::kStoreBf16 : q4t::Epilogue::kStoreF32;
  cudaError_t e;
  if (M >= pair_min_rows()) {  // large M: CTA pairs share the weight tiles
    const uint64_t ntk = static_cast<uint64_t>(K + 63) / 64;
    CUtensorMap tsa, tsb;
    if ((rc = make_sf_tmap(ds, &tsa, a_sf, static_cast<uint64_t>((M + 127) / 128) * ntk)) != Q4T_OK) return rc;
    if ((rc = make_sf_tmap(ds, &tsb, w_sf, static_cast<uint64_t>((N + 127) / 128) * ntk)) != Q4T_OK) return rc;
    e = q4t::launch_gemm_nvf4_pair(ta, tb, tsa, tsb, g, epi, ds->num_sms, static_cast<cudaStream_t>(stream));
  } else {
    e = q4t::launch_gemm_nvf4(ta, tb, g, epi, ds->num_sms, static_cast<cudaStream_t>(stream));
  }
  return e == cudaSuccess ? Q4T_OK : fail_cuda("NVFP4 GEMM launch", e);
}

int32_t q4t_router_topk(const uint16_t* logits, int32_t* expert_ids, float* router_w, int32_t T, int32_t E,
                        int32_t k, void* stream) {
  if (T <= 0) return Q4T_OK;
  if (k <= 0 || k > 16) return fail(Q4T_ERR_INVALID, "k out of range");
  if (E <= 0 || E > 512 || k > E) return fail(Q4T_ERR_INVALID, "E out of range (1..512, >= k)");
  if (!logits || !expert_ids || !router_w) return fail(Q4T_ERR_INVALID, "null pointer");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  cudaError_t e = q4t::launch_topk(logits, nullptr, expert_ids, router_w, T, E, k, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("topk launch", e);
}

int32_t q4t_bf16_linear(const uint16_t* x, const uint16_t* w, uint16_t* y, int32_t M, int32_t N, int32_t K,
                        void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return fail(Q4T_ERR_INVALID, "invalid GEMM dims");
  if (!x || !w || !y) return fail(Q4T_ERR_INVALID, "null pointer");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  return run_bf16_linear(ds, x, w, y, M, N, K, static_cast<cudaStream_t>(stream));
}

size_t q4t_moe_routed_workspace_bytes(int32_t M, int32_t k, int32_t hs, int32_t moe_is, int32_t E) {
  if (M <= 0 || k <= 0 || hs <= 0 || moe_is <= 0 || E <= 0) return 0;
  q4t_routed_ws_layout L;
  routed_layout(M, k, hs, moe_is, E, &L);
  return L.total;
}

int32_t q4t_moe_routed_workspace_layout(int32_t M, int32_t k, int32_t hs, int32_t moe_is, int32_t E,
                                        q4t_routed_ws_layout* out) {
  if (M <= 0 || k <= 0 || hs <= 0 || moe_is <= 0 || E <= 0 || !out) return fail(Q4T_ERR_INVALID, "invalid MoE forward dims");
  routed_layout(M, k, hs, moe_is, E, out);
  return Q4T_OK;
}

int32_t q4t_moe_routed_forward(const uint16_t* x, const int32_t* expert_ids, const float* router_w, float* y,
                               const q4t_routed_weights* w, void* workspace, size_t workspace_bytes, int32_t M,
                               int32_t k, uint32_t flags, void* stream) {
  if (!w) return fail(Q4T_ERR_INVALID, "null weights");
  if (M <= 0 || k <= 0 || w->E <= 0 || w->hs <= 0 || w->moe_is <= 0)
    return fail(Q4T_ERR_INVALID, "invalid MoE forward dims");  // src/quant/moe_gemm.cu:321-323
  if (!routed_dims_ok(w->E, w->hs, w->moe_is))
    return fail(Q4T_ERR_INVALID, "hs and moe_is must be multiples of 128 and E <= 1024");
  if (!x || !expert_ids || !router_w || !y || !workspace) return fail(Q4T_ERR_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(Q4T_ERR_INVALID, "workspace must be 256-byte aligned");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  RoutedPtrs P;
  routed_layout(M, k, w->hs, w->moe_is, w->E, &P.L);
  if (workspace_bytes < P.L.total) return fail(Q4T_ERR_WORKSPACE, "workspace too small");
  P.base = static_cast<uint8_t*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  stage_begin(st);
  stage_end(1, st);
  if ((rc = run_routed_core(ds, x, expert_ids, w, P, M, k, flags, st)) != Q4T_OK) return rc;
  cudaError_t e = q4t::launch_routed_combine(P.at<uint16_t>(P.L.dn_out), P.at<int32_t>(P.L.row_of_flat), router_w,
                                             y, M, k, w->hs, st);
  stage_end(6, st);
  stage_end(7, st);
  return e == cudaSuccess ? Q4T_OK : fail_cuda("combine launch", e);
}

size_t q4t_moe_forward_workspace_bytes(int32_t T, int32_t k, int32_t hs, int32_t moe_is, int32_t shared_is,
                                       int32_t E) {
  if (T <= 0 || k <= 0 || hs <= 0 || moe_is <= 0 || shared_is <= 0 || E <= 0) return 0;
  q4t_forward_ws_layout F;
  forward_layout(T, k, hs, moe_is, shared_is, E, &F);
  return F.total;
}

int32_t q4t_moe_forward_workspace_layout(int32_t T, int32_t k, int32_t hs, int32_t moe_is, int32_t shared_is,
                                         int32_t E, q4t_forward_ws_layout* out) {
  if (T <= 0 || k <= 0 || hs <= 0 || moe_is <= 0 || shared_is <= 0 || E <= 0 || !out)
    return fail(Q4T_ERR_INVALID, "invalid MoE forward dims");
  forward_layout(T, k, hs, moe_is, shared_is, E, out);
  return Q4T_OK;
}

}  // extern "C"

namespace {
// The whole layer for either kind of routed experts (exactly one of routed / routed_bf16 is set).
// trace_ids_out (optional): the selected expert ids are copied there right after the top-k.
// slot_of_expert (optional, NVFP4 only): the routed weights hold `routed->E` resident slots
// and expert id e runs as slot slot_of_expert[e] (negative: skipped).
int moe_forward_impl(const uint16_t* x, const q4t_routed_weights* routed, const q4t_bf16_expert_weights* routed_bf16,
                     const q4t_extra_weights* extra, uint16_t* y, int32_t T, int32_t k, void* workspace,
                     size_t workspace_bytes, const int32_t* fixed_ids, int32_t* trace_ids_out,
                     const int32_t* slot_of_expert, uint32_t flags, void* stream,
                     const q4t::HcWrite& hcw = q4t::HcWrite{}, const q4t::NormWrite& nw = q4t::NormWrite{}) {
  if (T <= 0) return Q4T_OK;                                           // src/model/moe.cu:442
  if (k <= 0 || k > 16) return fail(Q4T_ERR_INVALID, "k out of range");  // moe.cu:443
  if ((!routed && !routed_bf16) || !extra) return fail(Q4T_ERR_INVALID, "null weights");
  const int E = extra->E, hs = extra->hs, sis = extra->shared_is;
  const int is = routed ? routed->moe_is : routed_bf16->moe_is;
  const int E_routed = routed ? routed->E : routed_bf16->E;
  if (slot_of_expert && !routed) return fail(Q4T_ERR_INVALID, "slot mode needs NVFP4 routed weights");
  if ((routed ? routed->hs : routed_bf16->hs) != hs || (!slot_of_expert && E_routed != E))
    return fail(Q4T_ERR_INVALID, "routed and extra weights disagree on E/hs");
  if (slot_of_expert && (E_routed <= 0 || E_routed > E))
    return fail(Q4T_ERR_INVALID, "slot count must be in [1, number of experts]");
  if (!routed_dims_ok(E, hs, is) || E > 512 || k > E || sis <= 0 || sis % 128)
    return fail(Q4T_ERR_INVALID, "unsupported dims (hs, moe_is, shared_is multiples of 128; E <= 512)");
  q4t_forward_ws_layout F;
  forward_layout(T, k, hs, is, sis, E, &F);
  // BF16 experts: the gathered bf16 rows [T*k, hs] follow the regions of the NVFP4 layout
  const size_t compact_at = F.total;
  if (routed_bf16) F.total = align_up(compact_at + static_cast<size_t>(T) * k * hs * 2, 256);
  if (workspace_bytes < F.total) return fail(Q4T_ERR_WORKSPACE, "workspace too small");  // moe.cu:444-447
  if (!x || !y || !workspace) return fail(Q4T_ERR_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(Q4T_ERR_INVALID, "workspace must be 256-byte aligned");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(workspace);
  uint16_t* logits = reinterpret_cast<uint16_t*>(base + F.logits);
  int32_t* ids = reinterpret_cast<int32_t*>(base + F.expert_ids);
  float* rw = reinterpret_cast<float*>(base + F.router_w);
  // the fp32 routed sum is a diagnostic region: written only on request (flags bit 1)
  float* routed_f32 = (flags & 2u) ? reinterpret_cast<float*>(base + F.routed) : nullptr;
  uint16_t* sgu = reinterpret_cast<uint16_t*>(base + F.shared_gu);
  uint16_t* sact = reinterpret_cast<uint16_t*>(base + F.shared_act);
  uint16_t* sdown = reinterpret_cast<uint16_t*>(base + F.shared_down);
  cudaError_t e;

  // The shared expert runs beside the routed chain unless the stage timer is on
  // (its marks assume one stream) or the batch is large enough to fill the GPU.
  // (forking at 4096 and 16 384 tokens measured within 1.3 % of not forking)
  const bool fork = !g_timer.enabled && T <= 1024;
  // Once the side stream has been forked, every way out joins it again: an error
  // return that left it dangling would, under stream capture, invalidate the graph.
  bool forked = false;
  auto leave = [&](int code) {
    if (forked) {
      const std::string kept = g_error;
      if (cudaEventRecord(ds->join_event, ds->side_stream) == cudaSuccess) cudaStreamWaitEvent(st, ds->join_event, 0);
      g_error = kept;
    }
    return code;
  };
  if (fork) {
    if ((e = cudaEventRecord(ds->fork_event, st)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(ds->side_stream, ds->fork_event, 0)) != cudaSuccess)
      return fail_cuda("fork", e);
    forked = true;
    q4t::chain_break();  // first kernel behind an event wait
    if ((rc = run_shared_expert(ds, x, extra, sgu, sact, sdown, T, flags, ds->side_stream)) != Q4T_OK) return leave(rc);
    if ((e = cudaEventRecord(ds->join_event, ds->side_stream)) != cudaSuccess) return leave(fail_cuda("join record", e));
    q4t::chain_break();  // back on the caller's stream, behind the caller's own work
  }

  // 1-2. router logits and top-k
  stage_begin(st);
  if ((rc = run_bf16_linear(ds, x, extra->gate, logits, T, E, hs, st)) != Q4T_OK) return leave(rc);
  stage_end(0, st);
  RoutedPtrs P;
  routed_layout(T, k, hs, is, E, &P.L);
  P.base = base + F.routed_ws;
  const bool observe = trace_ids_out != nullptr || slot_of_expert != nullptr;
  // decode-sized NVFP4 batches need no permutation tables
  const bool small = routed && small_batch_applies(T, k, routed->E, hs, is, flags);
  const bool fused_route = !observe && !small && q4t::route_and_plan_fits(T, k);
  static const bool no_cluster_route = std::getenv("Q4T_NO_CLUSTER_ROUTE") != nullptr;
  const bool cluster_route = !observe && !small && !fused_route && !no_cluster_route &&
                             static_cast<int64_t>(T) * k < pair_min_rows() && q4t::route_plan_cluster_fits(T, k, E);
  if (fused_route) {  // small batch: top-k and the permutation tables in one launch
    if ((e = q4t::launch_route_and_plan(logits, fixed_ids, ids, rw, T, E, k, static_cast<int>(P.L.max_tiles),
                                        plan_tables(P, E), st)) != cudaSuccess)
      return leave(fail_cuda("route+plan launch", e));
  } else if (cluster_route) {  // up to 256 tokens: the same by a cluster of eight CTAs
    if ((e = q4t::launch_route_plan_cluster(logits, fixed_ids, ids, rw, T, E, k, static_cast<int>(P.L.max_tiles),
                                            plan_tables(P, E), st)) != cudaSuccess)
      return leave(fail_cuda("route+plan launch", e));
  } else {
    if ((e = q4t::launch_topk(logits, fixed_ids, ids, rw, T, E, k, st)) != cudaSuccess)
      return leave(fail_cuda("topk launch", e));
  }
  // the router-trace observer sees the experts as selected (src/model/moe.cu:485-488,
  // RouterCollector::CaptureLayer: a device-to-device copy of [T,k] ids on the stream)
  if (trace_ids_out) {
    if ((e = cudaMemcpyAsync(trace_ids_out, ids, static_cast<size_t>(T) * k * 4, cudaMemcpyDeviceToDevice, st)) !=
        cudaSuccess)
      return leave(fail_cuda("trace copy", e));
    q4t::chain_break();
  }
  // slot mode (include/q4t/quant/moe_weights.h:47-51): the GEMMs consume slot ids; the
  // workspace keeps the original ids in `expert_ids` and the slots in `slot_ids`
  const int32_t* routed_ids = ids;
  if (slot_of_expert) {
    int32_t* slots = reinterpret_cast<int32_t*>(base + F.slot_ids);
    if ((e = q4t::launch_remap_ids(ids, slot_of_expert, slots, T * k, E, E_routed, st)) != cudaSuccess)
      return leave(fail_cuda("slot remap launch", e));
    routed_ids = slots;
  }
  stage_end(1, st);

  // 3. routed experts
  if (routed) {
    if ((rc = run_routed_core(ds, x, routed_ids, routed, P, T, k, flags, st, fused_route || cluster_route)) != Q4T_OK) return leave(rc);
  } else if ((rc = run_routed_core_bf16(ds, x, ids, routed_bf16, P, reinterpret_cast<uint16_t*>(base + compact_at), T, k,
                                        st, fused_route || cluster_route)) != Q4T_OK) {
    return leave(rc);
  }

  // 4-6. shared expert
  if (fork) {
    if ((e = cudaStreamWaitEvent(st, ds->join_event, 0)) != cudaSuccess) return fail_cuda("join", e);
    forked = false;
    q4t::chain_break();
  } else {
    if ((rc = run_shared_expert(ds, x, extra, sgu, sact, sdown, T, flags, st)) != Q4T_OK) return rc;
  }
  stage_end(6, st);

  // 7. routed sum + sigmoid-gated shared expert
  if ((e = q4t::launch_final_combine(P.at<uint16_t>(P.L.dn_out), P.at<int32_t>(P.L.row_of_flat), rw, sdown, x,
                                     extra->shared_gate_scalar, routed_f32, y, T, k, hs, st, hcw, nw)) != cudaSuccess)
    return fail_cuda("combine launch", e);
  stage_end(7, st);
  return Q4T_OK;
}
}  // namespace

extern "C" {

int32_t q4t_moe_forward(const uint16_t* x, const q4t_routed_weights* routed, const q4t_extra_weights* extra,
                        uint16_t* y, int32_t T, int32_t k, void* workspace, size_t workspace_bytes,
                        const int32_t* fixed_ids, uint32_t flags, void* stream) {
  if (T > 0 && k > 0 && k <= 16 && !routed) return fail(Q4T_ERR_INVALID, "null weights");
  return moe_forward_impl(x, routed, nullptr, extra, y, T, k, workspace, workspace_bytes, fixed_ids, nullptr, nullptr,
                          flags, stream);
}

int32_t q4t_moe_forward_ex(const uint16_t* x, const q4t_routed_weights* routed, const q4t_extra_weights* extra,
                           uint16_t* y, int32_t T, int32_t k, void* workspace, size_t workspace_bytes,
                           const q4t_forward_options* opt, void* stream) {
  if (T > 0 && k > 0 && k <= 16 && !routed) return fail(Q4T_ERR_INVALID, "null weights");
  if (!opt) return fail(Q4T_ERR_INVALID, "null options");
  q4t::HcWrite hcw{};
  if (opt->hc_count != 0) {
    if (opt->hc_count < 0 || opt->hc_count > 16 || !opt->hc_residual || !opt->hc_inject_gate || !opt->hc_out)
      return fail(Q4T_ERR_INVALID, "gated residual write: 1..16 branches and three non-null buffers");
    if ((reinterpret_cast<uintptr_t>(opt->hc_residual) | reinterpret_cast<uintptr_t>(opt->hc_out)) & 15u)
      return fail(Q4T_ERR_INVALID, "gated residual write: buffers must be 16-byte aligned");
    hcw = q4t::HcWrite{opt->hc_residual, opt->hc_inject_gate, opt->hc_out, opt->hc_count};
  }
  q4t::NormWrite nw{};
  if (opt->norm_residual) {
    if (!opt->norm_out || opt->norm_out == opt->norm_residual)
      return fail(Q4T_ERR_INVALID, "residual + RMSNorm write: two distinct non-null buffers");
    if ((reinterpret_cast<uintptr_t>(opt->norm_residual) | reinterpret_cast<uintptr_t>(opt->norm_out)) & 15u)
      return fail(Q4T_ERR_INVALID, "residual + RMSNorm write: buffers must be 16-byte aligned");
    if (extra && (extra->hs > q4t::kNormWriteMaxHs || extra->hs % 8))
      return fail(Q4T_ERR_INVALID, "residual + RMSNorm write: hs must be a multiple of 8, at most 8192");
    nw = q4t::NormWrite{opt->norm_residual, opt->norm_out, opt->norm_eps};
  }
  return moe_forward_impl(x, routed, nullptr, extra, y, T, k, workspace, workspace_bytes, opt->fixed_ids,
                          opt->trace_ids_out, opt->slot_of_expert, opt->flags, stream, hcw, nw);
}

// ---- BF16 routed experts (the MTP draft layer)
size_t q4t_moe_bf16_workspace_bytes(int32_t M, int32_t k, int32_t hs, int32_t moe_is, int32_t E) {
  if (M <= 0 || k <= 0 || !routed_dims_ok(E, hs, moe_is)) return 0;
  q4t_routed_ws_layout L;
  routed_layout(M, k, hs, moe_is, E, &L);
  return align_up(L.total, 256) + align_up(static_cast<size_t>(M) * k * hs * 2, 256);
}

int32_t q4t_moe_bf16_routed_forward(const uint16_t* x, const int32_t* expert_ids, const float* router_w, float* y,
                                    const q4t_bf16_expert_weights* w, void* workspace, size_t workspace_bytes,
                                    int32_t M, int32_t k, void* stream) {
  if (!w) return fail(Q4T_ERR_INVALID, "null weights");
  if (M <= 0 || k <= 0 || w->E <= 0 || w->hs <= 0 || w->moe_is <= 0) return fail(Q4T_ERR_INVALID, "invalid MoE forward dims");
  if (!routed_dims_ok(w->E, w->hs, w->moe_is))
    return fail(Q4T_ERR_INVALID, "hs and moe_is must be multiples of 128 and E <= 1024");
  if (!x || !expert_ids || !router_w || !y || !workspace || !w->gu || !w->down) return fail(Q4T_ERR_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(Q4T_ERR_INVALID, "workspace must be 256-byte aligned");
  if (workspace_bytes < q4t_moe_bf16_workspace_bytes(M, k, w->hs, w->moe_is, w->E))
    return fail(Q4T_ERR_WORKSPACE, "workspace too small");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  RoutedPtrs P;
  routed_layout(M, k, w->hs, w->moe_is, w->E, &P.L);
  P.base = static_cast<uint8_t*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  stage_begin(st);
  stage_end(1, st);
  uint16_t* compact = reinterpret_cast<uint16_t*>(P.base + align_up(P.L.total, 256));
  if ((rc = run_routed_core_bf16(ds, x, expert_ids, w, P, compact, M, k, st, false)) != Q4T_OK) return rc;
  cudaError_t e = q4t::launch_routed_combine(P.at<uint16_t>(P.L.dn_out), P.at<int32_t>(P.L.row_of_flat), router_w, y, M,
                                             k, w->hs, st);
  stage_end(7, st);
  return e == cudaSuccess ? Q4T_OK : fail_cuda("combine launch", e);
}

size_t q4t_moe_bf16_forward_workspace_bytes(int32_t T, int32_t k, int32_t hs, int32_t moe_is, int32_t shared_is,
                                            int32_t E) {
  if (T <= 0 || k <= 0 || shared_is <= 0 || !routed_dims_ok(E, hs, moe_is)) return 0;
  q4t_forward_ws_layout F;
  forward_layout(T, k, hs, moe_is, shared_is, E, &F);
  return align_up(F.total + static_cast<size_t>(T) * k * hs * 2, 256);
}

int32_t q4t_moe_bf16_forward(const uint16_t* x, const q4t_bf16_expert_weights* routed, const q4t_extra_weights* extra,
                             uint16_t* y, int32_t T, int32_t k, void* workspace, size_t workspace_bytes,
                             void* stream) {
  if (T > 0 && k > 0 && k <= 16 && (!routed || !routed->gu || !routed->down)) return fail(Q4T_ERR_INVALID, "null weights");
  return moe_forward_impl(x, nullptr, routed, extra, y, T, k, workspace, workspace_bytes, nullptr, nullptr, nullptr, 0,
                          stream);
}

// ---------------------------------------------------------------- expert parallelism
namespace {
struct EpDispatchLayout {
  size_t dest, local, offsets, flat_of_row, row_tile, ntiles, tile_expert, tile_row0, tile_nrows, tile_off,
      blk_counts, total;
  size_t max_tiles;
};
void ep_dispatch_layout(int T, int k, int n_ranks, EpDispatchLayout* L) {
  const size_t R = static_cast<size_t>(T) * k;
  const size_t nblk = (R + q4t::kPlanChunk - 1) / q4t::kPlanChunk;
  L->max_tiles = R / 128 + n_ranks + 1;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    off = align_up(off, 256);
    const size_t at = off;
    off += bytes;
    return at;
  };
  L->dest = take(R * 4);
  L->local = take(R * 4);
  L->offsets = take(static_cast<size_t>(n_ranks + 1) * 4);
  L->flat_of_row = take(R * 4);
  L->row_tile = take(R * 4);
  L->ntiles = take(256);
  L->tile_expert = take(L->max_tiles * 4);
  L->tile_row0 = take(L->max_tiles * 4);
  L->tile_nrows = take(L->max_tiles * 4);
  L->tile_off = take(static_cast<size_t>(n_ranks + 1) * 4);
  L->blk_counts = take(nblk * static_cast<size_t>(n_ranks) * 4);
  L->total = align_up(off, 256);
}
struct FinishLayout {
  size_t routed, shared_gu, shared_act, shared_down, total;
};
void finish_layout(int T, int hs, int sis, FinishLayout* F) {
  size_t off = 0;
  auto take = [&](size_t bytes) {
    off = align_up(off, 256);
    const size_t at = off;
    off += bytes;
    return at;
  };
  F->routed = take(static_cast<size_t>(T) * hs * 4);
  F->shared_gu = take(static_cast<size_t>(T) * 2 * sis * 2);
  F->shared_act = take(static_cast<size_t>(T) * sis * 2);
  F->shared_down = take(static_cast<size_t>(T) * hs * 2);
  F->total = align_up(off, 256);
}
}  // namespace

size_t q4t_ep_dispatch_workspace_bytes(int32_t T, int32_t k, int32_t n_ranks) {
  if (T <= 0 || k <= 0 || n_ranks <= 0) return 0;
  EpDispatchLayout L;
  ep_dispatch_layout(T, k, n_ranks, &L);
  return L.total;
}

int32_t q4t_ep_dispatch(const uint16_t* x, const int32_t* expert_ids, int32_t T, int32_t k, int32_t E, int32_t hs,
                        int32_t n_ranks, uint16_t* send_rows, int32_t* send_local_expert, int32_t* send_counts,
                        int32_t* row_of_flat, void* workspace, size_t workspace_bytes, void* stream) {
  if (T <= 0 || k <= 0 || E <= 0 || hs <= 0 || hs % 8 || n_ranks <= 0 || n_ranks > 1024 || E % n_ranks)
    return fail(Q4T_ERR_INVALID, "invalid dispatch dims (E must be a multiple of n_ranks, hs of 8)");
  if (!x || !expert_ids || !send_rows || !send_local_expert || !send_counts || !row_of_flat || !workspace)
    return fail(Q4T_ERR_INVALID, "null pointer");
  EpDispatchLayout L;
  ep_dispatch_layout(T, k, n_ranks, &L);
  if (workspace_bytes < L.total) return fail(Q4T_ERR_WORKSPACE, "workspace too small");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(workspace);
  auto at = [&](size_t off) { return reinterpret_cast<int32_t*>(base + off); };
  const int R = T * k;
  cudaError_t e;
  if ((e = q4t::launch_ep_split_ids(expert_ids, R, E, E / n_ranks, at(L.dest), at(L.local), st)) != cudaSuccess)
    return fail_cuda("split ids launch", e);
  q4t::PlanTables pt;
  pt.blk_counts = at(L.blk_counts);
  pt.counts = send_counts;
  pt.offsets = at(L.offsets);
  pt.tile_off = at(L.tile_off);
  pt.tile_expert = at(L.tile_expert);
  pt.tile_row0 = at(L.tile_row0);
  pt.tile_nrows = at(L.tile_nrows);
  pt.ntiles = at(L.ntiles);
  pt.row_of_flat = row_of_flat;
  pt.flat_of_row = at(L.flat_of_row);
  pt.row_tile = at(L.row_tile);
  pt.status = nullptr;
  if ((e = q4t::launch_plan(at(L.dest), R, n_ranks, static_cast<int>(L.max_tiles), pt, st)) != cudaSuccess)
    return fail_cuda("dispatch plan launch", e);
  // rows in destination order: source token = flat / k; the expert's index on its owner rides along
  if ((e = q4t::launch_gather_rows(x, pt.flat_of_row, k, pt.offsets + n_ranks, R, hs, send_rows, at(L.local),
                                   send_local_expert, st)) != cudaSuccess)
    return fail_cuda("dispatch gather launch", e);
  return Q4T_OK;
}

int32_t q4t_moe_expert_rows(const uint16_t* x_rows, const int32_t* local_expert, uint16_t* out_rows,
                            const q4t_routed_weights* w, void* workspace, size_t workspace_bytes, int32_t rows,
                            uint32_t flags, void* stream) {
  if (rows == 0) return Q4T_OK;
  if (!w) return fail(Q4T_ERR_INVALID, "null weights");
  if (rows < 0 || w->E <= 0 || w->hs <= 0 || w->moe_is <= 0) return fail(Q4T_ERR_INVALID, "invalid MoE forward dims");
  if (!routed_dims_ok(w->E, w->hs, w->moe_is))
    return fail(Q4T_ERR_INVALID, "hs and moe_is must be multiples of 128 and E <= 1024");
  if (!x_rows || !local_expert || !out_rows || !workspace) return fail(Q4T_ERR_INVALID, "null pointer");
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(Q4T_ERR_INVALID, "workspace must be 256-byte aligned");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  RoutedPtrs P;
  routed_layout(rows, 1, w->hs, w->moe_is, w->E, &P.L);
  if (workspace_bytes < P.L.total) return fail(Q4T_ERR_WORKSPACE, "workspace too small");
  P.base = static_cast<uint8_t*>(workspace);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  stage_begin(st);
  stage_end(1, st);
  if ((rc = run_routed_core(ds, x_rows, local_expert, w, P, rows, 1, flags, st)) != Q4T_OK) return rc;
  // back to the order the rows arrived in
  cudaError_t e = q4t::launch_gather_rows(P.at<uint16_t>(P.L.dn_out), P.at<int32_t>(P.L.row_of_flat), 1, nullptr, rows,
                                          w->hs, out_rows, nullptr, nullptr, st);
  stage_end(7, st);
  return e == cudaSuccess ? Q4T_OK : fail_cuda("row gather launch", e);
}

size_t q4t_moe_finish_workspace_bytes(int32_t T, int32_t hs, int32_t shared_is) {
  if (T <= 0 || hs <= 0 || shared_is <= 0) return 0;
  FinishLayout F;
  finish_layout(T, hs, shared_is, &F);
  return F.total;
}

namespace {
int finish_args_ok(const q4t_extra_weights* extra, int T, int k, const void* workspace, size_t workspace_bytes,
                   FinishLayout* F) {
  if (k <= 0 || k > 16) return fail(Q4T_ERR_INVALID, "k out of range");
  if (!extra || extra->hs <= 0 || extra->hs % 128 || extra->shared_is <= 0 || extra->shared_is % 128)
    return fail(Q4T_ERR_INVALID, "unsupported dims (hs, shared_is multiples of 128)");
  if (!workspace) return fail(Q4T_ERR_INVALID, "null pointer");
  finish_layout(T, extra->hs, extra->shared_is, F);
  if (workspace_bytes < F->total) return fail(Q4T_ERR_WORKSPACE, "workspace too small");
  return Q4T_OK;
}
}  // namespace

int32_t q4t_moe_shared_expert(const uint16_t* x, const q4t_extra_weights* extra, int32_t T, void* workspace,
                              size_t workspace_bytes, void* stream) {
  if (T <= 0) return Q4T_OK;
  FinishLayout F;
  int rc = finish_args_ok(extra, T, 1, workspace, workspace_bytes, &F);
  if (rc != Q4T_OK) return rc;
  if (!x) return fail(Q4T_ERR_INVALID, "null pointer");
  const DeviceState* ds;
  if ((rc = device_state(&ds)) != Q4T_OK) return rc;
  uint8_t* base = static_cast<uint8_t*>(workspace);
  return run_shared_expert(ds, x, extra, reinterpret_cast<uint16_t*>(base + F.shared_gu),
                           reinterpret_cast<uint16_t*>(base + F.shared_act),
                           reinterpret_cast<uint16_t*>(base + F.shared_down), T, 0, static_cast<cudaStream_t>(stream));
}

int32_t q4t_moe_combine(const uint16_t* x, const uint16_t* expert_rows, const int32_t* row_of_flat,
                        const float* router_w, const q4t_extra_weights* extra, uint16_t* y, int32_t T, int32_t k,
                        void* workspace, size_t workspace_bytes, void* stream) {
  if (T <= 0) return Q4T_OK;
  FinishLayout F;
  int rc = finish_args_ok(extra, T, k, workspace, workspace_bytes, &F);
  if (rc != Q4T_OK) return rc;
  if (!x || !expert_rows || !row_of_flat || !router_w || !y) return fail(Q4T_ERR_INVALID, "null pointer");
  const DeviceState* ds;
  if ((rc = device_state(&ds)) != Q4T_OK) return rc;
  uint8_t* base = static_cast<uint8_t*>(workspace);
  cudaError_t e = q4t::launch_final_combine(expert_rows, row_of_flat, router_w,
                                            reinterpret_cast<uint16_t*>(base + F.shared_down), x,
                                            extra->shared_gate_scalar, reinterpret_cast<float*>(base + F.routed), y, T,
                                            k, extra->hs, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("combine launch", e);
}

int32_t q4t_moe_finish(const uint16_t* x, const uint16_t* expert_rows, const int32_t* row_of_flat,
                       const float* router_w, const q4t_extra_weights* extra, uint16_t* y, int32_t T, int32_t k,
                       void* workspace, size_t workspace_bytes, void* stream) {
  if (T <= 0) return Q4T_OK;
  if (k <= 0 || k > 16) return fail(Q4T_ERR_INVALID, "k out of range");
  int rc = q4t_moe_shared_expert(x, extra, T, workspace, workspace_bytes, stream);
  if (rc != Q4T_OK) return rc;
  return q4t_moe_combine(x, expert_rows, row_of_flat, router_w, extra, y, T, k, workspace, workspace_bytes, stream);
}

// ---- pull/push expert parallelism over peer memory
int32_t q4t_peer_buffer_alloc(size_t bytes, void** ptr) {
  if (!ptr || bytes == 0) return fail(Q4T_ERR_INVALID, "invalid arguments");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  cudaError_t e = cudaMalloc(ptr, align_up(bytes, 256));
  if (e != cudaSuccess) return fail_cuda("peer buffer allocation", e);
  // zero-filled (a sync buffer's flags must start at zero); completes before the call returns
  if ((e = cudaMemset(*ptr, 0, align_up(bytes, 256))) != cudaSuccess || (e = cudaDeviceSynchronize()) != cudaSuccess) {
    cudaFree(*ptr);
    *ptr = nullptr;
    return fail_cuda("peer buffer clear", e);
  }
  return Q4T_OK;
}
int32_t q4t_peer_buffer_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  return e == cudaSuccess ? Q4T_OK : fail_cuda("peer buffer free", e);
}
int32_t q4t_peer_buffer_export(const void* ptr, uint8_t handle[Q4T_PEER_HANDLE_BYTES]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == Q4T_PEER_HANDLE_BYTES, "handle size");
  if (!ptr || !handle) return fail(Q4T_ERR_INVALID, "null pointer");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (e != cudaSuccess) return fail_cuda("peer buffer export", e);
  std::memcpy(handle, &h, sizeof(h));
  return Q4T_OK;
}
int32_t q4t_peer_buffer_open(const uint8_t handle[Q4T_PEER_HANDLE_BYTES], void** ptr) {
  if (!ptr || !handle) return fail(Q4T_ERR_INVALID, "null pointer");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? Q4T_OK : fail_cuda("peer buffer open", e);
}
int32_t q4t_peer_buffer_close(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  return e == cudaSuccess ? Q4T_OK : fail_cuda("peer buffer close", e);
}

int32_t q4t_ep_publish(const uint16_t* x, const q4t_ep_peer_table* peers, int32_t hs, float input_scale,
                       void* stream) {
  if (!x || !peers) return fail(Q4T_ERR_INVALID, "null pointer");
  const int world = peers->world, rank = peers->rank, tpr = peers->tokens_per_rank;
  if (world <= 0 || world > Q4T_EP_MAX_RANKS || rank < 0 || rank >= world || tpr <= 0)
    return fail(Q4T_ERR_INVALID, "invalid peer table (world in [1,8], rank < world, tokens_per_rank > 0)");
  if (hs <= 0 || hs % 64) return fail(Q4T_ERR_INVALID, "hs must be a multiple of 64");
  if (!(input_scale > 0.0f)) return fail(Q4T_ERR_INVALID, "input scale must be positive");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  q4t::PublishTargets dst{};
  dst.n = world;
  const size_t code_block = static_cast<size_t>(tpr) * (hs / 2), sf_block = static_cast<size_t>(tpr) * (hs / 16);
  for (int i = 0; i < world; ++i) {
    // own copy first: the peers' copies follow in ring order so that the ranks do not all
    // write to the same GPU at the same moment
    const int p = (rank + i) % world;
    if (!peers->xq_packed[p] || !peers->xq_sf[p]) return fail(Q4T_ERR_INVALID, "peer table has a null buffer");
    dst.packed[i] = const_cast<uint8_t*>(peers->xq_packed[p]) + code_block * rank;
    dst.sf[i] = const_cast<uint8_t*>(peers->xq_sf[p]) + sf_block * rank;
  }
  cudaError_t e = q4t::launch_publish_tokens(x, dst, tpr, hs, input_scale, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("publish launch", e);
}

int32_t q4t_ep_publish_selected(const uint16_t* x, const int32_t* expert_ids, const q4t_ep_peer_table* peers,
                                int32_t k, int32_t E, int32_t hs, float input_scale, void* stream) {
  if (!x || !peers || !expert_ids) return fail(Q4T_ERR_INVALID, "null pointer");
  const int world = peers->world, rank = peers->rank, tpr = peers->tokens_per_rank;
  if (world <= 0 || world > Q4T_EP_MAX_RANKS || rank < 0 || rank >= world || tpr <= 0)
    return fail(Q4T_ERR_INVALID, "invalid peer table (world in [1,8], rank < world, tokens_per_rank > 0)");
  if (hs <= 0 || hs % 64) return fail(Q4T_ERR_INVALID, "hs must be a multiple of 64");
  if (k <= 0 || k > 16 || E <= 0) return fail(Q4T_ERR_INVALID, "k out of range");
  if (!(input_scale > 0.0f)) return fail(Q4T_ERR_INVALID, "input scale must be positive");
  const int map = peers->expert_map;
  if (map < 0 || map > 2) return fail(Q4T_ERR_INVALID, "expert_map must be 0, 1 or 2");
  if (map == 2 && (!peers->expert_owner || peers->experts_total != E))
    return fail(Q4T_ERR_INVALID, "expert_map 2 needs an owner table over all experts");
  if (map != 2 && E % world) return fail(Q4T_ERR_INVALID, "E must be a multiple of the number of ranks");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  q4t::PublishTargets dst{};
  dst.n = world;
  const size_t code_block = static_cast<size_t>(tpr) * (hs / 2), sf_block = static_cast<size_t>(tpr) * (hs / 16);
  for (int p = 0; p < world; ++p) {
    if (!peers->xq_packed[p] || !peers->xq_sf[p]) return fail(Q4T_ERR_INVALID, "peer table has a null buffer");
    dst.packed[p] = const_cast<uint8_t*>(peers->xq_packed[p]) + code_block * rank;
    dst.sf[p] = const_cast<uint8_t*>(peers->xq_sf[p]) + sf_block * rank;
  }
  cudaError_t e = q4t::launch_publish_selected(x, expert_ids, dst, tpr, hs, k, E, map, rank, peers->expert_owner,
                                               input_scale, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("publish launch", e);
}

int32_t q4t_ep_route_publish(const uint16_t* x, const q4t_extra_weights* extra, const q4t_ep_peer_table* peers,
                             int32_t k, float input_scale, uint16_t* logits, int32_t* expert_ids, float* router_w,
                             void* finish_workspace, size_t finish_workspace_bytes, void* stream) {
  if (!x || !extra || !peers || !logits || !expert_ids || !router_w) return fail(Q4T_ERR_INVALID, "null pointer");
  const int T = peers->tokens_per_rank;
  if (T <= 0) return fail(Q4T_ERR_INVALID, "invalid peer table (tokens_per_rank > 0)");
  if (k <= 0 || k > 16 || k > extra->E) return fail(Q4T_ERR_INVALID, "k out of range");
  FinishLayout F;
  int rc = finish_args_ok(extra, T, k, finish_workspace, finish_workspace_bytes, &F);
  if (rc != Q4T_OK) return rc;
  const DeviceState* ds;
  if ((rc = device_state(&ds)) != Q4T_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint8_t* base = static_cast<uint8_t*>(finish_workspace);
  cudaError_t e;
  // A token is published only to the ranks that serve one of its experts, so the publish
  // step follows the top-k on the caller's stream (a few megabytes over the links instead of
  // every token to every rank).  Without an owner table (expert_map 2, older callers) every
  // token goes everywhere, from the side stream, beside the router.  The shared expert, which
  // nothing needs before the combine, runs on the side stream in both cases.
  const bool selective = peers->expert_map != 2 || peers->expert_owner != nullptr;
  bool forked = false;
  auto leave = [&](int code) {   // every way out joins the side stream again
    if (forked) {
      const std::string kept = g_error;
      if (cudaEventRecord(ds->join_event, ds->side_stream) == cudaSuccess) cudaStreamWaitEvent(st, ds->join_event, 0);
      g_error = kept;
    }
    return code;
  };
  auto fork = [&]() -> int {
    if ((e = cudaEventRecord(ds->fork_event, st)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(ds->side_stream, ds->fork_event, 0)) != cudaSuccess)
      return fail_cuda("fork", e);
    forked = true;
    q4t::chain_break();
    return Q4T_OK;
  };
  auto shared_on_side = [&]() -> int {
    if ((rc = run_shared_expert(ds, x, extra, reinterpret_cast<uint16_t*>(base + F.shared_gu),
                                reinterpret_cast<uint16_t*>(base + F.shared_act),
                                reinterpret_cast<uint16_t*>(base + F.shared_down), T, 0, ds->side_stream)) != Q4T_OK)
      return rc;
    if ((e = cudaEventRecord(ds->join_event, ds->side_stream)) != cudaSuccess) return fail_cuda("join record", e);
    q4t::chain_break();
    return Q4T_OK;
  };
  if (selective) {
    // router, top-k and the selective publish first, alone on the GPU: the other ranks wait
    // for these tokens.  The shared expert is forked after them, so that it fills the time
    // this rank spends waiting for the exchange of ids instead of competing with the router.
    if ((rc = run_bf16_linear(ds, x, extra->gate, logits, T, extra->E, extra->hs, st)) != Q4T_OK) return rc;
    if ((e = q4t::launch_topk(logits, nullptr, expert_ids, router_w, T, extra->E, k, st)) != cudaSuccess)
      return fail_cuda("topk launch", e);
    if ((rc = q4t_ep_publish_selected(x, expert_ids, peers, k, extra->E, extra->hs, input_scale, st)) != Q4T_OK) return rc;
    if ((rc = fork()) != Q4T_OK) return rc;
    if ((rc = shared_on_side()) != Q4T_OK) return leave(rc);
    return Q4T_OK;   // the side stream is joined by q4t_ep_combine
  }
  if ((rc = fork()) != Q4T_OK) return rc;
  if ((rc = q4t_ep_publish(x, peers, extra->hs, input_scale, ds->side_stream)) != Q4T_OK) return leave(rc);
  if ((e = cudaEventRecord(ds->mid_event, ds->side_stream)) != cudaSuccess) return leave(fail_cuda("publish record", e));
  q4t::chain_break();
  if ((rc = shared_on_side()) != Q4T_OK) return leave(rc);
  if ((rc = run_bf16_linear(ds, x, extra->gate, logits, T, extra->E, extra->hs, st)) != Q4T_OK) return leave(rc);
  if ((e = q4t::launch_topk(logits, nullptr, expert_ids, router_w, T, extra->E, k, st)) != cudaSuccess)
    return leave(fail_cuda("topk launch", e));
  if ((e = cudaStreamWaitEvent(st, ds->mid_event, 0)) != cudaSuccess) return leave(fail_cuda("publish join", e));
  return Q4T_OK;   // the side stream is joined by q4t_ep_combine (the shared expert's result is needed there)
}

int32_t q4t_ep_combine(const uint16_t* x, const uint16_t* landed_rows, const int32_t* expert_ids,
                       const float* router_w, const q4t_extra_weights* extra, uint16_t* y, int32_t T, int32_t k,
                       int32_t* row_of_flat, void* finish_workspace, size_t finish_workspace_bytes, void* stream) {
  if (T <= 0) return Q4T_OK;
  FinishLayout F;
  int rc = finish_args_ok(extra, T, k, finish_workspace, finish_workspace_bytes, &F);
  if (rc != Q4T_OK) return rc;
  if (!x || !landed_rows || !expert_ids || !router_w || !y || !row_of_flat) return fail(Q4T_ERR_INVALID, "null pointer");
  const DeviceState* ds;
  if ((rc = device_state(&ds)) != Q4T_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  // the shared expert started by q4t_ep_route_publish (a no-op wait when there was none)
  if ((e = cudaStreamWaitEvent(st, ds->join_event, 0)) != cudaSuccess) return fail_cuda("join", e);
  q4t::chain_break();
  if ((e = q4t::launch_ep_flat_rows(expert_ids, T * k, extra->E, row_of_flat, st)) != cudaSuccess)
    return fail_cuda("flat rows launch", e);
  uint8_t* base = static_cast<uint8_t*>(finish_workspace);
  e = q4t::launch_final_combine(landed_rows, row_of_flat, router_w, reinterpret_cast<uint16_t*>(base + F.shared_down), x,
                                extra->shared_gate_scalar, reinterpret_cast<float*>(base + F.routed), y, T, k,
                                extra->hs, st);
  return e == cudaSuccess ? Q4T_OK : fail_cuda("combine launch", e);
}

size_t q4t_moe_expert_peer_workspace_bytes(int32_t tokens_all, int32_t k, int32_t hs, int32_t moe_is,
                                           int32_t E_local) {
  if (tokens_all <= 0 || k <= 0 || !routed_dims_ok(E_local, hs, moe_is)) return 0;
  q4t_routed_ws_layout L;
  routed_layout(tokens_all, k, hs, moe_is, E_local, &L);
  return align_up(L.total, 256) + align_up(static_cast<size_t>(tokens_all) * k * 4, 256);
}

int32_t q4t_moe_expert_peer(const int32_t* ids_all, const q4t_ep_peer_table* peers, const q4t_routed_weights* w,
                            int32_t k, void* workspace, size_t workspace_bytes, uint32_t flags, void* stream) {
  if (!peers || !w || !ids_all || !workspace) return fail(Q4T_ERR_INVALID, "null pointer");
  const int world = peers->world, rank = peers->rank, tpr = peers->tokens_per_rank;
  if (world <= 0 || world > Q4T_EP_MAX_RANKS || rank < 0 || rank >= world || tpr <= 0)
    return fail(Q4T_ERR_INVALID, "invalid peer table (world in [1,8], rank < world, tokens_per_rank > 0)");
  if (k <= 0 || k > 16) return fail(Q4T_ERR_INVALID, "k out of range");
  if (!routed_dims_ok(w->E, w->hs, w->moe_is))
    return fail(Q4T_ERR_INVALID, "hs and moe_is must be multiples of 128 and E <= 1024");
  if (!(w->gu_input_scale_uniform > 0.0f))
    return fail(Q4T_ERR_INVALID, "the peer path needs one gate/up input scale for all experts");
  if (static_cast<int64_t>(world) * tpr * k > (1ll << 30)) return fail(Q4T_ERR_INVALID, "too many rows");
  for (int i = 0; i < world; ++i)
    if (!peers->xq_packed[i] || !peers->xq_sf[i] || !peers->dn_rows[i])
      return fail(Q4T_ERR_INVALID, "peer table has a null buffer");
  if (reinterpret_cast<uintptr_t>(workspace) & 255u) return fail(Q4T_ERR_INVALID, "workspace must be 256-byte aligned");
  const int T_all = world * tpr, R = T_all * k;
  if (workspace_bytes < q4t_moe_expert_peer_workspace_bytes(T_all, k, w->hs, w->moe_is, w->E))
    return fail(Q4T_ERR_WORKSPACE, "workspace too small");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RoutedPtrs P;
  routed_layout(T_all, k, w->hs, w->moe_is, w->E, &P.L);
  P.base = static_cast<uint8_t*>(workspace);
  int32_t* local_ids = reinterpret_cast<int32_t*>(P.base + align_up(P.L.total, 256));
  const int map = peers->expert_map;
  if (map < 0 || map > 2) return fail(Q4T_ERR_INVALID, "expert_map must be 0, 1 or 2");
  if (map == 2 && (!peers->placement || peers->experts_total <= 0))
    return fail(Q4T_ERR_INVALID, "expert_map 2 needs a placement table");
  const int E_total = map == 2 ? peers->experts_total : w->E * world;
  cudaError_t e = q4t::launch_ep_localise_ids(ids_all, R, E_total, world, rank, map, peers->placement, tpr * k,
                                              local_ids, st);
  if (e != cudaSuccess) return fail_cuda("id localise launch", e);
  PeerRoute route{};
  route.xq_packed = peers->xq_packed[rank];
  route.xq_sf = peers->xq_sf[rank];
  route.rows_per_rank = tpr * k;
  for (int i = 0; i < q4t::kMaxPeers; ++i) route.dn_rows[i] = peers->dn_rows[i < world ? i : 0];
  stage_begin(st);
  stage_end(1, st);
  return run_routed_core(ds, nullptr, local_ids, w, P, T_all, k, flags, st, false, &route);
}

size_t q4t_ep_sync_buffer_bytes(int32_t world, int32_t tokens_per_rank, int32_t k) {
  if (world <= 0 || world > Q4T_EP_MAX_RANKS || tokens_per_rank <= 0 || k <= 0) return 0;
  return align_up(Q4T_EP_SYNC_IDS_OFFSET + static_cast<size_t>(world) * tokens_per_rank * k * 4, 256);
}

namespace {
int sync_table_ok(const q4t_ep_peer_table* peers) {
  if (!peers) return fail(Q4T_ERR_INVALID, "null pointer");
  if (peers->world <= 0 || peers->world > Q4T_EP_MAX_RANKS || peers->rank < 0 || peers->rank >= peers->world ||
      peers->tokens_per_rank <= 0)
    return fail(Q4T_ERR_INVALID, "invalid peer table (world in [1,8], rank < world, tokens_per_rank > 0)");
  for (int i = 0; i < peers->world; ++i)
    if (!peers->sync[i]) return fail(Q4T_ERR_INVALID, "peer table has no sync buffers");
  return Q4T_OK;
}
int post(const int32_t* ids, const q4t_ep_peer_table* peers, int k, int row, uint32_t epoch, void* stream) {
  int rc = sync_table_ok(peers);
  if (rc != Q4T_OK) return rc;
  const DeviceState* ds;
  if ((rc = device_state(&ds)) != Q4T_OK) return rc;
  q4t::EpPostTargets dst{};
  const size_t block = static_cast<size_t>(peers->tokens_per_rank) * k * 4;
  for (int p = 0; p < peers->world; ++p) {
    dst.ids[p] = reinterpret_cast<int32_t*>(peers->sync[p] + Q4T_EP_SYNC_IDS_OFFSET + block * peers->rank);
    dst.flag[p] = reinterpret_cast<uint32_t*>(peers->sync[p]) + row * Q4T_EP_MAX_RANKS + peers->rank;
  }
  cudaError_t e = q4t::launch_ep_post(ids, ids ? peers->tokens_per_rank * k : 0, dst, peers->world, epoch,
                                      static_cast<cudaStream_t>(stream));
  q4t::chain_break();
  return e == cudaSuccess ? Q4T_OK : fail_cuda("post launch", e);
}
}  // namespace

int32_t q4t_ep_post_ids(const int32_t* expert_ids, const q4t_ep_peer_table* peers, int32_t k, uint32_t epoch,
                        void* stream) {
  if (!expert_ids) return fail(Q4T_ERR_INVALID, "null pointer");
  if (k <= 0 || k > 16) return fail(Q4T_ERR_INVALID, "k out of range");
  return post(expert_ids, peers, k, 0, epoch, stream);
}

int32_t q4t_ep_post_rows(const q4t_ep_peer_table* peers, uint32_t epoch, void* stream) {
  return post(nullptr, peers, 1, 1, epoch, stream);
}

int32_t q4t_ep_wait(const q4t_ep_peer_table* peers, int32_t phase, uint32_t epoch, void* stream) {
  int rc = sync_table_ok(peers);
  if (rc != Q4T_OK) return rc;
  if (phase < 0 || phase > 1) return fail(Q4T_ERR_INVALID, "phase must be 0 or 1");
  const DeviceState* ds;
  if ((rc = device_state(&ds)) != Q4T_OK) return rc;
  uint8_t* own = peers->sync[peers->rank];
  cudaError_t e = q4t::launch_ep_wait(reinterpret_cast<const uint32_t*>(own) + phase * Q4T_EP_MAX_RANKS, peers->world,
                                      epoch, reinterpret_cast<int32_t*>(own + 128), static_cast<cudaStream_t>(stream));
  q4t::chain_break();   // what follows reads other ranks' writes: an ordinary launch
  return e == cudaSuccess ? Q4T_OK : fail_cuda("wait launch", e);
}

int32_t q4t_ep_sync_status(const q4t_ep_peer_table* peers) {
  int rc = sync_table_ok(peers);
  if (rc != Q4T_OK) return rc;
  int32_t word = 0;
  cudaError_t e = cudaMemcpy(&word, peers->sync[peers->rank] + 128, 4, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail_cuda("status read", e);
  if (word != 0) return fail(Q4T_ERR_KERNEL, "a wait for another rank ran out (code " + std::to_string(word) + ")");
  return Q4T_OK;
}

int32_t q4t_ep_flat_rows(const int32_t* expert_ids, int32_t rows, int32_t E, int32_t* row_of_flat, void* stream) {
  if (rows <= 0) return Q4T_OK;
  if (!expert_ids || !row_of_flat || E <= 0) return fail(Q4T_ERR_INVALID, "invalid arguments");
  cudaError_t e = q4t::launch_ep_flat_rows(expert_ids, rows, E, row_of_flat, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("flat rows launch", e);
}

int32_t q4t_residual_rmsnorm_bf16(uint16_t* x, const uint16_t* y, uint16_t* h, int32_t T, int32_t hs, float eps,
                                  void* stream) {
  if (T <= 0) return Q4T_OK;
  if (!x || !h) return fail(Q4T_ERR_INVALID, "null pointer");
  if (hs <= 0 || hs % 8) return fail(Q4T_ERR_INVALID, "hs must be a multiple of 8");
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(h)) & 15u)
    return fail(Q4T_ERR_INVALID, "rows must be 16-byte aligned");
  const DeviceState* ds;
  int rc = device_state(&ds);
  if (rc != Q4T_OK) return rc;
  cudaError_t e = q4t::launch_residual_rmsnorm(x, y, h, T, hs, eps, static_cast<cudaStream_t>(stream));
  return e == cudaSuccess ? Q4T_OK : fail_cuda("rmsnorm launch", e);
}

int32_t q4t_moe_workspace_status(const void* workspace, int32_t M, int32_t k, int32_t hs, int32_t moe_is,
                                 int32_t E) {
  if (!workspace || M <= 0 || k <= 0) return fail(Q4T_ERR_INVALID, "invalid arguments");
  q4t_routed_ws_layout L;
  routed_layout(M, k, hs, moe_is, E, &L);
  int32_t word = 0;
  cudaError_t e = cudaMemcpy(&word, static_cast<const uint8_t*>(workspace) + L.status, 4, cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return fail_cuda("status read", e);
  if (word != 0) return fail(Q4T_ERR_KERNEL, "a bounded device-side wait ran out (role " + std::to_string(word) + ")");
  if (q4t::small_m_gemm_timed_out()) return fail(Q4T_ERR_KERNEL, "a bounded device-side wait ran out (bf16 linear)");
  return Q4T_OK;
}

int32_t q4t_stage_timing_enable(int32_t enable) {
  StageTimer& t = g_timer;
  if (enable && !t.enabled) {
    for (auto& ev : t.ev)
      if (cudaEventCreate(&ev) != cudaSuccess) return fail(Q4T_ERR_CUDA, "cudaEventCreate failed");
    t.enabled = true;
  } else if (!enable && t.enabled) {
    for (auto& ev : t.ev) cudaEventDestroy(ev);
    t.enabled = false;
  }
  return Q4T_OK;
}

int32_t q4t_stage_timing_read(float* ms_out) {
  StageTimer& t = g_timer;
  if (!ms_out) return fail(Q4T_ERR_INVALID, "null pointer");
  if (!t.enabled || !t.marked[0]) return fail(Q4T_ERR_INVALID, "stage timing is not enabled or nothing was recorded");
  int last = 0;
  for (int i = 0; i <= Q4T_NUM_STAGES; ++i)
    if (t.marked[i]) last = i;
  cudaError_t e = cudaEventSynchronize(t.ev[last]);
  if (e != cudaSuccess) return fail_cuda("cudaEventSynchronize", e);
  int prev = 0;
  for (int i = 0; i < Q4T_NUM_STAGES; ++i) {
    ms_out[i] = 0.0f;
    if (!t.marked[i + 1]) continue;
    if ((e = cudaEventElapsedTime(&ms_out[i], t.ev[prev], t.ev[i + 1])) != cudaSuccess)
      return fail_cuda("cudaEventElapsedTime", e);
    prev = i + 1;
  }
  return Q4T_OK;
}

}  // extern "C"
