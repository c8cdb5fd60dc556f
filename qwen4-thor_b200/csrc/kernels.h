// Internal launch interface between the C ABI (api.cu) and the kernel files.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace q4t {

constexpr int kTileM = 128;        // rows of one GEMM tile (tokens of one expert)
// Launches `kernel` with programmatic stream serialisation: it may become resident once
// the previous kernel's blocks have exited, and calls chain_wait() before touching global
// memory.  Worth about 6 % of a decode step (launch and prologue of each kernel overlap
// with the tail of the one before).  Measured: a kernel launched this way directly after a
// cudaStreamWaitEvent did not wait for the other stream's work, hence chain_break().
// chaining_enabled() is false when the environment variable Q4T_NO_CHAIN is set (ordinary
// launches, for comparison runs).
bool chaining_enabled();
// The next launch_chained() of this thread is an ordinary launch.  Called at the start of
// every public entry point and after every cross-stream event wait: a kernel that follows
// anything but a kernel of this library in its stream (a copy, an event wait, a caller's
// kernel) must keep the full stream ordering.
void chain_break();
bool chain_break_pending();  // reads and clears the mark
template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  const bool plain = chain_break_pending();
  cfg.numAttrs = (chaining_enabled() && !plain) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose blocks form clusters of `cluster_x` along x.
template <typename... KArgs, typename... Args>
cudaError_t launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                   unsigned cluster_x, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_x;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  const bool plain = chain_break_pending();
  cfg.numAttrs = (chaining_enabled() && !plain) ? 2 : 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

constexpr int kPlanChunk = 2048;   // (token,slot) entries handled by one planning block

// ---- quantise / dequantise (quant_kernels.cu)
cudaError_t launch_quantize(const uint16_t* x, uint8_t* packed, uint8_t* sf, int M, int K,
                            float global_scale, cudaStream_t stream);
cudaError_t launch_gather_quantize(const uint16_t* x, uint8_t* packed, uint8_t* sf_tiles, int R,
                                   int K, const int32_t* flat_of_row, const int32_t* expert_ids,
                                   const float* input_scale, const int32_t* row_tile,
                                   const int32_t* tile_row0, const int32_t* rows_dev, int k, int E,
                                   cudaStream_t stream);
// One input scale for all experts: quantise each of the T tokens once and write codes and
// scales to its k grouped rows (row_of_flat[t*k+s], -1 = skipped); K % 64 == 0, K >= 128, k <= 16.
cudaError_t launch_quantize_scatter(const uint16_t* x, uint8_t* packed, uint8_t* sf_tiles, int T, int K,
                                    float global_scale, const int32_t* row_of_flat, const int32_t* row_tile,
                                    const int32_t* tile_row0, int k, cudaStream_t stream);
// Expert parallelism over peer memory: a rank quantises its tokens once and writes the
// codes and the scale bytes (row-major [tokens, K/16], not swizzled) into its block of
// every rank's gathered buffer (the targets may be peer GPUs' memory; K a multiple of 64).
constexpr int kMaxPeers = 8;
struct PublishTargets {
  uint8_t* packed[kMaxPeers];  // start of this rank's block in each gathered code buffer
  uint8_t* sf[kMaxPeers];      // start of this rank's block in each gathered scale buffer
  int n;
};
cudaError_t launch_publish_tokens(const uint16_t* x, const PublishTargets& dst, int M, int K, float global_scale,
                                  cudaStream_t stream);
// The selective form: packed[r] / sf[r] are rank r's buffers (rank order); a token is stored
// only on the ranks that own one of its k selected experts, and on `self`.
cudaError_t launch_publish_selected(const uint16_t* x, const int32_t* ids, const PublishTargets& dst, int M, int K,
                                    int k, int E, int map, int self, const int32_t* owner, float global_scale,
                                    cudaStream_t stream);
// Copies each grouped row's codes and scales out of the gathered buffers of all ranks' tokens:
// xq_packed [tokens, K/2], xq_sf [tokens, K/16] row-major.
cudaError_t launch_gather_codes_rowsf(const uint8_t* xq_packed, const uint8_t* xq_sf, uint8_t* packed,
                                      uint8_t* sf_tiles, int R, int K, const int32_t* flat_of_row,
                                      const int32_t* row_tile, const int32_t* tile_row0, const int32_t* rows_dev,
                                      int k, cudaStream_t stream);
// Collective-free exchange of ids and "done" marks between expert-parallel ranks: ids[p] /
// flag[p] are rank p's gathered-id block for this rank and this rank's slot in rank p's flag row.
struct EpPostTargets {
  int32_t* ids[kMaxPeers];
  uint32_t* flag[kMaxPeers];
};
// ids may be null (flag only).  Plain launches: they follow and precede other ranks' work.
cudaError_t launch_ep_post(const int32_t* ids, int n_ids, const EpPostTargets& dst, int world, uint32_t epoch,
                           cudaStream_t stream);
cudaError_t launch_ep_wait(const uint32_t* flags, int world, uint32_t epoch, int32_t* status, cudaStream_t stream);
cudaError_t launch_dequant(const uint8_t* packed, const uint8_t* group_scale, uint16_t* out,
                           float inv_global, int N, int K, cudaStream_t stream);
// ---- routing, permutation, combine (routing_kernels.cu)
// Tables produced by the planning step, all in the routed workspace.
struct PlanTables {
  int32_t* blk_counts;   // [nblk, E] scratch
  int32_t* counts;       // [E]
  int32_t* offsets;      // [E+1]
  int32_t* tile_off;     // [E+1]
  int32_t* tile_expert;  // [max_tiles]
  int32_t* tile_row0;    // [max_tiles]
  int32_t* tile_nrows;   // [max_tiles]
  int32_t* ntiles;       // [1]
  int32_t* row_of_flat;  // [R]
  int32_t* flat_of_row;  // [R]
  int32_t* row_tile;     // [R]
  int32_t* status;       // [4] kernel status words, cleared by the planner (may be null)
};
cudaError_t routing_set_attributes();
cudaError_t launch_small_m_linear(const uint16_t* x, const uint16_t* w, uint16_t* y, int M, int N,
                                  int K, cudaStream_t stream);
cudaError_t launch_topk(const uint16_t* logits, const int32_t* fixed_ids, int32_t* ids, float* rw,
                        int T, int E, int k, cudaStream_t stream);
// Small batches: top-k and the permutation tables in one single-block launch.
bool route_and_plan_fits(int T, int k);
cudaError_t launch_route_and_plan(const uint16_t* logits, const int32_t* fixed_ids, int32_t* ids, float* rw, int T,
                                  int E, int k, int max_tiles, const PlanTables& p, cudaStream_t stream);
// 17..256 tokens: the same in one launch of an eight-CTA cluster (counts exchanged through
// distributed shared memory).
bool route_plan_cluster_fits(int T, int k, int E);
cudaError_t launch_route_plan_cluster(const uint16_t* logits, const int32_t* fixed_ids, int32_t* ids, float* rw,
                                      int T, int E, int k, int max_tiles, const PlanTables& p, cudaStream_t stream);
// even_tiles: every expert with rows gets an even number of row tiles (the last one may be
// empty), as the CTA-pair GEMMs need.
cudaError_t launch_plan(const int32_t* ids, int R, int E, int max_tiles, const PlanTables& p,
                        cudaStream_t stream, bool even_tiles = false);
cudaError_t launch_ep_split_ids(const int32_t* ids, int R, int E, int experts_per_rank, int32_t* dest,
                                int32_t* local, cudaStream_t stream);
// local[f] = index of expert ids[f] on `rank` (-1 when it is served elsewhere or out of range).
// map 0: expert e lives on rank e / (E/world) as local e % (E/world); 1: on rank e % world as
// local e / world; 2: placement[e] = -1, the local index, or (1<<30 | local index) for an expert
// replicated on all ranks, which serves only the entries of this rank's own tokens
// (f / flats_per_rank == rank).
cudaError_t launch_ep_localise_ids(const int32_t* ids, int R, int E, int world, int rank, int map,
                                   const int32_t* placement, int flats_per_rank, int32_t* local,
                                   cudaStream_t stream);
// out[f] = slot_of_expert[ids[f]] (an id outside [0,E) or a slot outside [0,slots) gives -1).
cudaError_t launch_remap_ids(const int32_t* ids, const int32_t* slot_of_expert, int32_t* out, int R, int E, int slots,
                             cudaStream_t stream);
// row_of_flat[f] = f for ids[f] in [0,E), else -1 (rows delivered in flat order).
cudaError_t launch_ep_flat_rows(const int32_t* ids, int R, int E, int32_t* row_of_flat, cudaStream_t stream);
cudaError_t launch_gather_rows(const uint16_t* src, const int32_t* index, int div, const int32_t* rows_dev,
                               int rows, int width, uint16_t* out, const int32_t* aux, int32_t* aux_out,
                               cudaStream_t stream);
cudaError_t launch_routed_combine(const uint16_t* dn_out, const int32_t* row_of_flat,
                                  const float* rw, float* y, int T, int k, int hs,
                                  cudaStream_t stream);
cudaError_t launch_swiglu(const uint16_t* gu, uint16_t* out, int T, int inner, cudaStream_t stream);
// x <- bf16(x + y) (y may be null), h <- RMSNorm(x) without a weight; hs % 8 == 0.
cudaError_t launch_residual_rmsnorm(uint16_t* x, const uint16_t* y, uint16_t* h, int T, int hs, float eps,
                                    cudaStream_t stream);
// Optional gated residual write fused into the final combine: out[t, b, :] =
// bf16(residual[t, b, :] + y[t, :] * inject_gate[t, b]) for b < hc (hc = 0: nothing).
struct HcWrite {
  const uint16_t* residual;     // [T, hc, hs] bf16
  const uint16_t* inject_gate;  // [T, hc] bf16
  uint16_t* out;                // [T, hc, hs] bf16
  int hc;
};
// The step between two layers of a decode stack fused into the combine: residual <- bf16(residual + y),
// out <- RMSNorm(residual) without a weight, bit for bit what launch_residual_rmsnorm computes.
constexpr int kNormWriteMaxHs = 8192;
struct NormWrite {
  uint16_t* residual;   // [T, hs] bf16, read and written (null = off)
  uint16_t* out;        // [T, hs] bf16
  float eps;
};
cudaError_t launch_final_combine(const uint16_t* dn_out, const int32_t* row_of_flat, const float* rw,
                                 const uint16_t* shared_down, const uint16_t* x,
                                 const uint16_t* gate_scalar, float* routed, uint16_t* y, int T,
                                 int k, int hs, cudaStream_t stream, const HcWrite& hcw = HcWrite{},
                                 const NormWrite& nw = NormWrite{});

// ---- routed experts for decode-sized batches (decode_small.cu)
constexpr int kSmallN = 16;            // token rows per pass of one CTA (the N side of the MMA)
constexpr int kSmallMaxTokens = 128;   // largest batch that may take this path
constexpr int kSmallMaxEntries = 2048; // (token,slot) entries: 128 tokens x top-16
constexpr int kSmallMaxExperts = 2048; // expert ids the per-expert tables (8 bytes each, inside one ring stage) can index
struct SmallBatchArgs {
  const int32_t* ids;        // [R] expert (or slot) of each (token,slot) entry; outside [0,E) = skipped
  int R, k, E;
  int K;                     // reduction length: hs (gate/up) or moe_is (down)
  int n_tiles;               // 128-row weight tiles per expert
  int w_rows_per_expert;     // 2*moe_is (gate/up) or hs (down)
  const uint8_t* w_sf;       // the experts' swizzled scale buffers
  size_t w_sf_stride;        // bytes between two experts' buffers
  const float* alpha_w;      // per-expert weight scale
  const float* alpha_a;      // per-expert activation scale
  const float* in_scale;     // per-expert global scale the token-side operand is quantised with
  const uint16_t* src;       // gate/up: x [T, hs]; down: the bf16 gate|up rows [R, 2*moe_is]
  int src_ld;
  uint16_t* out;             // [R, ldo] bf16, rows in (token,slot) order
  int ldo;
  int32_t* row_of_flat;      // gate/up only: written as the identity (-1 for skipped entries)
  int32_t* status;
  int stages;                // TMA ring depth (small_batch_stages)
  uint32_t tmem_cols;        // tensor-memory columns: 32 (accumulator) + 32 per stage, rounded up to a power of two
  int release_next;          // gate/up only: let the down kernel become resident while this one runs
};
// Ring depth for reduction length K, `tiles` weight tiles and `entries` (token,slot) entries,
// 0 when the token-side operand does not fit shared memory.
int small_batch_stages(int K, int tiles, int entries);
cudaError_t small_batch_set_attributes();
// mode 0 = gate/up, 1 = down.
cudaError_t launch_small_batch(int mode, const CUtensorMap& tmap_w, const SmallBatchArgs& a, int num_sms,
                               cudaStream_t stream);

// ---- bf16 linear for one tile of token rows (bf16_small_m.cu): M <= 128, N a multiple of 64, K a
// multiple of 64.  tmap_x / tmap_w are 3-D maps (64 elements x rows x K/64) with boxes of
// 64 x bf16_small_m_box_rows(M) x 4 and 64 x 64 x 4.
// beside_others: the launch runs next to another stream's kernels (the shared expert beside the routed
// experts): a shallow ring, so that it leaves them the SM's shared memory.
cudaError_t bf16_small_m_set_attributes();
bool bf16_small_m_fits(int M, int N, int K);
int bf16_small_m_box_rows(int M);
cudaError_t launch_bf16_small_m(const CUtensorMap& tmap_x, const CUtensorMap& tmap_w, uint16_t* y, int M, int N, int K,
                                int num_sms, bool beside_others, cudaStream_t stream);
// The shared expert's gate/up projection with SwiGLU: w has 2*N rows (gate rows, then up rows), tmap_w
// is the 4-D map 64 elements x N rows x 2 halves x K/64 with a box of 64 x 32 x 2 x 4; act [M, N];
// gu_dump (optional) receives the bf16 projections [M, 2*N].
bool bf16_small_m_swiglu_fits(int M, int N, int K);
cudaError_t launch_bf16_small_m_swiglu(const CUtensorMap& tmap_x, const CUtensorMap& tmap_w, uint16_t* act, int M, int N,
                                       int K, uint16_t* gu_dump, int num_sms, cudaStream_t stream);
// Grouped form: blockIdx.y runs over the row tiles of the permutation tables (the rows of one expert,
// consecutive in x; at most max_row_tiles of them), the weights are [groups * w_rows_per_group, K];
// x's box has box_rows rows (a tile with more rows takes several passes over its weights).
cudaError_t launch_bf16_small_m_grouped(const CUtensorMap& tmap_x, const CUtensorMap& tmap_w, uint16_t* y, bool swiglu,
                                        int box_rows, int max_row_tiles, int N, int K, const int32_t* tile_expert,
                                        const int32_t* tile_row0, const int32_t* tile_nrows, const int32_t* ntiles,
                                        int w_rows_per_group, int num_sms, cudaStream_t stream);
bool small_m_gemm_timed_out();   // reads and clears the kernel's time-out flag

// ---- tensor-core GEMMs (tc_gemm.cu)
enum class Epilogue : int {
  kStoreBf16 = 0,     // out[row, n] = bf16(alpha * acc)
  kStoreF32 = 1,      // out[row, n] = alpha * acc
  kSwigluBf16 = 2,    // gate|up tile -> bf16((g*sig(g))*u), g/u rounded to bf16 first
  kSwigluQuant = 3,   // as above, then NVFP4 quantisation with the expert's down input scale
  kStoreBf16Rows = 4  // kStoreBf16 written as whole 128-byte row segments, rows optionally scattered
                      // (NVFP4 only; the form used when rows may go to peer GPUs)
};
struct GemmArgs {
  // problem
  int K;                 // reduction length (elements)
  int n_tiles;           // column tiles per row tile
  int n_per_tile;        // output columns produced per tile (tile_cols, or half of it for the SwiGLU epilogues)
  int tile_cols;         // accumulator columns per tile: 256 (0 means 256), or 64 for BF16 narrow tiles
  int up_row_offset;     // SwiGLU: row distance between a gate row and its up row in B
  int b_rows_per_group;  // rows of B belonging to one expert (0 for a dense GEMM)
  int b_rows_valid;      // output columns that exist (N); columns beyond are neither loaded as scales nor stored
  // row tiles: dense (tile t = rows [128 t, ..)) when tile_expert == nullptr
  const int32_t* ntiles_dev;   // device count of row tiles (grouped) or nullptr
  int ntiles_host;             // row tiles (dense)
  const int32_t* tile_expert;
  const int32_t* tile_row0;
  const int32_t* tile_nrows;
  int total_rows;              // dense: M
  // block scales (NVFP4 only)
  const uint8_t* sfa_tiles;    // tile-local atoms: tile t at t * ceil(K/64) * 512
  const uint8_t* sfb;          // standard swizzled buffer per group
  size_t sfb_group_stride;     // bytes between groups' scale buffers
  int sfb_group_atoms;         // the same in 512-byte atoms (pair kernels address atoms through a tensor map)
  // epilogue
  void* out;                   // bf16 / f32 / packed codes
  int ldo;                     // leading dimension of out, in elements (bytes for codes)
  const float* alpha_w;        // per-group weight scale (grouped) or nullptr
  const float* alpha_a;        // per-group activation scale or nullptr
  float alpha_const;           // used when alpha_w == nullptr
  const float* next_scale;     // kSwigluQuant: per-group input scale of the next GEMM
  uint8_t* out_sf_tiles;       // kSwigluQuant: tile-local scale atoms of the intermediate
  uint16_t* gu_dump;           // optional bf16 [rows, 2*inner] copy of the rounded gate|up values
  int gu_dump_ld;
  // kStoreBf16Rows only: when scatter_flat is set, row r of the output goes to
  // scatter_base[f / scatter_rows_per_rank] + (f % scatter_rows_per_rank) * ldo with
  // f = scatter_flat[r] (the bases may be peer GPUs' memory) instead of out + r * ldo.
  const int32_t* scatter_flat;
  int scatter_rows_per_rank;
  uint16_t* scatter_base[kMaxPeers];
  int32_t* status;             // device status word (non-zero = a bounded wait ran out)
  long long* trace;            // timestamps of CTA 0 (only read by builds with Q4T_TRACE; null otherwise)
};
// tmap_a: [rows, K] operand A; tmap_b: [all groups' rows, K] operand B (K-major, 128-byte boxes).
cudaError_t launch_gemm_nvf4(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const GemmArgs& a,
                             Epilogue epi, int num_sms, cudaStream_t stream);
cudaError_t launch_gemm_bf16(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const GemmArgs& a,
                             Epilogue epi, int num_sms, cudaStream_t stream);
// CTA-pair forms (tc_gemm_pair.cu: tcgen05 cta_group::2; clusters of two CTAs share each weight tile).  Row
// tiles 2j and 2j+1 of a grouped tile list must belong to the same expert.  tmap_sfa /
// tmap_sfb: [atoms, 512 bytes] views of the scale buffers (make them with 128 x uint32
// rows and a box of four atoms).
cudaError_t launch_gemm_nvf4_pair(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const CUtensorMap& tmap_sfa,
                                  const CUtensorMap& tmap_sfb, const GemmArgs& a, Epilogue epi, int num_sms,
                                  cudaStream_t stream);
cudaError_t launch_gemm_bf16_pair(const CUtensorMap& tmap_a, const CUtensorMap& tmap_b, const GemmArgs& a,
                                  Epilogue epi, int num_sms, cudaStream_t stream);
cudaError_t gemm_set_attributes();
cudaError_t gemm_pair_set_attributes();   // tc_gemm_pair.cu

}  // namespace q4t
