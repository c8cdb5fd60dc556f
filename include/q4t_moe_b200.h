/*
 * C ABI of libq4t_moe_b200.so: a B200 (sm_100a) implementation of the
 * qwen4-thor NVFP4 W4A4 MoE layer operators.
 *
 * Every entry point takes plain device/host pointers and sizes, enqueues its
 * work on the caller's CUDA stream (passed as void*, i.e. a cudaStream_t; NULL
 * is the default stream), performs no host synchronisation and returns 0 on
 * success or a negative q4t_status.  q4t_last_error() returns the message of
 * the calling thread's last failure.  There is no CPU fallback: on a machine
 * without a usable sm_100 device the compute entry points fail.
 *
 * Each declaration names the reference interface (file:line in the
 * qwen4-thor tree) whose behaviour it reproduces.  The C++ shims in
 * qwen4-thor_b200/host/ rebuild those C++ signatures on top of this ABI.
 *
 * Data formats (unchanged from the reference engine):
 *   packed NVFP4  : row-major [rows, K/2] bytes, two e2m1 codes per byte, low
 *                   nibble = even element;
 *   block scales  : one unsigned e4m3 byte per 16 elements along K, stored in
 *                   128-row x 4-group atoms of 512 bytes (byte (r%32)*16 +
 *                   ((r%128)/32)*4 + g%4 of atom (r/128)*ceil(K/64) + g/4);
 *   global scales : one fp32 per tensor (weight_scale_2, input_scale);
 *   bf16          : uint16_t bit patterns.
 */
#ifndef Q4T_MOE_B200_H_
#define Q4T_MOE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  Q4T_OK = 0,
  Q4T_ERR_INVALID = -1,    /* bad dimensions or null pointers            */
  Q4T_ERR_WORKSPACE = -2,  /* workspace too small                        */
  Q4T_ERR_CUDA = -3,       /* a CUDA call failed                         */
  Q4T_ERR_DEVICE = -4,     /* no sm_100 device / driver entry point      */
  Q4T_ERR_KERNEL = -5      /* a kernel reported a bounded wait that ran out */
} q4t_status;

/* Message of the calling thread's last failing call ("" if none). */
const char* q4t_last_error(void);
/* Library version string. */
const char* q4t_version(void);

/* One layer's routed-expert weights on the device: the POD image of
 * q4t::quant::MoEWeightLayout (include/q4t/quant/moe_weights.h:43-109).
 * Expert e's gate/up codes start at gu_packed + e*moe_is*hs (gate rows, then
 * up rows), its gate/up scale block at gu_sf + e*q4t_sf_buffer_size(2*moe_is,
 * hs); likewise dn_packed + e*hs*moe_is/2 and dn_sf.                         */
typedef struct {
  int32_t E, hs, moe_is;
  int32_t slot_mode;             /* carried for the host shim; not interpreted */
  const uint8_t* gu_packed;
  const uint8_t* gu_sf;
  const uint8_t* dn_packed;
  const uint8_t* dn_sf;
  const float* gu_w_scale2;      /* [E] device */
  const float* gu_input_scale;   /* [E] device */
  const float* dn_w_scale2;      /* [E] device */
  const float* dn_input_scale;   /* [E] device */
  /* > 0: every expert's gate/up input scale equals this value (the caller
   * checked its host copies).  Lets large batches quantise each token once and
   * copy the codes to its top-k rows instead of quantising every (token,slot)
   * row; the bytes produced are the same.  0: no such promise.               */
  float gu_input_scale_uniform;
  int32_t reserved;
} q4t_routed_weights;

/* Router and shared-expert BF16 weights on the device: the POD image of
 * q4t::model::MoEExtraWeights (include/q4t/model/moe.h:39-56), without the
 * optional FP8 shadows.                                                       */
typedef struct {
  int32_t E, hs, shared_is;
  const uint16_t* gate;               /* [E, hs]            */
  const uint16_t* shared_gu;          /* [2*shared_is, hs]  */
  const uint16_t* shared_down;        /* [hs, shared_is]    */
  const uint16_t* shared_gate_scalar; /* [hs]               */
} q4t_extra_weights;

/* ---- CTA-pair GEMMs (no reference counterpart).  GEMMs with at least `rows` A
 * rows (grouped: rows of the whole batch) run as pairs of CTAs on neighbouring
 * SMs sharing each weight tile (tcgen05 cta_group::2).  rows <= 0 (the default)
 * never uses them: on B200 the pair form measured slower than one CTA per tile.
 * The routed workspace of such batches holds more row tiles (every expert is
 * padded to an even tile count), so call this BEFORE sizing workspaces.  The
 * environment variable Q4T_PAIR_MIN_ROWS gives the initial value.              */
int32_t q4t_set_pair_min_rows(int64_t rows);

/* ---- layout helpers: SfNumGtiles / SfBufferSize / SfOffset
 *      (include/q4t/quant/swizzle.h:34-57)                                   */
int32_t q4t_sf_num_gtiles(int32_t K);
size_t q4t_sf_buffer_size(int32_t rows, int32_t K);
size_t q4t_sf_offset(int32_t row, int32_t group, int32_t num_g_tiles);

/* ---- host-side packer: the per-expert body of LoadMoEWeights
 * (src/quant/moe_weights.cpp:163-291).  Copies one expert's checkpoint tensors
 * (gate/up/down codes unchanged; gate then up scale rows concatenated and
 * swizzled; down scales swizzled) into HOST staging images of the device
 * layout.  gate_w/up_w: [moe_is, hs/2]; down_w: [hs, moe_is/2]; *_s row-major
 * e4m3 [rows, K/16].  The four destination pointers address expert e's slice.
 * Enforces the loader's divisibility rules (moe_weights.cpp:49-57).           */
int32_t q4t_pack_expert_host(const uint8_t* gate_w, const uint8_t* up_w,
                             const uint8_t* down_w, const uint8_t* gate_s,
                             const uint8_t* up_s, const uint8_t* down_s,
                             int32_t hs, int32_t moe_is, uint8_t* gu_packed_e,
                             uint8_t* gu_sf_e, uint8_t* dn_packed_e,
                             uint8_t* dn_sf_e);

/* ---- QuantizeActivationToFp4Async (include/q4t/quant/act_quant.h:30-34,
 * src/quant/act_quant.cu:47-108).  bf16 [M,K] -> codes [M,K/2] + swizzled
 * scales (>= q4t_sf_buffer_size(M,K) bytes; only bytes of real rows/groups
 * are written).  K % 16 == 0.                                                */
int32_t q4t_quantize_activation_fp4(const uint16_t* bf16, uint8_t* packed_out,
                                    uint8_t* sf_out, int32_t M, int32_t K,
                                    float global_scale, void* stream);

/* ---- DequantFp4ToBf16Async (include/q4t/quant/dequant.h:22-25,
 * src/quant/dequant.cu:31-71).  Row-major (not swizzled) scales.             */
int32_t q4t_dequant_fp4_to_bf16(const uint8_t* packed, const uint8_t* group_scale,
                                uint16_t* bf16_out, float inv_global_scale,
                                int32_t N, int32_t K, void* stream);

/* ---- Fp4Gemm<OutT> (include/q4t/quant/fp4_gemm.h:58-213): out[M,N] =
 * (inv_w_global*inv_a_global) * A[M,K] . W[N,K]^T with swizzled block scales
 * on both operands.  out_is_bf16 selects uint16_t (bf16) or float output.
 * N % 128 == 0, K % 64 == 0.  The reference's cuBLASLt workspace arguments are
 * accepted by the C++ shim and ignored.                                       */
int32_t q4t_fp4_gemm(const uint8_t* w_packed, const uint8_t* w_sf,
                     const uint8_t* a_packed, const uint8_t* a_sf, void* out,
                     int32_t out_is_bf16, int32_t M, int32_t N, int32_t K,
                     float inv_w_global, float inv_a_global, void* stream);

/* ---- RouterTopkKernel (src/model/moe.cu:134-212): logits bf16 [T,E] ->
 * ids int32 [T,k], weights fp32 [T,k]; selection by (value desc, id asc),
 * softmax over the selected k in selection order.  E <= 512, k <= 16.        */
int32_t q4t_router_topk(const uint16_t* logits, int32_t* expert_ids,
                        float* router_w, int32_t T, int32_t E, int32_t k,
                        void* stream);

/* ---- Bf16Gemm (include/q4t/model/linear.h:103-180): y[M,N] = bf16(x[M,K] .
 * w[N,K]^T).  For M <= 8 the accumulation order is the reference's warp-per-
 * output GEMV order (src/model/gemv.cu:56-119), bit for bit; larger M runs on
 * the tensor cores (order unspecified, as with the reference's library call).
 * N % 128 == 0 and K % 64 == 0 for M > 8; K % 8 == 0 otherwise.               */
int32_t q4t_bf16_linear(const uint16_t* x, const uint16_t* w, uint16_t* y,
                        int32_t M, int32_t N, int32_t K, void* stream);

/* ---- MoEWorkspace::RequiredBytes (include/q4t/quant/moe_gemm.h:34-53).
 * The first four regions keep the reference's order and sizes (a_packed,
 * a_sf, gu_out, dn_out); this implementation's routing tables and tile-local
 * scale blocks follow them, so the total is larger than the reference's.      */
size_t q4t_moe_routed_workspace_bytes(int32_t M, int32_t k, int32_t hs,
                                      int32_t moe_is, int32_t E);
/* Byte offsets of the regions inside a routed workspace.  Rows of the
 * expert-grouped buffers are cut into row tiles of at most 128 rows that
 * never span two experts; scale bytes of grouped rows live in tile-local
 * atoms: tile t, scale tile g/4 at (t*ceil(K/64) + g/4)*512, row index inside
 * the atom = row - tile_row0[t].                                              */
typedef struct {
  size_t a_packed, a_sf, gu_out, dn_out;   /* reference regions (a_sf unused)  */
  size_t counts;                           /* int32 [E]   rows per expert      */
  size_t offsets;                          /* int32 [E+1] first grouped row    */
  size_t row_of_flat;                      /* int32 [M*k] grouped row of (token,slot), -1 if skipped */
  size_t flat_of_row;                      /* int32 [M*k] inverse map          */
  size_t row_tile;                         /* int32 [M*k] row tile of a grouped row */
  size_t ntiles;                           /* int32 [1]   number of row tiles  */
  size_t tile_expert, tile_row0, tile_nrows; /* int32 [max_tiles]              */
  size_t a_sf_tiles;                       /* input scales, tile-local atoms   */
  size_t xq_packed, xq_sf;                 /* per-token codes / scales (uniform input scale path) */
  size_t inter_packed;                     /* [M*k, moe_is/2] intermediate codes */
  size_t inter_sf_tiles;                   /* intermediate scales, tile-local  */
  size_t status;                           /* int32 [4] kernel status words    */
  size_t max_tiles;                        /* capacity of the tile tables      */
  size_t total;
} q4t_routed_ws_layout;
int32_t q4t_moe_routed_workspace_layout(int32_t M, int32_t k, int32_t hs,
                                        int32_t moe_is, int32_t E,
                                        q4t_routed_ws_layout* out);

/* ---- MoERoutedForward (include/q4t/quant/moe_gemm.h:55-74,
 * src/quant/moe_gemm.cu:314-621).  y fp32 [M,hs] must be zeroed by the caller
 * and is accumulated into.  After the call the workspace's dn_out region
 * holds the bf16 down-projection rows in grouped order (expert ascending,
 * then (token,slot) ascending) and row_of_flat maps (token,slot) to its row.
 * Expert ids outside [0,E) are skipped.  flags: bit 0 = also materialise the
 * bf16 gate/up outputs in gu_out (parity/debug; slower).
 * Decode-sized batches (M <= 64 by default, M*k <= 2048, E <= 2048) take a
 * path of their own, the counterpart of MoEDeviceDecode / MoEDeviceDecodeMulti
 * (include/q4t/quant/moe_decode.h:8-36): no permutation, rows kept in
 * (token,slot) order (row_of_flat is the identity, -1 for skipped entries;
 * gu_out always holds the bf16 gate|up rows; the grouped tables, a_packed and
 * the intermediate codes are not produced).  Same arithmetic, same bits in
 * dn_out rows and y.  flags bit 2 = take the general grouped path anyway;
 * flags bit 3 = take the decode-sized path up to its limit of 128 tokens
 * (beyond 64 tokens the grouped path is as fast or faster).                   */
int32_t q4t_moe_routed_forward(const uint16_t* x, const int32_t* expert_ids,
                               const float* router_w, float* y,
                               const q4t_routed_weights* weights,
                               void* workspace, size_t workspace_bytes,
                               int32_t M, int32_t k, uint32_t flags,
                               void* stream);

/* ---- q4t_moe_routed_forward for callers that cannot allocate device memory.
 * This entry point has no counterpart in the reference.  It is meant for hosts
 * whose device-memory budget is sealed after start-up (every later cudaMalloc
 * is refused by a quota, or allocation is not permitted from the calling
 * context at all), so that no workspace can be created for the call.  The
 * workspace is a fixed array of Q4T_NOALLOC_SCRATCH_BYTES inside the
 * library's device image: every GPU that loads the library holds that much
 * memory until the process exits.  Arguments and results are those of
 * q4t_moe_routed_forward (y fp32 [M,hs], zeroed by the caller, accumulated
 * into).  Limits and rules:
 *   - the batch must satisfy q4t_moe_routed_workspace_bytes(M, k, hs, moe_is,
 *     E) <= Q4T_NOALLOC_SCRATCH_BYTES (8 tokens x top-10 at hs 2048 / is 512
 *     and at hs 2560 / is 640 fit); larger batches fail with
 *     Q4T_ERR_WORKSPACE and a message that states both sizes;
 *   - the call itself performs no cudaMalloc / cudaFree and uses no allocating
 *     library routine; the first call on each device resolves the array's
 *     device address (cudaGetSymbolAddress) and sets kernel attributes, so
 *     make that first call during set-up, before any stream capture;
 *   - all calls on one device share the one array: two calls whose kernels
 *     can overlap on the GPU (different streams, no ordering between them)
 *     race on it.  Issue them on one stream or order them with events.  The
 *     array keeps the previous call's tables; the status words are cleared at
 *     the start of each call and everything else is rewritten before use.    */
#define Q4T_NOALLOC_SCRATCH_BYTES (3u << 20)
int32_t q4t_moe_routed_forward_noalloc(const uint16_t* x, const int32_t* expert_ids,
                                       const float* router_w, float* y,
                                       const q4t_routed_weights* weights,
                                       int32_t M, int32_t k, uint32_t flags,
                                       void* stream);
/* The kernel status words of the built-in scratch (no reference counterpart
 * either): q4t_moe_workspace_status for the workspace the caller of the entry
 * point above never sees.  Call it with the dimensions of the last
 * q4t_moe_routed_forward_noalloc on the current device, after synchronising
 * its stream: 0 = clean, Q4T_ERR_KERNEL = a bounded device-side wait ran out
 * and y is undefined.  Reads four bytes with cudaMemcpy; allocates nothing.    */
int32_t q4t_moe_noalloc_status(int32_t M, int32_t k, int32_t hs, int32_t moe_is,
                               int32_t E);

/* ---- MoEForwardWorkspaceBytes (include/q4t/model/moe.h:72-76,
 * src/model/moe.cu:403-417).                                                  */
size_t q4t_moe_forward_workspace_bytes(int32_t T, int32_t k, int32_t hs,
                                       int32_t moe_is, int32_t shared_is,
                                       int32_t E);
/* Offsets of the regions MoEForward leaves readable (src/model/moe.cu:449-469):
 * the routed workspace first, then logits, ids, router weights, routed fp32,
 * shared gate/up, shared activation, shared down.                             */
typedef struct {
  size_t routed_ws, logits, expert_ids, router_w, routed, shared_gu,
      shared_act, shared_down;
  size_t slot_ids;   /* int32 [T,k]: slot mode only, the ids the GEMMs consumed */
  size_t total;
} q4t_forward_ws_layout;
int32_t q4t_moe_forward_workspace_layout(int32_t T, int32_t k, int32_t hs,
                                         int32_t moe_is, int32_t shared_is,
                                         int32_t E, q4t_forward_ws_layout* out);

/* ---- MoEForward (include/q4t/model/moe.h:78-114, src/model/moe.cu:427-976):
 * router logits + top-k, routed NVFP4 experts, BF16 shared expert, sigmoid-
 * gated combine; y bf16 [T,hs], no residual add.  T <= 0 is a no-op; k must
 * be in [1,16] ("k out of range"); a short workspace fails with "workspace
 * too small".  fixed_ids (may be NULL) replaces the selected experts by a
 * caller-supplied int32 [T,k] table while the weights are still the softmax of
 * the current logits at those ids (the replay hook, moe.cu:214-237).
 * flags: bit 0 = materialise the bf16 gate|up projections (gu_out and the
 * shared expert's), bit 1 = materialise the fp32 routed sum in the workspace's
 * `routed` region; both are what the reference always writes and only its
 * diagnostics read, so they are off unless asked for; bit 2 = no decode-sized
 * path for the routed experts, bit 3 = that path up to 128 tokens (see
 * q4t_moe_routed_forward).                                                    */
int32_t q4t_moe_forward(const uint16_t* x, const q4t_routed_weights* routed,
                        const q4t_extra_weights* extra, uint16_t* y, int32_t T,
                        int32_t k, void* workspace, size_t workspace_bytes,
                        const int32_t* fixed_ids, uint32_t flags, void* stream);

/* ---- MoEForward with the two optional per-layer hooks the engine passes on
 * every layer (src/model/decoder_layer.cu:700-703):
 *   trace_ids_out  : RouterCollector::CaptureLayer (src/model/moe.cu:485-488,
 *                    src/trace/router_collector.cpp:245-266): when not NULL, the
 *                    selected expert ids int32 [T,k] are copied to this device
 *                    buffer on the stream right after the top-k (the ORIGINAL
 *                    ids, also in slot mode).  NULL: nothing is captured.
 *   slot_of_expert : slot mode (include/q4t/quant/moe_weights.h:47-51,
 *                    include/q4t/model/moe.h:96-103).  `routed` then describes
 *                    routed->E RESIDENT SLOTS (each slot's bytes are one expert
 *                    slice) while the router still chooses among extra->E
 *                    experts; this device table int32 [extra->E] maps an expert
 *                    to its slot (negative or >= routed->E: not resident, its
 *                    (token,slot) entries are skipped).  The reference resolves
 *                    the slots on the host after reading the ids back; here the
 *                    residency tier (out of this library's scope) publishes its
 *                    table to the device and no host synchronisation happens.
 *                    The workspace keeps the original ids in `expert_ids` and
 *                    the slots in `slot_ids`.  NULL: routed->E == extra->E.
 * hc_*            : the layer's gated residual write fused into the final
 *                    combine (GatedResidualFrame::Write after MoEForward,
 *                    src/model/decoder_layer.cu:708, CombineWithGateKernel,
 *                    src/model/hyperconnection.cu:286-305): with hc_count = hc
 *                    branches (0 = off), hc_out[t, b, c] = bf16(hc_residual[t, b, c]
 *                    + y[t, c] * hc_inject_gate[t, b]) for b < hc, computed from
 *                    the bf16-rounded y with one fused multiply-add as the
 *                    reference's kernel compiles to.  hc_residual / hc_out are
 *                    bf16 [T, hc*hs] (16-byte aligned, may not overlap y),
 *                    hc_inject_gate is bf16 [T, hc] as ApplyInjectGateKernel
 *                    leaves it (2*sigmoid(inject/hc)).  y is still written.
 * norm_*          : the step between two layers of a decode stack fused into the
 *                    final combine: with norm_residual != NULL (bf16 [T,hs], the
 *                    residual stream, read and written) norm_residual <-
 *                    bf16(norm_residual + y) and norm_out (bf16 [T,hs], distinct
 *                    from norm_residual; it may be the buffer x points to) <-
 *                    RMSNorm(norm_residual) with eps norm_eps and no weight: bit
 *                    for bit what q4t_residual_rmsnorm_bf16 computes after the
 *                    layer.  hs a multiple of 8, at most 8192.  y is still written.
 * fixed_ids and flags as in q4t_moe_forward.                                   */
typedef struct q4t_forward_options {
  const int32_t* fixed_ids;
  int32_t* trace_ids_out;
  const int32_t* slot_of_expert;
  uint32_t flags;
  int32_t hc_count;
  const uint16_t* hc_residual;
  const uint16_t* hc_inject_gate;
  uint16_t* hc_out;
  uint16_t* norm_residual;
  uint16_t* norm_out;
  float norm_eps;
} q4t_forward_options;
int32_t q4t_moe_forward_ex(const uint16_t* x, const q4t_routed_weights* routed,
                           const q4t_extra_weights* extra, uint16_t* y, int32_t T,
                           int32_t k, void* workspace, size_t workspace_bytes,
                           const q4t_forward_options* options, void* stream);

/* ---- BF16 routed experts: the MTP draft layer's MoE (include/q4t/mtp/moe_bf16.h:
 * 36-123, src/mtp/moe_bf16.cu).  Same orchestration as the NVFP4 layer with
 * plain BF16 expert GEMMs: h = bf16(x.W_gu[e]^T), inter = bf16((g*sigmoid(g))*u),
 * out = bf16(inter.W_dn[e]^T), y[t] += r[t,e]*out.  Weights as in the
 * checkpoint: gu [E, 2*moe_is, hs] (gate rows then up rows per expert), down
 * [E, hs, moe_is], bf16 row-major.  The routed sum is formed in slot order
 * (the reference adds with atomicAdd in no particular order), the router is
 * the one of q4t_moe_forward (same selected set and weights as the MTP path's
 * own top-k kernel, ids in value order).  y of the routed call: fp32 [M,hs],
 * accumulated into (zero it first), as in MoeBf16RoutedForward.              */
typedef struct q4t_bf16_expert_weights {
  int32_t E, hs, moe_is, reserved;
  const uint16_t* gu;
  const uint16_t* down;
} q4t_bf16_expert_weights;
size_t q4t_moe_bf16_workspace_bytes(int32_t M, int32_t k, int32_t hs,
                                    int32_t moe_is, int32_t E);
int32_t q4t_moe_bf16_routed_forward(const uint16_t* x, const int32_t* expert_ids,
                                    const float* router_w, float* y,
                                    const q4t_bf16_expert_weights* weights,
                                    void* workspace, size_t workspace_bytes,
                                    int32_t M, int32_t k, void* stream);
size_t q4t_moe_bf16_forward_workspace_bytes(int32_t T, int32_t k, int32_t hs,
                                            int32_t moe_is, int32_t shared_is,
                                            int32_t E);
int32_t q4t_moe_bf16_forward(const uint16_t* x,
                             const q4t_bf16_expert_weights* routed,
                             const q4t_extra_weights* extra, uint16_t* y,
                             int32_t T, int32_t k, void* workspace,
                             size_t workspace_bytes, void* stream);

/* ---- expert parallelism.  The reference engine is single-GPU (it has no
 * NCCL/MPI code), so these three entry points have no counterpart there; they
 * cut q4t_moe_forward at the two points where rows cross GPUs.  Experts are
 * split into n_ranks contiguous blocks of E/n_ranks; the caller moves the
 * buffers between ranks (all-to-all with the counts as split sizes).
 *
 * q4t_ep_dispatch: sorts the (token,slot) entries of this rank's T tokens by
 * the rank that owns their expert (stable) and gathers the bf16 token rows in
 * that order.  send_rows [T*k, hs], send_local_expert [T*k] (expert index on
 * its owner), send_counts [n_ranks] (rows per destination), row_of_flat [T*k]
 * (position of (token,slot) in send order, -1 for ids outside [0,E)).        */
size_t q4t_ep_dispatch_workspace_bytes(int32_t T, int32_t k, int32_t n_ranks);
int32_t q4t_ep_dispatch(const uint16_t* x, const int32_t* expert_ids, int32_t T,
                        int32_t k, int32_t E, int32_t hs, int32_t n_ranks,
                        uint16_t* send_rows, int32_t* send_local_expert,
                        int32_t* send_counts, int32_t* row_of_flat,
                        void* workspace, size_t workspace_bytes, void* stream);
/* q4t_moe_expert_rows: the routed-expert FFN on `rows` received rows, each
 * with one local expert: out_rows[r] = bf16 down-projection of row r through
 * expert local_expert[r], un-weighted, in the order received (bit-identical
 * to the dn_out rows of q4t_moe_routed_forward).  `weights` describes this
 * rank's expert block (E = experts on this rank).  workspace >=
 * q4t_moe_routed_workspace_bytes(rows, 1, hs, moe_is, E).                     */
int32_t q4t_moe_expert_rows(const uint16_t* x_rows, const int32_t* local_expert,
                            uint16_t* out_rows, const q4t_routed_weights* weights,
                            void* workspace, size_t workspace_bytes,
                            int32_t rows, uint32_t flags, void* stream);
/* q4t_moe_finish: on the rank that owns the tokens, the shared expert and the
 * gated combine (src/model/moe.cu:291-321, 955-971) with the routed rows taken
 * from expert_rows [T*k, hs] (send order) through row_of_flat.                */
size_t q4t_moe_finish_workspace_bytes(int32_t T, int32_t hs, int32_t shared_is);
int32_t q4t_moe_finish(const uint16_t* x, const uint16_t* expert_rows,
                       const int32_t* row_of_flat, const float* router_w,
                       const q4t_extra_weights* extra, uint16_t* y, int32_t T,
                       int32_t k, void* workspace, size_t workspace_bytes,
                       void* stream);

/* The two halves of q4t_moe_finish, for callers that run the shared expert
 * beside the exchange (another stream): q4t_moe_shared_expert leaves the
 * shared expert's down projection in the workspace, q4t_moe_combine reads it
 * from there.  Same workspace for both (q4t_moe_finish_workspace_bytes).      */
int32_t q4t_moe_shared_expert(const uint16_t* x, const q4t_extra_weights* extra,
                              int32_t T, void* workspace, size_t workspace_bytes,
                              void* stream);
int32_t q4t_moe_combine(const uint16_t* x, const uint16_t* expert_rows,
                        const int32_t* row_of_flat, const float* router_w,
                        const q4t_extra_weights* extra, uint16_t* y, int32_t T,
                        int32_t k, void* workspace, size_t workspace_bytes,
                        void* stream);

/* ---- expert parallelism over peer memory (no reference counterpart either).
 * Instead of exchanging rows through collectives, the kernels themselves write
 * into the other GPUs' memory.  Every rank owns two buffers its peers can
 * write: a GATHERED token buffer (codes [world*tokens_per_rank, hs/2] and
 * scale bytes [world*tokens_per_rank, hs/16], row-major, not swizzled) and a
 * LANDING buffer dn_rows [tokens_per_rank*k, hs].  One step:
 *   1. q4t_ep_publish: quantises this rank's tokens once (the layer's single
 *      gate/up input scale) and stores codes and scales into its block of
 *      EVERY rank's gathered buffer (stores over NVLink from the quantiser).
 *   2. the ranks' int32 [tokens_per_rank,k] expert ids are all-gathered in
 *      rank order (any collective; it also orders step 1 before step 3).
 *   3. q4t_moe_expert_peer: keeps the (token,slot) entries of ALL ranks whose
 *      expert lives here, groups their codes from the local gathered buffer,
 *      runs the gate/up and down GEMMs; the down GEMM's epilogue stores each
 *      bf16 row directly at dn_rows[owner][(token*k + slot), :] (stores over
 *      NVLink, overlapped with the tiles still being computed).
 *   4. a barrier (any collective) = "all rows have landed"; then
 *      q4t_moe_finish on the landing buffer, row_of_flat from q4t_ep_flat_rows.
 * The caller issues the collectives stream-ordered; no kernel waits on another
 * rank.  Results are bit-identical to q4t_moe_forward on one GPU.  Needs
 * weights->gu_input_scale_uniform > 0 (one input scale for all experts;
 * otherwise use the row-exchange entry points above).
 *
 * q4t_peer_buffer_*: device buffers that another process on the same node can
 * map: alloc (zero-filled) / free on the owner, export -> 64-byte handle to send to the peers
 * (any host channel), open/close on a peer.                                    */
#define Q4T_EP_MAX_RANKS 8
#define Q4T_PEER_HANDLE_BYTES 64
typedef struct q4t_ep_peer_table {
  int32_t world, rank;
  int32_t tokens_per_rank;  /* rows every rank publishes (pad the last rank's) */
  int32_t expert_map;       /* 0: expert e on rank e / (E/world), local e % (E/world);
                               1: on rank e % world, local e / world;
                               2: by `placement` (below)                       */
  const uint8_t* xq_packed[Q4T_EP_MAX_RANKS]; /* rank r's gathered code buffer  */
  const uint8_t* xq_sf[Q4T_EP_MAX_RANKS];     /* rank r's gathered scale bytes  */
  uint16_t* dn_rows[Q4T_EP_MAX_RANKS];        /* rank r's landing buffer        */
  /* expert_map 2: THIS rank's device table int32 [experts_total]: -1 = the
   * expert is served elsewhere; v >= 0 = served here as local expert v for
   * tokens of every rank; v | Q4T_EP_REPLICATED = the expert is replicated on
   * all ranks and served here, as local expert v, for this rank's own tokens
   * only.  The ranks' tables must agree (every expert either has exactly one
   * rank with v >= 0 or is replicated everywhere).                            */
  const int32_t* placement;
  int32_t experts_total;
  int32_t reserved;
  /* expert_map 2, optional: device table int32 [experts_total], the same on every
   * rank: the rank that serves expert e for all tokens, or a negative value for an
   * expert replicated on every rank.  With it q4t_ep_route_publish sends a token only
   * to the ranks that serve one of its selected experts; without it (NULL) every
   * token goes to every rank.  Maps 0 and 1 need no table.                      */
  const int32_t* expert_owner;
  /* Optional: rank r's SYNC buffer (q4t_ep_sync_buffer_bytes, zeroed once by its owner,
   * peer-writable like the others).  With it the two collectives of a step can be
   * replaced by q4t_ep_post_ids / q4t_ep_post_rows / q4t_ep_wait (below).            */
  uint8_t* sync[Q4T_EP_MAX_RANKS];
} q4t_ep_peer_table;
#define Q4T_EP_REPLICATED (1 << 30)
/* ---- the step's two collectives as kernels over peer memory (optional).
 * A SYNC buffer holds, at offset 0, two rows of Q4T_EP_MAX_RANKS uint32 flags (row 0:
 * "rank r's tokens and ids of step `epoch` are in your buffers", row 1: "rank r's
 * result rows of step `epoch` have been stored"), at offset 128 an int32 status word,
 * and from Q4T_EP_SYNC_IDS_OFFSET on the gathered ids int32 [world*tokens_per_rank, k]
 * in rank order (what q4t_moe_expert_peer takes as ids_all).  Per step, with a counter
 * `epoch` that every rank advances by one (start at 1; flags start at 0):
 *   q4t_ep_route_publish; q4t_ep_post_ids(ids, …, epoch)    -- stores the ids block into
 *       every rank's SYNC buffer, then raises flag row 0 there (after a system fence,
 *       so the published tokens are visible too);
 *   q4t_ep_wait(…, 0, epoch); q4t_moe_expert_peer(own SYNC + Q4T_EP_SYNC_IDS_OFFSET, …);
 *   q4t_ep_post_rows(…, epoch); q4t_ep_wait(…, 1, epoch); q4t_ep_combine.
 * All stream-ordered, no host synchronisation, no collective library call.  The waits
 * are bounded (about two seconds): a rank that never posts makes the others' wait give
 * up and raise the status word, which q4t_ep_sync_status reports (synchronise the
 * stream first); the context stays usable.  Every rank must run the same sequence.    */
#define Q4T_EP_SYNC_IDS_OFFSET 256
size_t q4t_ep_sync_buffer_bytes(int32_t world, int32_t tokens_per_rank, int32_t k);
int32_t q4t_ep_post_ids(const int32_t* expert_ids, const q4t_ep_peer_table* peers, int32_t k,
                        uint32_t epoch, void* stream);
int32_t q4t_ep_post_rows(const q4t_ep_peer_table* peers, uint32_t epoch, void* stream);
int32_t q4t_ep_wait(const q4t_ep_peer_table* peers, int32_t phase, uint32_t epoch, void* stream);
int32_t q4t_ep_sync_status(const q4t_ep_peer_table* peers);
int32_t q4t_peer_buffer_alloc(size_t bytes, void** ptr);
int32_t q4t_peer_buffer_free(void* ptr);
int32_t q4t_peer_buffer_export(const void* ptr, uint8_t handle[Q4T_PEER_HANDLE_BYTES]);
int32_t q4t_peer_buffer_open(const uint8_t handle[Q4T_PEER_HANDLE_BYTES], void** ptr);
int32_t q4t_peer_buffer_close(void* ptr);
/* x: bf16 [tokens_per_rank, hs]; hs a multiple of 64.                         */
int32_t q4t_ep_publish(const uint16_t* x, const q4t_ep_peer_table* peers, int32_t hs,
                       float input_scale, void* stream);
/* The selective form of step 1: expert_ids int32 [tokens_per_rank,k] (already
 * selected); a token's codes are stored only into the gathered buffers of the
 * ranks that own one of its k experts (by expert_map / expert_owner) and into
 * this rank's own.  Ranks read only the tokens of entries they serve, so the
 * other slots of their buffers may keep stale rows.  At 8 ranks with the most
 * used experts replicated this moves a twelfth of the bytes of q4t_ep_publish. */
int32_t q4t_ep_publish_selected(const uint16_t* x, const int32_t* expert_ids,
                                const q4t_ep_peer_table* peers, int32_t k, int32_t E,
                                int32_t hs, float input_scale, void* stream);
/* Steps 1 and 4 as single calls, for drivers that count host overhead:
 * q4t_ep_route_publish = router logits (scratch bf16 [tokens_per_rank, E]) + top-k
 * (expert_ids, router_w) + q4t_ep_publish_selected (q4t_ep_publish for expert_map 2
 * without an owner table), and it starts the shared expert on the library's side
 * stream (result left in finish_workspace);
 * q4t_ep_combine = wait for that shared expert + q4t_ep_flat_rows (row_of_flat:
 * int32 [T*k] scratch) + q4t_moe_combine on the landing buffer.                */
int32_t q4t_ep_route_publish(const uint16_t* x, const q4t_extra_weights* extra,
                             const q4t_ep_peer_table* peers, int32_t k,
                             float input_scale, uint16_t* logits,
                             int32_t* expert_ids, float* router_w,
                             void* finish_workspace, size_t finish_workspace_bytes,
                             void* stream);
int32_t q4t_ep_combine(const uint16_t* x, const uint16_t* landed_rows,
                       const int32_t* expert_ids, const float* router_w,
                       const q4t_extra_weights* extra, uint16_t* y, int32_t T,
                       int32_t k, int32_t* row_of_flat, void* finish_workspace,
                       size_t finish_workspace_bytes, void* stream);
/* ids_all: int32 [world*tokens_per_rank, k] global expert ids (entries outside
 * [0, E_local*world) are skipped); weights: this rank's experts.              */
size_t q4t_moe_expert_peer_workspace_bytes(int32_t tokens_all, int32_t k, int32_t hs,
                                           int32_t moe_is, int32_t E_local);
int32_t q4t_moe_expert_peer(const int32_t* ids_all, const q4t_ep_peer_table* peers,
                            const q4t_routed_weights* weights, int32_t k,
                            void* workspace, size_t workspace_bytes,
                            uint32_t flags, void* stream);
/* row_of_flat[f] = f where expert_ids[f] is in [0,E), else -1: the table
 * q4t_moe_finish needs when the rows arrive in (token,slot) order.            */
int32_t q4t_ep_flat_rows(const int32_t* expert_ids, int32_t rows, int32_t E,
                         int32_t* row_of_flat, void* stream);

/* ---- the step between two layers of a decode stack (the 48-layer harness):
 * x <- bf16(x + y) in place (fp32 add, one rounding; y may be NULL), then
 * h <- x * rsqrt(mean(x^2) + eps) in bf16, no learned weight.  Summation order
 * of GroupedRmsNormKernel (src/model/hyperconnection.cu:55-110) with the
 * correctly rounded reciprocal square root in place of rsqrtf.  x, y, h: bf16
 * [T, hs], 16-byte aligned; hs a multiple of 8.                                */
int32_t q4t_residual_rmsnorm_bf16(uint16_t* x, const uint16_t* y, uint16_t* h,
                                  int32_t T, int32_t hs, float eps, void* stream);

/* Reads the kernel status words of a workspace after the stream has been
 * synchronised by the caller: 0 = clean, otherwise a bounded device-side wait
 * ran out (the output is then undefined).  Copies with cudaMemcpy.            */
int32_t q4t_moe_workspace_status(const void* workspace, int32_t M, int32_t k,
                                 int32_t hs, int32_t moe_is, int32_t E);

/* ---- stage timer, after MoESubTiming (include/q4t/quant/moe_subtiming.h:
 * 14-97): when enabled, q4t_moe_forward / q4t_moe_routed_forward record CUDA
 * events on the caller's stream between their stages.  q4t_stage_timing_read
 * synchronises on the last event of the calling thread's most recent call and
 * writes the elapsed milliseconds of the Q4T_NUM_STAGES stages:
 *   0 router logits, 1 top-k, 2 permutation tables, 3 gather-quantise,
 *   4 gate/up GEMM (+SwiGLU, requantise), 5 down GEMM, 6 shared expert,
 *   7 combine.  Stages a call does not run read as 0.  Off by default.        */
#define Q4T_NUM_STAGES 8
int32_t q4t_stage_timing_enable(int32_t enable);
int32_t q4t_stage_timing_read(float* ms_out);

#ifdef __cplusplus
}
#endif
#endif /* Q4T_MOE_B200_H_ */
