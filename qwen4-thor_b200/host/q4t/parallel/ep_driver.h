// Expert-parallel MoE layer for a C++ engine: one process (or thread) per GPU, NCCL for the
// collectives, the C ABI of libq4t_moe_b200 for everything else.  The reference engine is
// single-GPU, so nothing here has a counterpart there; the classes take what an engine
// already has (an ncclComm_t, a stream, this rank's weights) and give back MoEForward's
// result for this rank's tokens, bit-identical to the single-GPU layer.
//
//   PeerExpertParallel     the default: tokens and result rows travel as stores into peer
//                          memory issued by the quantiser and by the down GEMM's epilogue;
//                          the expert ids and the two orderings of a step ("published",
//                          "rows landed") travel the same way, as flag kernels over peer
//                          memory (q4t_ep_post_ids / q4t_ep_post_rows / q4t_ep_wait), or, with
//                          use_collectives, as ncclAllGather + a one-word ncclAllReduce.  NCCL
//                          is otherwise only used once, to exchange the buffer handles.  No host
//                          synchronisation per step.
//   RowExchangeExpertParallel  the plain form: bf16 rows both ways with grouped
//                          ncclSend / ncclRecv (an all-to-all-v); one host synchronisation per
//                          step for the split sizes.  Contiguous expert blocks.
//
// Buffers that peers write are allocated by the library (q4t_peer_buffer_*) and mapped across
// processes with 64-byte handles, exchanged here through NCCL itself.
#pragma once
#include <cuda_runtime.h>
#include <nccl.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

#include "q4t/status.h"
#include "q4t_moe_b200.h"

namespace q4t::parallel {

namespace detail {
inline Status Cuda(cudaError_t e, const char* what) {
  return e == cudaSuccess ? Status() : Status::Fail(std::string(what) + ": " + cudaGetErrorString(e));
}
inline Status Nccl(ncclResult_t r, const char* what) {
  return r == ncclSuccess ? Status() : Status::Fail(std::string(what) + ": " + ncclGetErrorString(r));
}
inline Status Abi(int rc) { return rc == Q4T_OK ? Status() : Status::Fail(q4t_last_error()); }
#define Q4T_EP_TRY(expr)          \
  do {                            \
    ::q4t::Status s__ = (expr);   \
    if (!s__.ok()) return s__;    \
  } while (0)
}  // namespace detail

struct EpShape {
  int world = 1, rank = 0;
  int tokens_per_rank = 0;  // every rank runs the same number of tokens per step
  int k = 0;                // experts per token
  int experts = 0;          // experts the router chooses among (all ranks together)
  int hs = 0, moe_is = 0, shared_is = 0;
};

class PeerExpertParallel {
 public:
  ~PeerExpertParallel() { Free(); }

  // local: this rank's experts (local.E of them) in local order; extra: router + shared expert
  // (replicated).  expert_map 0 / 1 as in q4t_ep_peer_table; for a placement table pass
  // expert_map 2 with placement (this rank's table) and expert_owner (the same on all ranks),
  // both device int32 [experts].  Collective: every rank calls it.
  Status Init(ncclComm_t comm, cudaStream_t stream, const EpShape& shape, const q4t_routed_weights& local,
              const q4t_extra_weights& extra, int expert_map = 0, const int32_t* placement = nullptr,
              const int32_t* expert_owner = nullptr, bool use_collectives = false) {
    using namespace detail;
    Free();
    comm_ = comm;
    collectives_ = use_collectives;
    epoch_ = 0;
    s_ = shape;
    local_ = local;
    extra_ = extra;
    if (s_.world < 1 || s_.world > Q4T_EP_MAX_RANKS) return Status::Fail("world must be in [1, 8]");
    if (!(local.gu_input_scale_uniform > 0.0f)) return Status::Fail("the peer path needs one gate/up input scale");
    const size_t T = s_.tokens_per_rank, k = s_.k, hs = s_.hs, W = s_.world;
    const size_t sizes[kBuffers] = {W * T * (hs / 2), W * T * (hs / 16), T * k * hs * 2,
                                    q4t_ep_sync_buffer_bytes(s_.world, s_.tokens_per_rank, s_.k)};
    for (int i = 0; i < kBuffers; ++i) Q4T_EP_TRY(Abi(q4t_peer_buffer_alloc(sizes[i], &own_[i])));
    // exchange the handles: 4 x 64 bytes per rank, all-gathered through a device staging buffer
    std::vector<uint8_t> mine(kBuffers * Q4T_PEER_HANDLE_BYTES), all(W * mine.size());
    for (int i = 0; i < kBuffers; ++i)
      Q4T_EP_TRY(Abi(q4t_peer_buffer_export(own_[i], mine.data() + i * Q4T_PEER_HANDLE_BYTES)));
    uint8_t* d_h = nullptr;
    Q4T_EP_TRY(Cuda(cudaMalloc(reinterpret_cast<void**>(&d_h), all.size() + mine.size()), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMemcpyAsync(d_h + all.size(), mine.data(), mine.size(), cudaMemcpyHostToDevice, stream), "copy"));
    Q4T_EP_TRY(Nccl(ncclAllGather(d_h + all.size(), d_h, mine.size(), ncclUint8, comm, stream), "ncclAllGather(handles)"));
    Q4T_EP_TRY(Cuda(cudaMemcpyAsync(all.data(), d_h, all.size(), cudaMemcpyDeviceToHost, stream), "copy"));
    Q4T_EP_TRY(Cuda(cudaStreamSynchronize(stream), "sync"));
    cudaFree(d_h);
    std::memset(&table_, 0, sizeof(table_));
    table_.world = s_.world;
    table_.rank = s_.rank;
    table_.tokens_per_rank = s_.tokens_per_rank;
    table_.expert_map = expert_map;
    table_.placement = placement;
    table_.experts_total = placement ? s_.experts : 0;
    table_.expert_owner = expert_owner;
    for (int r = 0; r < s_.world; ++r) {
      void* p[kBuffers];
      for (int i = 0; i < kBuffers; ++i) {
        if (r == s_.rank) {
          p[i] = own_[i];
        } else {
          Q4T_EP_TRY(Abi(q4t_peer_buffer_open(all.data() + (r * kBuffers + i) * Q4T_PEER_HANDLE_BYTES, &p[i])));
          opened_.push_back(p[i]);
        }
      }
      table_.xq_packed[r] = static_cast<const uint8_t*>(p[0]);
      table_.xq_sf[r] = static_cast<const uint8_t*>(p[1]);
      table_.dn_rows[r] = static_cast<uint16_t*>(p[2]);
      table_.sync[r] = static_cast<uint8_t*>(p[3]);
    }
    // per-step scratch
    ws_bytes_ = q4t_moe_expert_peer_workspace_bytes(s_.world * s_.tokens_per_rank, s_.k, s_.hs, s_.moe_is, local.E);
    fin_bytes_ = q4t_moe_finish_workspace_bytes(s_.tokens_per_rank, s_.hs, s_.shared_is);
    if (ws_bytes_ == 0 || fin_bytes_ == 0) return Status::Fail("unsupported dims");
    const size_t R = T * k;
    Q4T_EP_TRY(Cuda(cudaMalloc(&ws_, ws_bytes_), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMalloc(&fin_, fin_bytes_), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMalloc(reinterpret_cast<void**>(&logits_), T * s_.experts * 2), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMalloc(reinterpret_cast<void**>(&ids_), R * 4), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMalloc(reinterpret_cast<void**>(&rw_), R * 4), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMalloc(reinterpret_cast<void**>(&ids_all_), W * R * 4), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMalloc(reinterpret_cast<void**>(&rof_), R * 4), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMalloc(reinterpret_cast<void**>(&sync_), 4), "cudaMalloc"));
    Q4T_EP_TRY(Cuda(cudaMemsetAsync(sync_, 0, 4, stream), "memset"));
    return Cuda(cudaStreamSynchronize(stream), "sync");
  }

  // One layer step for this rank's tokens: x, y bf16 [tokens_per_rank, hs] on the device.
  // Everything is enqueued on `stream`; every rank calls it.
  Status Step(const uint16_t* x, uint16_t* y, cudaStream_t stream) {
    using namespace detail;
    const int T = s_.tokens_per_rank, k = s_.k;
    Q4T_EP_TRY(Abi(q4t_ep_route_publish(x, &extra_, &table_, k, local_.gu_input_scale_uniform, logits_, ids_, rw_, fin_,
                                        fin_bytes_, stream)));
    if (collectives_) {
      // the ids of all ranks, in rank order; also orders "published" before "used"
      Q4T_EP_TRY(Nccl(ncclAllGather(ids_, ids_all_, static_cast<size_t>(T) * k, ncclInt32, comm_, stream),
                      "ncclAllGather(ids)"));
      Q4T_EP_TRY(Abi(q4t_moe_expert_peer(ids_all_, &table_, &local_, k, ws_, ws_bytes_, 0, stream)));
      // "all rows have landed": every rank's down GEMM precedes its contribution in stream order
      Q4T_EP_TRY(Nccl(ncclAllReduce(sync_, sync_, 1, ncclInt32, ncclSum, comm_, stream), "ncclAllReduce(barrier)"));
    } else {
      // the same two steps as kernels over peer memory: ids stored into every rank's sync
      // buffer, flags raised and awaited on the device
      ++epoch_;
      Q4T_EP_TRY(Abi(q4t_ep_post_ids(ids_, &table_, k, epoch_, stream)));
      Q4T_EP_TRY(Abi(q4t_ep_wait(&table_, 0, epoch_, stream)));
      const int32_t* gathered = reinterpret_cast<const int32_t*>(static_cast<uint8_t*>(own_[3]) + Q4T_EP_SYNC_IDS_OFFSET);
      Q4T_EP_TRY(Abi(q4t_moe_expert_peer(gathered, &table_, &local_, k, ws_, ws_bytes_, 0, stream)));
      Q4T_EP_TRY(Abi(q4t_ep_post_rows(&table_, epoch_, stream)));
      Q4T_EP_TRY(Abi(q4t_ep_wait(&table_, 1, epoch_, stream)));
    }
    return Abi(q4t_ep_combine(x, static_cast<const uint16_t*>(own_[2]), ids_, rw_, &extra_, y, T, k, rof_, fin_,
                              fin_bytes_, stream));
  }

  // After synchronising the stream: did a bounded device-side wait run out?
  Status CheckStatus() const {
    Status s = detail::Abi(q4t_moe_workspace_status(ws_, s_.world * s_.tokens_per_rank, s_.k, s_.hs, s_.moe_is, local_.E));
    if (!s.ok() || collectives_) return s;
    return detail::Abi(q4t_ep_sync_status(&table_));   // a wait for another rank that ran out
  }

  void Free() {
    for (void* p : opened_) q4t_peer_buffer_close(p);
    opened_.clear();
    for (void*& p : own_) {
      if (p) q4t_peer_buffer_free(p);
      p = nullptr;
    }
    for (void* p : {ws_, fin_, static_cast<void*>(logits_), static_cast<void*>(ids_), static_cast<void*>(rw_),
                    static_cast<void*>(ids_all_), static_cast<void*>(rof_), static_cast<void*>(sync_)})
      if (p) cudaFree(p);
    ws_ = fin_ = nullptr;
    logits_ = nullptr;
    ids_ = ids_all_ = rof_ = sync_ = nullptr;
    rw_ = nullptr;
  }

 private:
  ncclComm_t comm_ = nullptr;
  EpShape s_;
  q4t_routed_weights local_{};
  q4t_extra_weights extra_{};
  q4t_ep_peer_table table_{};
  static constexpr int kBuffers = 4;   // gathered codes, gathered scales, landing rows, sync (flags + gathered ids)
  void* own_[kBuffers] = {nullptr, nullptr, nullptr, nullptr};
  bool collectives_ = false;
  uint32_t epoch_ = 0;
  std::vector<void*> opened_;
  void* ws_ = nullptr;
  void* fin_ = nullptr;
  size_t ws_bytes_ = 0, fin_bytes_ = 0;
  uint16_t* logits_ = nullptr;
  int32_t* ids_ = nullptr;
  float* rw_ = nullptr;
  int32_t* ids_all_ = nullptr;
  int32_t* rof_ = nullptr;
  int32_t* sync_ = nullptr;
};

class RowExchangeExpertParallel {
 public:
  ~RowExchangeExpertParallel() { Free(); }

  // local: this rank's contiguous block of experts/world experts.  cap_rows: the most rows this
  // rank may receive in one step (world * tokens_per_rank * k is always enough).
  Status Init(ncclComm_t comm, const EpShape& shape, const q4t_routed_weights& local, const q4t_extra_weights& extra,
              int cap_rows) {
    using namespace detail;
    Free();
    comm_ = comm;
    s_ = shape;
    local_ = local;
    extra_ = extra;
    cap_ = cap_rows;
    if (s_.experts % s_.world) return Status::Fail("experts must be a multiple of world");
    const size_t T = s_.tokens_per_rank, R = T * s_.k, hs = s_.hs, W = s_.world;
    disp_bytes_ = q4t_ep_dispatch_workspace_bytes(s_.tokens_per_rank, s_.k, s_.world);
    ews_bytes_ = q4t_moe_routed_workspace_bytes(cap_, 1, s_.hs, s_.moe_is, local.E);
    fin_bytes_ = q4t_moe_finish_workspace_bytes(s_.tokens_per_rank, s_.hs, s_.shared_is);
    if (!disp_bytes_ || !ews_bytes_ || !fin_bytes_) return Status::Fail("unsupported dims");
    auto alloc = [&](void** p, size_t bytes) { return Cuda(cudaMalloc(p, bytes ? bytes : 4), "cudaMalloc"); };
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&logits_), T * s_.experts * 2));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&ids_), R * 4));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&rw_), R * 4));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&send_rows_), R * hs * 2));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&send_local_), R * 4));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&send_counts_), W * 4));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&counts_all_), W * W * 4));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&rof_), R * 4));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&ret_rows_), R * hs * 2));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&recv_rows_), static_cast<size_t>(cap_) * hs * 2));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&recv_local_), static_cast<size_t>(cap_) * 4));
    Q4T_EP_TRY(alloc(reinterpret_cast<void**>(&out_rows_), static_cast<size_t>(cap_) * hs * 2));
    Q4T_EP_TRY(alloc(&disp_, disp_bytes_));
    Q4T_EP_TRY(alloc(&ews_, ews_bytes_));
    Q4T_EP_TRY(alloc(&fin_, fin_bytes_));
    return Status();
  }

  Status Step(const uint16_t* x, uint16_t* y, cudaStream_t stream) {
    using namespace detail;
    const int T = s_.tokens_per_rank, k = s_.k, W = s_.world, hs = s_.hs;
    Q4T_EP_TRY(Abi(q4t_bf16_linear(x, extra_.gate, logits_, T, s_.experts, hs, stream)));
    Q4T_EP_TRY(Abi(q4t_router_topk(logits_, ids_, rw_, T, s_.experts, k, stream)));
    Q4T_EP_TRY(Abi(q4t_ep_dispatch(x, ids_, T, k, s_.experts, hs, W, send_rows_, send_local_, send_counts_, rof_, disp_,
                                   disp_bytes_, stream)));
    // every rank learns every rank's split sizes (one host synchronisation per step)
    Q4T_EP_TRY(Nccl(ncclAllGather(send_counts_, counts_all_, W, ncclInt32, comm_, stream), "ncclAllGather(counts)"));
    std::vector<int32_t> c(static_cast<size_t>(W) * W);
    Q4T_EP_TRY(Cuda(cudaMemcpyAsync(c.data(), counts_all_, c.size() * 4, cudaMemcpyDeviceToHost, stream), "copy"));
    Q4T_EP_TRY(Cuda(cudaStreamSynchronize(stream), "sync"));
    // c[src * W + dst] rows go from src to dst
    std::vector<size_t> send_off(W + 1, 0), recv_off(W + 1, 0);
    for (int r = 0; r < W; ++r) {
      send_off[r + 1] = send_off[r] + c[static_cast<size_t>(s_.rank) * W + r];
      recv_off[r + 1] = recv_off[r] + c[static_cast<size_t>(r) * W + s_.rank];
    }
    const size_t n_recv = recv_off[W];
    if (n_recv > static_cast<size_t>(cap_)) return Status::Fail("received more rows than the configured capacity");
    Q4T_EP_TRY(Nccl(ncclGroupStart(), "ncclGroupStart"));
    for (int r = 0; r < W; ++r) {
      const size_t ns = send_off[r + 1] - send_off[r], nr = recv_off[r + 1] - recv_off[r];
      if (ns) {
        ncclSend(send_rows_ + send_off[r] * hs, ns * hs, ncclBfloat16, r, comm_, stream);
        ncclSend(send_local_ + send_off[r], ns, ncclInt32, r, comm_, stream);
      }
      if (nr) {
        ncclRecv(recv_rows_ + recv_off[r] * hs, nr * hs, ncclBfloat16, r, comm_, stream);
        ncclRecv(recv_local_ + recv_off[r], nr, ncclInt32, r, comm_, stream);
      }
    }
    Q4T_EP_TRY(Nccl(ncclGroupEnd(), "ncclGroupEnd(dispatch)"));
    Q4T_EP_TRY(Abi(q4t_moe_expert_rows(recv_rows_, recv_local_, out_rows_, &local_, ews_, ews_bytes_,
                                       static_cast<int32_t>(n_recv), 0, stream)));
    Q4T_EP_TRY(Nccl(ncclGroupStart(), "ncclGroupStart"));
    for (int r = 0; r < W; ++r) {
      const size_t ns = send_off[r + 1] - send_off[r], nr = recv_off[r + 1] - recv_off[r];
      if (nr) ncclSend(out_rows_ + recv_off[r] * hs, nr * hs, ncclBfloat16, r, comm_, stream);
      if (ns) ncclRecv(ret_rows_ + send_off[r] * hs, ns * hs, ncclBfloat16, r, comm_, stream);
    }
    Q4T_EP_TRY(Nccl(ncclGroupEnd(), "ncclGroupEnd(return)"));
    return Abi(q4t_moe_finish(x, ret_rows_, rof_, rw_, &extra_, y, T, k, fin_, fin_bytes_, stream));
  }

  void Free() {
    for (void* p : {static_cast<void*>(logits_), static_cast<void*>(ids_), static_cast<void*>(rw_),
                    static_cast<void*>(send_rows_), static_cast<void*>(send_local_), static_cast<void*>(send_counts_),
                    static_cast<void*>(counts_all_), static_cast<void*>(rof_), static_cast<void*>(ret_rows_),
                    static_cast<void*>(recv_rows_), static_cast<void*>(recv_local_), static_cast<void*>(out_rows_),
                    disp_, ews_, fin_})
      if (p) cudaFree(p);
    logits_ = send_rows_ = ret_rows_ = recv_rows_ = out_rows_ = nullptr;
    ids_ = send_local_ = send_counts_ = counts_all_ = rof_ = recv_local_ = nullptr;
    rw_ = nullptr;
    disp_ = ews_ = fin_ = nullptr;
  }

 private:
  ncclComm_t comm_ = nullptr;
  EpShape s_;
  q4t_routed_weights local_{};
  q4t_extra_weights extra_{};
  int cap_ = 0;
  uint16_t *logits_ = nullptr, *send_rows_ = nullptr, *ret_rows_ = nullptr, *recv_rows_ = nullptr, *out_rows_ = nullptr;
  int32_t *ids_ = nullptr, *send_local_ = nullptr, *send_counts_ = nullptr, *counts_all_ = nullptr, *rof_ = nullptr,
          *recv_local_ = nullptr;
  float* rw_ = nullptr;
  void *disp_ = nullptr, *ews_ = nullptr, *fin_ = nullptr;
  size_t disp_bytes_ = 0, ews_bytes_ = 0, fin_bytes_ = 0;
};

}  // namespace q4t::parallel
