"""Expert-parallel MoE layer over torch.distributed (one process per GPU).

Experts are split into world_size contiguous blocks; the router and the shared
expert are replicated and run where the token lives; tokens are sharded by
rank.  One step is

    router -> dispatch (sort (token,slot) by owner rank, gather rows)
           -> all-to-all of the per-rank row counts, then of the rows
           -> routed-expert FFN on the received rows (owner of the expert)
           -> all-to-all of the bf16 result rows back
           -> shared expert + slot-order combine (owner of the token)

which yields, bit for bit, the output of the single-GPU layer on the same
tokens: rows are quantised and multiplied per row, and the combine order is the
slot order in both cases.  torch.distributed (NCCL on GPUs, gloo in the CPU
tests) is plumbing only; every arithmetic step is an `ops` call.
"""
from __future__ import annotations


class LibraryOps:
    """The five steps on the GPU through the C ABI of libq4t_moe_b200."""

    def __init__(self, q4t, layer_local, E_total, hs, k, world, T_local, cap_rows, device="cuda"):
        import ctypes as C
        import torch
        self.q4t, self.C, self.torch = q4t, C, torch
        self.L, self.E, self.hs, self.k, self.world, self.T = layer_local, E_total, hs, k, world, T_local
        self.lib = q4t.load()
        R = T_local * k
        dev = device
        self.logits = torch.empty((T_local, E_total), dtype=torch.bfloat16, device=dev)
        self.ids = torch.empty((T_local, k), dtype=torch.int32, device=dev)
        self.rw = torch.empty((T_local, k), dtype=torch.float32, device=dev)
        self.send_rows = torch.empty((R, hs), dtype=torch.bfloat16, device=dev)
        self.send_local = torch.empty((R,), dtype=torch.int32, device=dev)
        self.send_counts = torch.empty((world,), dtype=torch.int32, device=dev)
        self.row_of_flat = torch.empty((R,), dtype=torch.int32, device=dev)
        self.dispatch_ws = torch.empty(self.lib.q4t_ep_dispatch_workspace_bytes(T_local, k, world), dtype=torch.uint8, device=dev)
        self.cap = cap_rows
        self.expert_ws_bytes = self.lib.q4t_moe_routed_workspace_bytes(cap_rows, 1, hs, layer_local.moe_is, layer_local.E)
        self.expert_ws = torch.empty(self.expert_ws_bytes, dtype=torch.uint8, device=dev)
        self.finish_ws_bytes = self.lib.q4t_moe_finish_workspace_bytes(T_local, hs, layer_local.shared_is)
        self.finish_ws = torch.empty(self.finish_ws_bytes, dtype=torch.uint8, device=dev)

    def _s(self):
        return self.C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def router(self, x):
        q = self.q4t
        q.check(self.lib.q4t_bf16_linear(x.data_ptr(), self.L.extra.gate, self.logits.data_ptr(), self.T, self.E, self.hs, self._s()))
        q.check(self.lib.q4t_router_topk(self.logits.data_ptr(), self.ids.data_ptr(), self.rw.data_ptr(), self.T, self.E, self.k, self._s()))
        return self.ids, self.rw

    def dispatch(self, x, ids):
        self.q4t.check(self.lib.q4t_ep_dispatch(x.data_ptr(), ids.data_ptr(), self.T, self.k, self.E, self.hs, self.world,
                                                self.send_rows.data_ptr(), self.send_local.data_ptr(),
                                                self.send_counts.data_ptr(), self.row_of_flat.data_ptr(),
                                                self.dispatch_ws.data_ptr(), self.dispatch_ws.numel(), self._s()))
        return self.send_rows, self.send_local, self.send_counts, self.row_of_flat

    def expert_rows(self, rows, local, out, n):
        self.q4t.check(self.lib.q4t_moe_expert_rows(rows.data_ptr(), local.data_ptr(), out.data_ptr(),
                                                    self.C.byref(self.L.routed), self.expert_ws.data_ptr(),
                                                    self.expert_ws_bytes, n, 0, self._s()))
        return out

    def finish(self, x, ret_rows, row_of_flat, rw, y):
        self.q4t.check(self.lib.q4t_moe_finish(x.data_ptr(), ret_rows.data_ptr(), row_of_flat.data_ptr(), rw.data_ptr(),
                                               self.C.byref(self.L.extra), y.data_ptr(), self.T, self.k,
                                               self.finish_ws.data_ptr(), self.finish_ws_bytes, self._s()))
        return y

    def empty_rows(self, n):
        return self.torch.empty((n, self.hs), dtype=self.torch.bfloat16, device=self.send_rows.device)


class ExpertParallelMoE:
    """Drives one expert-parallel layer step; `ops` supplies the arithmetic
    (LibraryOps on GPUs; the CPU tests plug in an oracle-backed twin)."""

    def __init__(self, ops, world: int, rank: int, group=None):
        import torch.distributed as dist
        self.ops, self.world, self.rank, self.group, self.dist = ops, world, rank, group, dist
        self.last = {}
        self.profile = False       # when set, forward() records CUDA events between its phases
        self.phase_ms = {}

    def exchange_counts(self, send_counts):
        """Row counts per destination -> row counts per source (host lists)."""
        import torch
        recv = torch.empty_like(send_counts)
        if self.world > 1:
            self.dist.all_to_all_single(recv, send_counts, group=self.group)
        else:
            recv.copy_(send_counts)
        return [int(v) for v in send_counts.tolist()], [int(v) for v in recv.tolist()]

    def all_to_all_rows(self, out, inp, out_splits, in_splits):
        if self.world > 1:
            self.dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits,
                                        group=self.group)
        else:
            out.copy_(inp)
        return out

    def _mark(self, marks, name):
        if self.profile:
            import torch
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

    def forward(self, x, y):
        ops = self.ops
        marks = []
        self._mark(marks, "start")
        ids, rw = ops.router(x)
        self._mark(marks, "router")
        send_rows, send_local, send_counts, row_of_flat = ops.dispatch(x, ids)
        self._mark(marks, "dispatch_build")
        s_counts, r_counts = self.exchange_counts(send_counts)      # host sync: split sizes
        self._mark(marks, "counts_exchange")
        n_send, n_recv = sum(s_counts), sum(r_counts)
        recv_rows = ops.empty_rows(n_recv)
        recv_local = send_local.new_empty((n_recv,))
        self.all_to_all_rows(recv_rows, send_rows[:n_send], r_counts, s_counts)
        self.all_to_all_rows(recv_local, send_local[:n_send], r_counts, s_counts)
        self._mark(marks, "dispatch_all_to_all")
        out_rows = ops.empty_rows(n_recv)
        ops.expert_rows(recv_rows, recv_local, out_rows, n_recv)
        self._mark(marks, "expert_rows")
        ret_rows = ops.empty_rows(max(n_send, 1))
        self.all_to_all_rows(ret_rows[:n_send], out_rows, s_counts, r_counts)
        self._mark(marks, "return_all_to_all")
        ops.finish(x, ret_rows, row_of_flat, rw, y)
        self._mark(marks, "finish")
        if self.profile:
            marks[-1][1].synchronize()
            self.phase_ms = {b[0]: a[1].elapsed_time(b[1]) for a, b in zip(marks[:-1], marks[1:])}
        self.last = dict(rows_sent=n_send, rows_received=n_recv, send_counts=s_counts, recv_counts=r_counts)
        return y


# ------------------------------------------------------------------ peer-memory path
def plan_placement(counts, world: int, hot: int):
    """Expert placement from per-expert row counts of a profiling batch.

    The `hot` most used experts are replicated on every rank (their rows never leave the GPU
    that owns the token, which also balances them perfectly); the others are dealt out one by
    one, busiest first, to the rank with the least load so far.  Returns (experts, tables):
    experts[r] = global ids served by rank r in local order, tables[r] = the int32 [E] table
    q4t_ep_peer_table.placement expects on rank r.  owner_table(tables) gives the table
    q4t_ep_peer_table.expert_owner expects (the same on every rank)."""
    import numpy as np
    counts = np.asarray(counts, dtype=np.int64)
    E = counts.shape[0]
    order = np.argsort(-counts, kind="stable")
    hot_ids = sorted(int(e) for e in order[:hot])
    experts = [[] for _ in range(world)]
    load = [0] * world
    for e in order[hot:]:
        r = min(range(world), key=lambda i: (load[i], len(experts[i]), i))
        experts[r].append(int(e))
        load[r] += int(counts[e])
    tables = []
    for r in range(world):
        # sharded experts first: their result rows are the ones that cross NVLink, and the
        # down GEMM walks the experts in local order, so those stores start early and
        # overlap with the replicated experts' tiles
        experts[r] = experts[r] + hot_ids
        t = np.full(E, -1, dtype=np.int32)
        for idx, e in enumerate(experts[r]):
            t[e] = idx | (1 << 30) if idx >= len(experts[r]) - len(hot_ids) else idx
        tables.append(t)
    return experts, tables


def owner_table(tables):
    """int32 [E]: the rank that serves expert e for every rank's tokens, or -1 for an expert
    replicated on all ranks (tables: plan_placement's second result)."""
    import numpy as np
    E = tables[0].shape[0]
    owner = np.full(E, -1, dtype=np.int32)
    for r, t in enumerate(tables):
        sharded = (t >= 0) & ((t >> 30) & 1 == 0)
        owner[sharded] = r
    return owner


def local_layer_from_list(q4t, full, experts):
    """The experts `experts` (global ids, local order) of a full device layer, copied."""
    import torch
    is_, hs, E = full.moe_is, full.hs, full.E
    pick = torch.as_tensor(experts, dtype=torch.long, device=full.t["gu_packed"].device)
    t = dict(full.t)
    t["gu_packed"] = full.t["gu_packed"].view(E, -1).index_select(0, pick).view(-1, hs // 2)
    t["gu_sf"] = full.t["gu_sf"].view(E, -1).index_select(0, pick).view(-1)
    t["dn_packed"] = full.t["dn_packed"].view(E, -1).index_select(0, pick).view(-1, is_ // 2)
    t["dn_sf"] = full.t["dn_sf"].view(E, -1).index_select(0, pick).view(-1)
    for n in ("gu_w_scale2", "gu_input_scale", "dn_w_scale2", "dn_input_scale"):
        t[n] = full.t[n].index_select(0, pick)
    return q4t.DeviceLayer(len(experts), hs, is_, full.shared_is, t, E_router=full.E_router)


class PeerBuffers:
    """One rank's peer-writable buffers (gathered quantised tokens of all ranks, landing rows
    of its own tokens) and its view of the peers' buffers.  Real ranks: allocated by the library and mapped across processes
    through exported handles (`connect`).  A single-process test can instead fill the
    table with plain device pointers (`from_pointers`)."""

    def __init__(self, q4t, world, rank, T_local, k, hs, expert_map=1, placement=None, expert_owner=None):
        """placement: this rank's device int32 [E] table (plan_placement) -> expert_map 2;
        expert_owner: device int32 [E] (owner_table), lets the publish step send a token only
        to the ranks that serve one of its experts."""
        self.q4t, self.lib = q4t, q4t.load()
        self.world, self.rank, self.T, self.k, self.hs = world, rank, T_local, k, hs
        self.table = q4t.EpPeerTable()
        self.table.world, self.table.rank = world, rank
        self.table.tokens_per_rank, self.table.expert_map = T_local, expert_map
        self.placement = placement          # keeps the device table alive
        if placement is not None:
            self.table.expert_map = 2
            self.table.placement = placement.data_ptr()
            self.table.experts_total = placement.numel()
        self.expert_owner = expert_owner    # keeps the device table alive
        if expert_owner is not None:
            self.table.expert_owner = expert_owner.data_ptr()
        # gathered codes, gathered scale blocks (all ranks' tokens), landing rows (own tokens),
        # and the sync buffer (flags + gathered ids) of the collective-free exchange
        self.sizes = (world * T_local * (hs // 2), world * T_local * (hs // 16), T_local * k * hs * 2,
                      self.lib.q4t_ep_sync_buffer_bytes(world, T_local, k))
        self.own = None
        self.opened = []

    def allocate(self):
        import ctypes as C
        own = []
        for nbytes in self.sizes:
            p = C.c_void_p()
            self.q4t.check(self.lib.q4t_peer_buffer_alloc(nbytes, C.byref(p)))
            own.append(p.value)
        self.own = own       # zero-filled by the library: the sync buffer's flags start at zero
        return self

    def handles(self):
        import ctypes as C
        out = []
        for p in self.own:
            h = C.create_string_buffer(self.q4t.PEER_HANDLE_BYTES)
            self.q4t.check(self.lib.q4t_peer_buffer_export(p, h))
            out.append(h.raw)
        return out

    def connect(self, all_handles):
        """all_handles[r] = rank r's three handles (e.g. from all_gather_object)."""
        import ctypes as C
        for r in range(self.world):
            ptrs = []
            for i in range(4):
                if r == self.rank:
                    ptrs.append(self.own[i])
                else:
                    p = C.c_void_p()
                    self.q4t.check(self.lib.q4t_peer_buffer_open(all_handles[r][i], C.byref(p)))
                    self.opened.append(p.value)
                    ptrs.append(p.value)
            self.table.xq_packed[r], self.table.xq_sf[r], self.table.dn_rows[r], self.table.sync[r] = ptrs
        return self

    def from_pointers(self, ptrs_by_rank):
        """ptrs_by_rank[r] = (codes, scales, landing rows[, sync]) of rank r; without sync
        buffers the driver uses the process group's collectives."""
        for r, ptrs in enumerate(ptrs_by_rank):
            self.table.xq_packed[r], self.table.xq_sf[r], self.table.dn_rows[r] = ptrs[:3]
            self.table.sync[r] = ptrs[3] if len(ptrs) > 3 else None
        self.own = list(ptrs_by_rank[self.rank])
        return self

    @property
    def has_sync(self):
        return self.own is not None and len(self.own) > 3 and bool(self.table.sync[self.rank])

    def close(self):
        for p in self.opened:
            self.lib.q4t_peer_buffer_close(p)
        self.opened = []


class _DeviceArray:
    """A device buffer owned by someone else, described through the CUDA array interface so that
    torch can view it without a copy."""

    def __init__(self, ptr, shape, typestr):
        self.__cuda_array_interface__ = dict(shape=tuple(shape), typestr=typestr, data=(int(ptr), False), version=2)


class PeerExpertParallelMoE:
    """Expert-parallel step without row collectives: each rank's quantiser stores its tokens
    into every rank's gathered buffer, and the down GEMM of an expert's owner stores the
    result rows straight into the token owners' landing buffers.  Only the expert ids travel
    through a collective (all-gather), which also orders "published" before "used"; one more
    tiny collective orders "pushed" before "combined".

    layer_local holds this rank's experts (expert_map 1: experts rank, rank+world, ...;
    0: a contiguous block) plus the replicated router and shared expert."""

    def __init__(self, q4t, layer_local, E_total, hs, k, world, rank, T_local, buffers: PeerBuffers,
                 group=None, device="cuda", exchange="auto"):
        """exchange: "flags" = ids and the two orderings travel by kernels over peer memory
        (q4t_ep_post_ids / q4t_ep_post_rows / q4t_ep_wait; needs the buffers' sync region),
        "collectives" = all-gather of the ids + a one-word all-reduce on the process group,
        "auto" = flags when the buffers have a sync region."""
        import ctypes as C
        import torch
        import torch.distributed as dist
        self.q4t, self.C, self.torch, self.dist = q4t, C, torch, dist
        self.lib = q4t.load()
        self.L, self.E, self.hs, self.k = layer_local, E_total, hs, k
        self.world, self.rank, self.T, self.group, self.buf = world, rank, T_local, group, buffers
        if not layer_local.routed.gu_input_scale_uniform > 0:
            raise q4t.Q4TError("the peer path needs one gate/up input scale for all experts")
        dev = device
        self.logits = torch.empty((T_local, E_total), dtype=torch.bfloat16, device=dev)
        self.ids = torch.empty((T_local, k), dtype=torch.int32, device=dev)
        self.rw = torch.empty((T_local, k), dtype=torch.float32, device=dev)
        self.ids_all = torch.empty((world * T_local, k), dtype=torch.int32, device=dev)
        self.row_of_flat = torch.empty((T_local * k,), dtype=torch.int32, device=dev)
        self.sync_word = torch.zeros((1,), dtype=torch.int32, device=dev)
        self.ws_bytes = self.lib.q4t_moe_expert_peer_workspace_bytes(world * T_local, k, hs, layer_local.moe_is,
                                                                     layer_local.E)
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=dev)
        self.finish_ws_bytes = self.lib.q4t_moe_finish_workspace_bytes(T_local, hs, layer_local.shared_is)
        self.finish_ws = torch.empty(self.finish_ws_bytes, dtype=torch.uint8, device=dev)
        self.profile = False
        self.phase_ms = {}
        self.flags = buffers.has_sync if exchange == "auto" else exchange == "flags"
        if self.flags and not buffers.has_sync:
            raise q4t.Q4TError("the flag exchange needs sync buffers in the peer table")
        self.epoch = 0
        if self.flags:
            # the gathered ids live in the sync buffer (peers store into it): a zero-copy view
            self.ids_all = torch.as_tensor(_DeviceArray(buffers.own[3] + q4t.EP_SYNC_IDS_OFFSET,
                                                        (world * T_local, k), "<i4"), device=dev)
        self._p_ids_all = self.ids_all.data_ptr()
        # argument values that never change, converted once
        self._extra, self._table = C.byref(layer_local.extra), C.byref(buffers.table)
        self._scale = float(layer_local.routed.gu_input_scale_uniform)
        self._p_logits, self._p_ids, self._p_rw = self.logits.data_ptr(), self.ids.data_ptr(), self.rw.data_ptr()
        self._p_fws, self._p_rof = self.finish_ws.data_ptr(), self.row_of_flat.data_ptr()

    def _s(self):
        return self.C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def _mark(self, marks, name):
        if self.profile:
            ev = self.torch.cuda.Event(enable_timing=True)
            ev.record()
            marks.append((name, ev))

    # the three device phases, separately callable so that a single-process test can
    # interleave several ranks (all publish, then all compute, then all finish)
    def publish(self, x):
        q, lib = self.q4t, self.lib
        q.check(lib.q4t_bf16_linear(x.data_ptr(), self.L.extra.gate, self.logits.data_ptr(), self.T, self.E, self.hs, self._s()))
        q.check(lib.q4t_router_topk(self.logits.data_ptr(), self.ids.data_ptr(), self.rw.data_ptr(), self.T, self.E, self.k, self._s()))
        q.check(lib.q4t_ep_publish(x.data_ptr(), self.C.byref(self.buf.table), self.hs,
                                   float(self.L.routed.gu_input_scale_uniform), self._s()))
        return self.ids

    def experts(self, ids_all):
        ids_all = ids_all if isinstance(ids_all, int) else ids_all.data_ptr()
        self.q4t.check(self.lib.q4t_moe_expert_peer(ids_all, self.C.byref(self.buf.table),
                                                    self.C.byref(self.L.routed), self.k, self.ws.data_ptr(),
                                                    self.ws_bytes, 0, self._s()))

    def shared(self, x):
        """The shared expert (needs nothing from the other ranks)."""
        self.q4t.check(self.lib.q4t_moe_shared_expert(x.data_ptr(), self.C.byref(self.L.extra), self.T,
                                                      self.finish_ws.data_ptr(), self.finish_ws_bytes, self._s()))

    def combine(self, x, y):
        q, lib = self.q4t, self.lib
        q.check(lib.q4t_ep_flat_rows(self.ids.data_ptr(), self.T * self.k, self.E, self.row_of_flat.data_ptr(), self._s()))
        q.check(lib.q4t_moe_combine(x.data_ptr(), self.buf.own[2], self.row_of_flat.data_ptr(), self.rw.data_ptr(),
                                    self.C.byref(self.L.extra), y.data_ptr(), self.T, self.k,
                                    self.finish_ws.data_ptr(), self.finish_ws_bytes, self._s()))
        return y

    def finish(self, x, y):
        self.shared(x)
        return self.combine(x, y)

    def route_publish(self, x):
        """publish() as one library call that also starts the shared expert on the library's
        side stream; pairs with combine_landed()."""
        self.q4t.check(self.lib.q4t_ep_route_publish(x.data_ptr(), self._extra, self._table, self.k, self._scale,
                                                     self._p_logits, self._p_ids, self._p_rw, self._p_fws,
                                                     self.finish_ws_bytes, self._s()))
        return self.ids

    def combine_landed(self, x, y):
        self.q4t.check(self.lib.q4t_ep_combine(x.data_ptr(), self.buf.own[2], self._p_ids, self._p_rw, self._extra,
                                               y.data_ptr(), self.T, self.k, self._p_rof, self._p_fws,
                                               self.finish_ws_bytes, self._s()))
        return y

    def sync_status(self):
        """Raises if a wait for another rank ran out (flag exchange only; synchronises first)."""
        if self.flags:
            self.torch.cuda.synchronize()
            self.q4t.check(self.lib.q4t_ep_sync_status(self._table))

    def forward(self, x, y):
        """One step.  Flag exchange: seven library calls, no collective; otherwise three library
        calls and two collectives (host time per step matters once the per-rank GPU work drops
        to a few hundred microseconds)."""
        marks = []
        self._mark(marks, "start")
        self.route_publish(x)
        self._mark(marks, "publish")
        if self.flags:
            # ids to every rank's sync buffer + "published" flag; wait for all ranks' flags
            self.epoch += 1
            q, lib, st = self.q4t, self.lib, self._s()
            q.check(lib.q4t_ep_post_ids(self._p_ids, self._table, self.k, self.epoch, st))
            q.check(lib.q4t_ep_wait(self._table, 0, self.epoch, st))
            self._mark(marks, "ids_all_gather")
            self.experts(self._p_ids_all)
            self._mark(marks, "experts_pull_push")
            q.check(lib.q4t_ep_post_rows(self._table, self.epoch, st))
            q.check(lib.q4t_ep_wait(self._table, 1, self.epoch, st))
            self._mark(marks, "landed_barrier")
        else:
            if self.world > 1:
                self.dist.all_gather_into_tensor(self.ids_all, self.ids, group=self.group)
            else:
                self.ids_all.copy_(self.ids)
            self._mark(marks, "ids_all_gather")
            self.experts(self.ids_all)
            self._mark(marks, "experts_pull_push")
            if self.world > 1:      # every rank's rows have landed once this returns on the stream
                self.dist.all_reduce(self.sync_word, group=self.group)
            self._mark(marks, "landed_barrier")
        self.combine_landed(x, y)
        self._mark(marks, "combine")
        if self.profile:
            marks[-1][1].synchronize()
            self.phase_ms = {b[0]: a[1].elapsed_time(b[1]) for a, b in zip(marks[:-1], marks[1:])}
        return y
