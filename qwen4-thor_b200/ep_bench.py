"""bench.py's multi-GPU arm: the expert-parallel prefill layer.

T = 32768 tokens per step sharded contiguously over the ranks, hidden 2048, 512 experts,
top-10, intermediate 512, shared expert 512, Zipf(s=1.1) expert popularity (the popularity
rank is a seeded permutation of the experts).  One process per GPU under torchrun.

Default exchange ("peer"): no row collectives.  After routing, each rank's quantiser stores a
token's NVFP4 codes into the gathered buffer of exactly the ranks that serve one of its
experts (peer stores over NVLink); the int32 expert ids are all-gathered with NCCL; every
rank runs its experts and the down GEMM's epilogue stores each result row straight into the
token owner's landing buffer; one tiny all-reduce says "all rows have landed"; the owner
combines.  Placement: the --hot-experts most used experts of a profiling batch (a batch that
is not one of the timed inputs) are replicated on every GPU, the rest dealt out by load; the
line also carries the time of plain contiguous sharding (512/N experts per GPU, nothing
replicated: the placement the benchmark configuration names) as `plain_sharding`.
--exchange rows is the all-to-all of bf16 rows over NCCL with contiguous blocks.
"""
from __future__ import annotations

import importlib
import json
import os
import sys

HS, E, K_TOP, MOE_IS, SHARED_IS = 2048, 512, 10, 512, 512
T_TOTAL = 32768


def _local_layer(q4t, full, lo, hi):
    """View of experts [lo, hi) of a full device layer (no copies)."""
    is_, hs = full.moe_is, full.hs
    gb = q4t.load().q4t_sf_buffer_size(2 * is_, hs)
    db = q4t.load().q4t_sf_buffer_size(hs, is_)
    t = dict(full.t)
    t["gu_packed"] = full.t["gu_packed"][lo * 2 * is_:hi * 2 * is_]
    t["gu_sf"] = full.t["gu_sf"][lo * gb:hi * gb]
    t["dn_packed"] = full.t["dn_packed"][lo * hs:hi * hs]
    t["dn_sf"] = full.t["dn_sf"][lo * db:hi * db]
    for n in ("gu_w_scale2", "gu_input_scale", "dn_w_scale2", "dn_input_scale"):
        t[n] = full.t[n][lo:hi]
    return q4t.DeviceLayer(hi - lo, hs, is_, full.shared_is, t, E_router=full.E_router)


def _local_layer_interleaved(q4t, full, rank, world):
    """Experts rank, rank+world, rank+2*world, ... of a full device layer (copied)."""
    is_, hs, E = full.moe_is, full.hs, full.E
    t = dict(full.t)
    pick = slice(rank, E, world)
    t["gu_packed"] = full.t["gu_packed"].view(E, -1)[pick].contiguous().view(-1, hs // 2)
    t["gu_sf"] = full.t["gu_sf"].view(E, -1)[pick].contiguous().view(-1)
    t["dn_packed"] = full.t["dn_packed"].view(E, -1)[pick].contiguous().view(-1, is_ // 2)
    t["dn_sf"] = full.t["dn_sf"].view(E, -1)[pick].contiguous().view(-1)
    for n in ("gu_w_scale2", "gu_input_scale", "dn_w_scale2", "dn_input_scale"):
        t[n] = full.t[n][pick].contiguous()
    return q4t.DeviceLayer(E // world, hs, is_, full.shared_is, t, E_router=full.E_router)


def main_multi(args):
    import torch
    import torch.distributed as dist
    bench = importlib.import_module("bench")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if args.impl == "reference":
        # the CPU formulation runs on rank 0 only; the other ranks have nothing to do
        if rank == 0:
            bench.main_single(args)
        return
    # NCCL's version banner goes to stdout, and the bench prints exactly one line there:
    # until the result line, whatever is written to descriptor 1 lands on stderr instead
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    q4t = importlib.import_module("qwen4-thor_b200")
    syn = importlib.import_module("qwen4-thor_b200.synthetic")
    ep = importlib.import_module("qwen4-thor_b200.ep")
    q4t.load()
    peaks = bench.load_peaks()

    T_loc = T_TOTAL // world
    per = E // world
    peer_mode = args.exchange == "peer"
    full = syn.device_layer(q4t, E, HS, MOE_IS, SHARED_IS, seed=20260921 + 4000, zipf_s=1.1)
    xs = [syn.make_x(T_loc, HS, seed=400 + 10 * i + rank, bias_column=True) for i in range(2)]
    y = torch.empty((T_loc, HS), dtype=torch.bfloat16, device="cuda")
    # row-exchange path (NCCL all-to-all both ways), contiguous expert blocks
    local = _local_layer(q4t, full, rank * per, (rank + 1) * per)
    ops = ep.LibraryOps(q4t, local, E, HS, K_TOP, world, T_loc, cap_rows=T_TOTAL * K_TOP)
    drv_rows = ep.ExpertParallelMoE(ops, world, rank)
    drv = drv_rows
    placement = None
    drv_plain = None
    equals_single = None
    exchange_note = None
    if peer_mode:
        def connect(buf):
            gathered = [None] * world
            dist.all_gather_object(gathered, buf.handles())
            buf.connect(gathered)
            return buf

        # Placement from a profiling batch that is NOT one of the timed inputs: the most used
        # experts are replicated on every rank, the others dealt out by load (hot_experts 0:
        # plain interleaving e % N instead).
        owner = None
        if args.hot_experts > 0:
            x_prof = syn.make_x(T_loc, HS, seed=7000 + rank, bias_column=True)
            ops.router(x_prof)
            counts = torch.bincount(ops.ids.flatten().long(), minlength=E)
            dist.all_reduce(counts)
            experts, tables = ep.plan_placement(counts.cpu().numpy(), world, args.hot_experts)
            local_i = ep.local_layer_from_list(q4t, full, experts[rank])
            placement = torch.from_numpy(tables[rank]).cuda()
            owner = torch.from_numpy(ep.owner_table(tables)).cuda()
            del x_prof
        else:
            local_i = _local_layer_interleaved(q4t, full, rank, world)
        buf = connect(ep.PeerBuffers(q4t, world, rank, T_loc, K_TOP, HS, expert_map=1, placement=placement,
                                     expert_owner=owner).allocate())
        drv = ep.PeerExpertParallelMoE(q4t, local_i, E, HS, K_TOP, world, rank, T_loc, buf)
        # the same step with the ids and the two orderings on NCCL collectives, for comparison
        drv_coll = None if args.quick else ep.PeerExpertParallelMoE(q4t, local_i, E, HS, K_TOP, world, rank, T_loc, buf,
                                                                   exchange="collectives")
        if not args.quick and args.hot_experts > 0:
            # the benchmark configuration's own placement: contiguous blocks of 512/N experts
            buf_p = connect(ep.PeerBuffers(q4t, world, rank, T_loc, K_TOP, HS, expert_map=0).allocate())
            drv_plain = ep.PeerExpertParallelMoE(q4t, local, E, HS, K_TOP, world, rank, T_loc, buf_p)
        # both paths must give the same bits
        y2 = torch.empty_like(y)
        drv_rows.forward(xs[0], y2)

        def agrees(d):
            ok = 1
            try:
                d.forward(xs[0], y)
                d.sync_status()
            except q4t.Q4TError:
                ok = 0
            torch.cuda.synchronize()
            same = torch.tensor([ok * int(torch.equal(y.view(torch.int16), y2.view(torch.int16)))], device="cuda")
            dist.all_reduce(same, op=dist.ReduceOp.MIN)
            return int(same.item()) == 1

        exchange_note = None
        if not agrees(drv):
            if not drv.flags:
                raise RuntimeError("peer path and row-exchange path disagree")
            # the flag exchange failed its check on this machine: keep the run alive on the
            # process group's collectives and say so in the line
            exchange_note = "flag exchange failed its check (time-out or mismatch); ids and orderings on NCCL collectives"
            drv = ep.PeerExpertParallelMoE(q4t, local_i, E, HS, K_TOP, world, rank, T_loc, buf, exchange="collectives")
            if drv_plain is not None:
                drv_plain = ep.PeerExpertParallelMoE(q4t, local, E, HS, K_TOP, world, rank, T_loc, buf_p,
                                                     exchange="collectives")
            if not agrees(drv):
                raise RuntimeError("peer path and row-exchange path disagree")
        # and the same bits as the unsharded layer: every rank runs its own tokens through the
        # whole layer on its GPU alone
        fwd1 = q4t.MoEForward(full, T_loc, K_TOP)
        fwd1(xs[0], y2)
        torch.cuda.synchronize()
        same1 = torch.tensor([int(torch.equal(y.view(torch.int16), y2.view(torch.int16)))], device="cuda")
        dist.all_reduce(same1, op=dist.ReduceOp.MIN)
        equals_single = bool(int(same1.item()))
        del y2, fwd1
        if args.quick:
            del drv_rows, ops
            torch.cuda.empty_cache()

    def step(i):
        drv.forward(xs[i % 2], y)

    def barrier():
        dist.barrier()

    with bench.ClockSampler(local_rank) as clocks:
        ms = bench.time_steps(torch, step, args.steps, args.warmup, barrier)
    t = torch.tensor([ms], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    coll = None
    if peer_mode and drv_coll is not None:
        ms_c = bench.time_steps(torch, lambda i: drv_coll.forward(xs[i % 2], y), max(3, min(args.steps, 10)), 3, barrier)
        t = torch.tensor([ms_c], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        coll = dict(ms_per_step=float(t.item()), tokens_per_s=T_TOTAL / (float(t.item()) * 1e-3),
                    exchange="ids by NCCL all-gather, 'rows landed' by a one-word NCCL all-reduce")
    if peer_mode:
        drv.sync_status()
    plain = None
    if drv_plain is not None:
        y_p = torch.empty_like(y)
        drv_plain.forward(xs[0], y_p)
        drv.forward(xs[0], y)
        torch.cuda.synchronize()
        same = torch.tensor([int(torch.equal(y.view(torch.int16), y_p.view(torch.int16)))], device="cuda")
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        ms_p = bench.time_steps(torch, lambda i: drv_plain.forward(xs[i % 2], y_p), max(3, min(args.steps, 10)), 3, barrier)
        t = torch.tensor([ms_p], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        plain = dict(ms_per_step=float(t.item()), tokens_per_s=T_TOTAL / (float(t.item()) * 1e-3),
                     placement=f"contiguous blocks of {per} experts per GPU, nothing replicated",
                     equals_replicated_placement_bits=bool(int(same.item())))
        del y_p

    # End to end: every step copies its input from pinned host memory and its result back.
    # The copies run on their own streams with two buffers each way, so the input of step i+1
    # and the result of step i-1 move while step i computes; the timed region ends only when
    # the last result has reached the host.
    hx = [x.cpu().pin_memory() for x in xs]
    hy = [torch.empty((T_loc, HS), dtype=torch.bfloat16).pin_memory() for _ in range(2)]
    dx = [torch.empty((T_loc, HS), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    dy = [torch.empty((T_loc, HS), dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    main_s, s_in, s_out = torch.cuda.current_stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_done = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    for ev in ev_done + ev_out:
        ev.record(main_s)

    def step_e2e(i):
        b = i & 1
        s_in.wait_event(ev_done[b])            # the step that last read dx[b] is over
        with torch.cuda.stream(s_in):
            dx[b].copy_(hx[i % 2], non_blocking=True)
            ev_in[b].record(s_in)
        main_s.wait_event(ev_in[b])
        main_s.wait_event(ev_out[b])           # dy[b] has been copied out
        drv.forward(dx[b], dy[b])
        ev_done[b].record(main_s)
        s_out.wait_event(ev_done[b])
        with torch.cuda.stream(s_out):
            hy[b].copy_(dy[b], non_blocking=True)
            ev_out[b].record(s_out)

    def drain():
        main_s.wait_event(ev_out[0])
        main_s.wait_event(ev_out[1])

    ms_e = bench.time_steps(torch, step_e2e, args.steps, args.warmup, barrier, finish=drain)
    t = torch.tensor([ms_e], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e = float(t.item())

    # phase breakdown of one more step on this rank (events between phases)
    drv.profile = True
    step(0)
    phases = dict(drv.phase_ms)
    drv.profile = False

    # stage times inside the expert phase, every rank (the slowest rank sets the step time)
    stage_all = None
    if peer_mode:
        q4t.stage_timing(True)
        drv.experts(drv.ids_all)
        st = q4t.stage_timing_read()
        q4t.stage_timing(False)
        mine = {n: round(v, 4) for n, v in st.items() if v > 0}
        stage_all = [None] * world
        dist.all_gather_object(stage_all, mine)
        dist.barrier()

    # per-rank load and link traffic of the last step
    if peer_mode:
        src_rank = torch.arange(world * T_loc, device="cuda").div(T_loc, rounding_mode="floor")[:, None].expand_as(drv.ids_all)
        if placement is not None:
            v = placement[drv.ids_all.long()]
            mine = (v >= 0) & (((v >> 30) & 1 == 0) | (src_rank == rank))
        else:
            mine = drv.ids_all.remainder(world) == rank
        rows_here = int(mine.sum().item())
        remote_rows = int((mine & (src_rank != rank)).sum().item())
        rows_recv = torch.tensor([float(rows_here)], device="cuda", dtype=torch.float64)
        # leaving this GPU: result rows pushed to other ranks (plus its token block to every peer)
        out_bytes = torch.tensor([remote_rows * HS * 2.0 + (world - 1) * T_loc * (HS // 2 + HS // 16)],
                                 device="cuda", dtype=torch.float64)
    else:
        rows_recv = torch.tensor([drv.last["rows_received"]], device="cuda", dtype=torch.float64)
        remote_out = sum(c for r, c in enumerate(drv.last["send_counts"]) if r != rank) + \
            sum(c for r, c in enumerate(drv.last["recv_counts"]) if r != rank)
        out_bytes = torch.tensor([remote_out * HS * 2.0], device="cuda", dtype=torch.float64)
    mx_rows, mx_bytes = rows_recv.clone(), out_bytes.clone()
    dist.all_reduce(mx_rows, op=dist.ReduceOp.MAX)
    dist.all_reduce(mx_bytes, op=dist.ReduceOp.MAX)

    # the same workload on one GPU (rank 0 holds all weights): lets a reader
    # derive strong-scaling efficiency from this one line
    n1 = None
    if rank == 0 and not args.quick:
        x_full = syn.make_x(T_TOTAL, HS, seed=999, bias_column=True)
        fwd = q4t.MoEForward(full, T_TOTAL, K_TOP)
        y_full = torch.empty((T_TOTAL, HS), dtype=torch.bfloat16, device="cuda")
        ms1 = bench.time_steps(torch, lambda i: fwd(x_full, y_full), 3, 2)
        n1 = dict(ms_per_step=ms1, tokens_per_s=T_TOTAL / (ms1 * 1e-3))
        del fwd, x_full, y_full
    dist.barrier()

    if rank == 0:
        flops_max = 6.0 * float(mx_rows.item()) * HS * MOE_IS
        t_comm = float(mx_bytes.item()) / 770e9
        t_flop = flops_max / (4 * peaks["bf16_tflops"] * 1e12)
        target = max(t_comm, t_flop)
        if plain is not None and n1 is not None:
            plain["strong_scaling_efficiency"] = n1["ms_per_step"] / (world * plain["ms_per_step"])
        line = dict(metric="moe_ep_prefill_tokens_per_s", value=T_TOTAL / (ms * 1e-3), unit="tokens/s", n_gpus=world,
                    steps=args.steps, warmup=args.warmup, ms_per_step=ms, higher_is_better=True, scaling="strong",
                    vs_baseline=None, dtype="nvfp4 (e2m1 x ue4m3, fp32 accumulate); bf16 router and shared expert",
                    data="synthetic",
                    config=dict(workload=f"expert-parallel prefill MoE layer, T={T_TOTAL} total over {world} GPUs",
                                expert_map=(f"{args.hot_experts} most used experts of a profiling batch replicated on every GPU, "
                                            "the rest dealt out by load" if placement is not None else
                                            "interleaved (e % N)" if peer_mode else "contiguous blocks"),
                                experts_on_rank0=local_i.E if peer_mode else per,
                                hidden=HS, experts=E, top_k=K_TOP, moe_intermediate=MOE_IS, shared_intermediate=SHARED_IS,
                                routing="zipf(s=1.1) bias on router column 0", parallelism=f"ep{world}",
                                l2="2 inputs alternated; one step moves > 1 GB per GPU",
                                exchange=("quantised tokens stored by the quantiser into the gathered buffers of the GPUs that "
                                          "serve one of their experts, bf16 result "
                                          "rows stored into the token owner's buffer by the down GEMM's epilogue (peer memory "
                                          "over NVLink); expert ids and the two orderings of a step by flag kernels over peer memory, no collective call; "
                                          "checked bit-identical to the row-exchange path") if peer_mode else
                                "bf16 rows both ways, NCCL all_to_all_single, one host sync per step for the split sizes"),
                    clocks=clocks.summary(),
                    e2e=dict(value=T_TOTAL / (ms_e * 1e-3), unit="tokens/s", h2d_bytes_per_step=T_TOTAL * HS * 2,
                             d2h_bytes_per_step=T_TOTAL * HS * 2),
                    # peer path: router logits, top-k, selective publish, [ids + flag, wait], id localise, 3 planning
                    # kernels, code gather, 2 expert GEMMs, [flag, wait], flat rows, combine, 2 shared-expert GEMMs
                    gpu_launches=((19 if drv.flags else 15) if peer_mode else 19) * args.steps * world,
                    roofline=dict(bound="nvlink", achieved=float(mx_bytes.item()) / (ms * 1e-3) / 1e9, peak=770.0,
                                  unit="GB/s", frac=target / (ms * 1e-3), traffic=None,
                                  note="frac = max(link time at 770 GB/s per direction, routed flops at 4x measured bf16) / step time; "
                                       "achieved = bytes leaving the busiest GPU per second"),
                    cpu_baseline=None,
                    load=dict(rows_received_max=float(mx_rows.item()), rows_received_mean=T_TOTAL * K_TOP / world,
                              imbalance=float(mx_rows.item()) / (T_TOTAL * K_TOP / world)),
                    phase_ms_rank0=phases, expert_stage_ms_by_rank=stage_all, single_gpu_same_workload=n1,
                    strong_scaling_efficiency=(n1["ms_per_step"] / (world * ms)) if n1 else None,
                    plain_sharding=plain, equals_single_gpu_bits=equals_single, collectives_exchange=coll,
                    exchange_note=exchange_note,
                    note="N = 1 of this metric is `also.ep_prefill_T32768_single_gpu` of the single-GPU line "
                         "(whose headline metric is the decode-shaped layer, another workload)")
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        print(json.dumps(line), flush=True)
        os.dup2(2, 1)
    dist.destroy_process_group()
