"""GPU parity of the expert-parallel entry points: the EP driver on one rank,
and two ranks emulated inside one process (the all-to-all done by slicing),
must reproduce q4t_moe_forward bit for bit.  A real 2-GPU NCCL run is covered
when two devices are visible."""
import importlib
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import synth
from gpu_util import dev, host

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _slice_layer(q4t, full, lo, hi):
    return importlib.import_module("qwen4-thor_b200.ep_bench")._local_layer(q4t, full, lo, hi)


@pytest.mark.parametrize("T", [4, 40, 300])
def test_ep_one_rank_equals_forward(q4t, gpu_lib, T):
    ep = importlib.import_module("qwen4-thor_b200.ep")
    E, hs, is_, sis, k = 32, 512, 256, 128, 4
    L = synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=61, per_expert_input_scale=True)
    dl = q4t.DeviceLayer.from_host(L)
    x = dev(synth.make_x(T, hs, seed=T)).view(torch.bfloat16)
    y_ref = torch.empty((T, hs), dtype=torch.bfloat16, device="cuda")
    fwd = q4t.MoEForward(dl, T, k)
    fwd(x, y_ref)
    fwd.status()
    ops = ep.LibraryOps(q4t, dl, E, hs, k, 1, T, cap_rows=T * k)
    y = torch.empty_like(y_ref)
    ep.ExpertParallelMoE(ops, 1, 0).forward(x, y)
    torch.cuda.synchronize()
    assert torch.equal(y.view(torch.int16), y_ref.view(torch.int16))


def test_ep_two_emulated_ranks_equal_forward(q4t, gpu_lib):
    """Two ranks' steps interleaved by hand on one GPU; the exchange is tensor slicing."""
    ep = importlib.import_module("qwen4-thor_b200.ep")
    E, hs, is_, sis, k, T, W = 16, 512, 128, 128, 3, 64, 2
    L = synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=62)
    full = q4t.DeviceLayer.from_host(L)
    x = dev(synth.make_x(T, hs, seed=9)).view(torch.bfloat16)
    y_ref = torch.empty((T, hs), dtype=torch.bfloat16, device="cuda")
    q4t.MoEForward(full, T, k)(x, y_ref)
    Tl, per = T // W, E // W
    ops = [ep.LibraryOps(q4t, _slice_layer(q4t, full, r * per, (r + 1) * per), E, hs, k, W, Tl, cap_rows=T * k)
           for r in range(W)]
    xs = [x[r * Tl:(r + 1) * Tl].contiguous() for r in range(W)]
    routed = [o.router(xr) for o, xr in zip(ops, xs)]
    disp = []
    for o, xr, (ids, rw) in zip(ops, xs, routed):
        rows, local, counts, rof = o.dispatch(xr, ids)
        disp.append((rows.clone(), local.clone(), counts.cpu().tolist(), rof.clone(), rw.clone()))
    offs = [np.concatenate([[0], np.cumsum(d[2])]) for d in disp]
    ret = [torch.empty((Tl * k, hs), dtype=torch.bfloat16, device="cuda") for _ in range(W)]
    for dst in range(W):   # rank dst receives its slice from every source, computes, sends back
        parts = [(src, int(offs[src][dst]), int(offs[src][dst + 1])) for src in range(W)]
        rows = torch.cat([disp[s][0][a:b] for s, a, b in parts])
        local = torch.cat([disp[s][1][a:b] for s, a, b in parts])
        out = torch.empty_like(rows)
        ops[dst].expert_rows(rows, local, out, rows.shape[0])
        pos = 0
        for s, a, b in parts:
            ret[s][a:b] = out[pos:pos + (b - a)]
            pos += b - a
    ys = []
    for r in range(W):
        y = torch.empty((Tl, hs), dtype=torch.bfloat16, device="cuda")
        ops[r].finish(xs[r], ret[r], disp[r][3], disp[r][4], y)
        ys.append(y)
    torch.cuda.synchronize()
    assert torch.equal(torch.cat(ys).view(torch.int16), y_ref.view(torch.int16))


@pytest.mark.parametrize("W,expert_map", [(2, 0), (2, 1), (4, 1), (2, 2), (4, 2)])
def test_peer_path_emulated_ranks_equal_forward(q4t, gpu_lib, W, expert_map):
    """The pull/push path with W ranks living in one process on one GPU: the "peer"
    pointers are ordinary device pointers and the ranks' phases are run one after the
    other (all publish, all compute, all finish), so no kernel waits on another."""
    ep = importlib.import_module("qwen4-thor_b200.ep")
    epb = importlib.import_module("qwen4-thor_b200.ep_bench")
    E, hs, is_, sis, k, T = 16, 512, 128, 128, 3, 400
    L = synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=63)
    full = q4t.DeviceLayer.from_host(L)
    assert full.routed.gu_input_scale_uniform > 0
    x = dev(synth.make_x(T, hs, seed=11)).view(torch.bfloat16)
    y_ref = torch.empty((T, hs), dtype=torch.bfloat16, device="cuda")
    fwd = q4t.MoEForward(full, T, k)
    fwd(x, y_ref)
    fwd.status()
    Tl, per = T // W, E // W
    sf_bytes = Tl * (hs // 16)
    sync_bytes = q4t.load().q4t_ep_sync_buffer_bytes(W, Tl, k)
    pub = [(torch.empty((W * Tl, hs // 2), dtype=torch.uint8, device="cuda"),
            torch.zeros(W * sf_bytes, dtype=torch.uint8, device="cuda"),
            torch.full((Tl * k, hs), -1, dtype=torch.int16, device="cuda"),
            torch.zeros(sync_bytes, dtype=torch.uint8, device="cuda")) for _ in range(W)]
    ptrs = [tuple(t.data_ptr() for t in p) for p in pub]
    drv = []
    if expert_map == 2:   # placement table: 3 experts replicated everywhere, the rest by load
        ids_ref = fwd.region("expert_ids", torch.int32, T * k).cpu().numpy()
        experts, tables = ep.plan_placement(np.bincount(ids_ref, minlength=E), W, hot=3)
        assert sorted(e for lst in experts for e in lst[:-3]) == sorted(set(range(E)) - set(experts[0][-3:]))
    for r in range(W):
        placement = owner = None
        if expert_map == 2:
            local = ep.local_layer_from_list(q4t, full, experts[r])
            placement = torch.from_numpy(tables[r]).cuda()
            owner = torch.from_numpy(ep.owner_table(tables)).cuda()
        elif expert_map == 1:
            local = epb._local_layer_interleaved(q4t, full, r, W)
        else:
            local = _slice_layer(q4t, full, r * per, (r + 1) * per)
        buf = ep.PeerBuffers(q4t, W, r, Tl, k, hs, expert_map=expert_map, placement=placement,
                             expert_owner=owner).from_pointers(ptrs)
        drv.append(ep.PeerExpertParallelMoE(q4t, local, E, hs, k, W, r, Tl, buf))
    xs = [x[r * Tl:(r + 1) * Tl].contiguous() for r in range(W)]
    # first step: the separate entry points; second step below: the two single-call entries
    ids_all = torch.cat([d.publish(xr) for d, xr in zip(drv, xs)])
    for d in drv:
        d.experts(ids_all)
    ys = [d.finish(xr, torch.empty((Tl, hs), dtype=torch.bfloat16, device="cuda")) for d, xr in zip(drv, xs)]
    torch.cuda.synchronize()
    for d in drv:
        q4t.check(q4t.load().q4t_moe_workspace_status(d.ws.data_ptr(), W * Tl, k, hs, is_, d.L.E))
    assert torch.equal(torch.cat(ys).view(torch.int16), y_ref.view(torch.int16))
    # a second step over the same buffers (stale rows from step one must not leak); this one
    # publishes selectively: a token is stored only on the ranks that serve one of its experts
    for p in pub:
        p[0].fill_(0xEE)     # whatever is not published this step must not be read either
    x2 = dev(synth.make_x(T, hs, seed=12)).view(torch.bfloat16)
    fwd(x2, y_ref)
    xs = [x2[r * Tl:(r + 1) * Tl].contiguous() for r in range(W)]
    ids_all = torch.cat([d.route_publish(xr) for d, xr in zip(drv, xs)])
    for d in drv:
        d.experts(ids_all)
    ys = [d.combine_landed(xr, torch.empty((Tl, hs), dtype=torch.bfloat16, device="cuda")) for d, xr in zip(drv, xs)]
    torch.cuda.synchronize()
    assert torch.equal(torch.cat(ys).view(torch.int16), y_ref.view(torch.int16))
    # a third step without any collective: the ids travel into every rank's sync buffer and the
    # two orderings are flags (every rank posts before any rank waits, so nothing waits here)
    lib = q4t.load()
    x3 = dev(synth.make_x(T, hs, seed=13)).view(torch.bfloat16)
    fwd(x3, y_ref)
    xs = [x3[r * Tl:(r + 1) * Tl].contiguous() for r in range(W)]
    st = q4t.C.c_void_p(torch.cuda.current_stream().cuda_stream)
    tabs = [q4t.C.byref(d.buf.table) for d in drv]
    for d, xr, tab in zip(drv, xs, tabs):
        d.route_publish(xr)
        q4t.check(lib.q4t_ep_post_ids(d.ids.data_ptr(), tab, k, 7, st))
    for d, tab, p in zip(drv, tabs, pub):
        q4t.check(lib.q4t_ep_wait(tab, 0, 7, st))
        d.experts(p[3].data_ptr() + q4t.EP_SYNC_IDS_OFFSET)
        q4t.check(lib.q4t_ep_post_rows(tab, 7, st))
    ys = []
    for d, xr, tab in zip(drv, xs, tabs):
        q4t.check(lib.q4t_ep_wait(tab, 1, 7, st))
        ys.append(d.combine_landed(xr, torch.empty((Tl, hs), dtype=torch.bfloat16, device="cuda")))
    torch.cuda.synchronize()
    for tab in tabs:
        q4t.check(lib.q4t_ep_sync_status(tab))
    assert torch.equal(torch.cat(ys).view(torch.int16), y_ref.view(torch.int16))
    gathered = pub[0][3][q4t.EP_SYNC_IDS_OFFSET:q4t.EP_SYNC_IDS_OFFSET + T * k * 4].view(torch.int32)
    assert torch.equal(gathered, torch.cat([d.ids.flatten() for d in drv]))


def test_wait_for_a_rank_that_never_posts_gives_up(q4t, gpu_lib):
    """A rank that never posts (it died between steps) must not hang the others: the wait is
    bounded (about two seconds), raises the sync buffer's status word and returns; the context
    stays usable.  The failure is made on the host side: nothing ever raises the flag."""
    ep = importlib.import_module("qwen4-thor_b200.ep")
    W, Tl, k, hs = 2, 8, 2, 256
    lib = q4t.load()
    pub = [(torch.empty((W * Tl, hs // 2), dtype=torch.uint8, device="cuda"),
            torch.zeros(W * Tl * (hs // 16), dtype=torch.uint8, device="cuda"),
            torch.zeros((Tl * k, hs), dtype=torch.int16, device="cuda"),
            torch.zeros(lib.q4t_ep_sync_buffer_bytes(W, Tl, k), dtype=torch.uint8, device="cuda")) for _ in range(W)]
    buf = ep.PeerBuffers(q4t, W, 0, Tl, k, hs, expert_map=0).from_pointers([tuple(t.data_ptr() for t in p) for p in pub])
    tab = q4t.C.byref(buf.table)
    st = q4t.C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ids = torch.zeros((Tl, k), dtype=torch.int32, device="cuda")
    q4t.check(lib.q4t_ep_post_ids(ids.data_ptr(), tab, k, 1, st))      # rank 0 posts, rank 1 never does
    q4t.check(lib.q4t_ep_wait(tab, 0, 1, st))
    torch.cuda.synchronize()
    assert lib.q4t_ep_sync_status(tab) != 0
    assert b"ran out" in lib.q4t_last_error()
    # the device is still usable
    assert int((torch.arange(10, device="cuda") * 2).sum().item()) == 90


def test_peer_path_forward_one_rank(q4t, gpu_lib):
    """The driver's own step (route+publish and combine as single library calls, shared expert
    on the library's side stream) on one rank, twice, against MoEForward."""
    ep = importlib.import_module("qwen4-thor_b200.ep")
    E, hs, is_, sis, k, T = 32, 1024, 256, 256, 5, 130
    L = synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=65)
    full = q4t.DeviceLayer.from_host(L)
    pub = (torch.empty((T, hs // 2), dtype=torch.uint8, device="cuda"),
           torch.zeros(T * (hs // 16), dtype=torch.uint8, device="cuda"),
           torch.full((T * k, hs), -1, dtype=torch.int16, device="cuda"),
           torch.zeros(q4t.load().q4t_ep_sync_buffer_bytes(1, T, k), dtype=torch.uint8, device="cuda"))
    buf = ep.PeerBuffers(q4t, 1, 0, T, k, hs, expert_map=0).from_pointers([tuple(t.data_ptr() for t in pub)])
    drv = ep.PeerExpertParallelMoE(q4t, full, E, hs, k, 1, 0, T, buf)
    assert drv.flags       # ids and orderings through the sync buffer, no collective
    fwd = q4t.MoEForward(full, T, k)
    for seed in (21, 22):
        x = dev(synth.make_x(T, hs, seed=seed)).view(torch.bfloat16)
        y_ref = torch.empty((T, hs), dtype=torch.bfloat16, device="cuda")
        y = torch.empty_like(y_ref)
        fwd(x, y_ref)
        drv.forward(x, y)
        torch.cuda.synchronize()
        assert torch.equal(y.view(torch.int16), y_ref.view(torch.int16))


def test_peer_path_rejects_per_expert_input_scales(q4t, gpu_lib):
    L = synth.make_layer(E=8, hs=256, moe_is=128, shared_is=128, seed=64, per_expert_input_scale=True)
    dl = q4t.DeviceLayer.from_host(L)
    table = q4t.EpPeerTable()
    table.world, table.rank, table.tokens_per_rank = 1, 0, 8
    ids = torch.zeros((8, 2), dtype=torch.int32, device="cuda")
    ws = torch.empty(1 << 20, dtype=torch.uint8, device="cuda")
    rc = q4t.load().q4t_moe_expert_peer(ids.data_ptr(), q4t.C.byref(table), q4t.C.byref(dl.routed), 2,
                                        ws.data_ptr(), ws.numel(), 0, None)
    assert rc != 0 and b"one gate/up input scale" in q4t.load().q4t_last_error()


def test_ep_two_gpus_nccl(q4t, gpu_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29655", os.path.join(ROOT, "bench.py"),
                        "--gpus", "2", "--steps", "2", "--warmup", "3", "--quick"],
                       capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    import json
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["n_gpus"] == 2 and line["metric"] == "moe_ep_prefill_tokens_per_s" and line["scaling"] == "strong"
    # the sharded step reproduces the single-GPU layer bit for bit
    assert line["equals_single_gpu_bits"] is True
    if line.get("plain_sharding"):     # timed only without --quick
        assert line["plain_sharding"]["equals_replicated_placement_bits"] is True
    assert line["value"] > 0 and 0 < line["ms_per_step"] < 50
    assert set(line["phase_ms_rank0"]) >= {"publish", "ids_all_gather", "experts_pull_push", "landed_barrier", "combine"}
