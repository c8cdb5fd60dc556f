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


def test_ep_two_gpus_nccl(q4t, gpu_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29655", os.path.join(ROOT, "bench.py"),
                        "--gpus", "2", "--steps", "2", "--warmup", "3", "--quick"],
                       capture_output=True, text=True, timeout=900, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    assert '"n_gpus": 2' in r.stdout
