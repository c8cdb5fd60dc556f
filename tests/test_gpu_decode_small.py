"""The decode-sized path of the routed experts (at most 64 tokens by default, 128 on request; the counterpart of the
reference's MoEDeviceDecode / MoEDeviceDecodeMulti, include/q4t/quant/moe_decode.h:8-36)
against the general grouped path, bit for bit: the reference's own check of its grouped decode
against its per-row decode asks for zero ulp (tests/moe_decode_grouped_test.cpp:328-411).  The
general path is compared with the CPU oracle's taps and with the reference's GPU code elsewhere.
"""
import importlib

import numpy as np
import pytest
import torch

import synth
from gpu_util import dev, host
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _both_paths(q4t, dl, x, ids, rw, T, k):
    out = []
    for flags in (q4t.FLAG_DUMP_GATE_UP | q4t.FLAG_GENERAL_PATH, q4t.FLAG_DECODE_PATH):
        rf = q4t.RoutedForward(dl, T, k)
        rf.ws.fill_(0xEE)
        y = torch.zeros((T, dl.hs), dtype=torch.float32, device="cuda")
        rf(x, ids, rw, y, flags=flags)
        rf.status()
        R = T * k
        out.append(dict(y=host(y), rof=host(rf.region("row_of_flat", torch.int32, R)),
                        gu=host(rf.region("gu_out", torch.int16, R * 2 * dl.moe_is)).reshape(R, -1),
                        dn=host(rf.region("dn_out", torch.int16, R * dl.hs)).reshape(R, -1)))
    return out


@pytest.mark.parametrize("E,hs,is_,T,k", [
    (512, 2048, 512, 1, 10), (512, 2048, 512, 8, 10), (512, 2048, 512, 16, 10),   # the benchmark layer
    (512, 2560, 640, 1, 10), (512, 2560, 640, 5, 10),      # the reference's decode shapes: K = 640 ends in a short k-block
    (16, 512, 256, 16, 4),                                 # few experts: up to 16 rows per expert
    (16, 256, 128, 16, 16),                                # 256 entries, 16 per expert
    (4, 256, 128, 16, 4),                                  # 16+ rows per expert: more than one pass per CTA
    (64, 1024, 384, 3, 6), (32, 4096, 1024, 2, 8),
    (512, 2048, 512, 32, 10), (512, 2048, 512, 128, 10),   # larger batches: the lists hold up to 2048 entries
    (16, 512, 256, 64, 4), (4, 256, 128, 100, 4),          # many rows per expert: several passes
    (64, 512, 128, 128, 16)])                              # 2048 entries
def test_decode_sized_path_equals_general_path(q4t, gpu_lib, E, hs, is_, T, k):
    if E >= 512:     # built on the device (seeded); the CPU oracle is left out at this size
        L = None
        dl = importlib.import_module("qwen4-thor_b200.synthetic").device_layer(q4t, E, hs, is_, 128, seed=E + T + k)
    else:
        L = synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=128, seed=E + T + k, per_expert_input_scale=True)
        dl = q4t.DeviceLayer.from_host(L)
    x = dev(synth.make_x(T, hs, seed=T + 11))
    ids_h, rw_h = synth.random_routing(T, k, E, seed=T + 12)
    if T * k > 6:
        ids_h.reshape(-1)[5] = -1          # skipped entries (src/quant/moe_gemm.cu:140)
        ids_h.reshape(-1)[2] = E
    if T > 1:
        ids_h[1, 0] = ids_h[1, 1]          # a token naming one expert twice (a replayed table may)
    if E == 4:
        ids_h[:, 1] = 0                    # expert 0 gets more than 16 rows
    general, small = _both_paths(q4t, dl, x, dev(ids_h), dev(rw_h), T, k)
    R = T * k
    valid = (ids_h.reshape(-1) >= 0) & (ids_h.reshape(-1) < E)
    assert np.array_equal(small["rof"], np.where(valid, np.arange(R), -1))
    assert np.array_equal((general["rof"] >= 0), valid)
    g_rows = general["rof"][valid]
    gu_bad = int((small["gu"][valid] != general["gu"][g_rows]).sum())
    dn_bad = int((small["dn"][valid] != general["dn"][g_rows]).sum())
    y_bad = int((small["y"] != general["y"]).sum())
    print(f"[decode-sized vs general E={E} hs={hs} is={is_} T={T} k={k}] differing values: gate|up {gu_bad}, "
          f"down rows {dn_bad}, routed sum {y_bad}")
    assert gu_bad == 0 and dn_bad == 0 and y_bad == 0
    if L is not None:
        want = O.routed_forward(host(x), ids_h, rw_h, L, 1)
        assert np.abs(small["y"] - want).max() <= 2e-3 * np.abs(want).max()


def test_whole_layer_decode_sized_equals_general(q4t, gpu_lib):
    """q4t_moe_forward at T = 1..128: same experts, same weights, same output bits on both paths
    (the decode-sized path by default up to 64 tokens, on request above)."""
    E, hs, is_, sis, k = 128, 1024, 256, 256, 8
    L = synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=77)
    dl = q4t.DeviceLayer.from_host(L)
    for T in (1, 2, 7, 9, 16, 33, 64, 128):
        x = dev(synth.make_x(T, hs, seed=T))
        ys = []
        for flags in (q4t.FLAG_GENERAL_PATH, q4t.FLAG_DECODE_PATH if T > 64 else 0):
            fwd = q4t.MoEForward(dl, T, k)
            y = torch.empty((T, hs), dtype=torch.bfloat16, device="cuda")
            fwd(x, y, flags=flags)
            fwd.status()
            ys.append((host(y), host(fwd.region("expert_ids", torch.int32, T * k)), host(fwd.region("router_w", torch.float32, T * k))))
        assert np.array_equal(ys[0][1], ys[1][1]) and np.array_equal(ys[0][2], ys[1][2])
        assert np.array_equal(ys[0][0], ys[1][0]), f"T={T}"


@pytest.mark.parametrize("T", [1, 8, 40])
def test_decode_sized_layer_in_a_cuda_graph(q4t, gpu_lib, T):
    """The layer on the decode-sized path (chained launches, the early release of the down kernel,
    the side-stream shared expert) captured as one CUDA graph: every replay gives the eager bits."""
    E, hs, is_, sis, k = 64, 1024, 256, 256, 6
    L = synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=91)
    dl = q4t.DeviceLayer.from_host(L)
    xs = [dev(synth.make_x(T, hs, seed=T + i)) for i in range(3)]
    fwd = q4t.MoEForward(dl, T, k)
    x = torch.empty((T, hs), dtype=torch.int16, device="cuda")
    y = torch.empty((T, hs), dtype=torch.bfloat16, device="cuda")
    eager = []
    for xi in xs:
        x.copy_(xi.view(torch.int16).reshape(T, hs))
        fwd(x, y)
        fwd.status()
        eager.append(host(y))
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fwd(x, y)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fwd(x, y)
    torch.cuda.current_stream().wait_stream(side)
    for rep in range(2):
        for xi, want in zip(xs, eager):
            x.copy_(xi.view(torch.int16).reshape(T, hs))
            graph.replay()
            torch.cuda.synchronize()
            assert np.array_equal(host(y), want), f"T={T} replay {rep}"
    fwd.status()
