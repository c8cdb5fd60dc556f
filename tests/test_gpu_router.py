"""GPU parity: BF16 projections, router top-k, permutation tables."""
import numpy as np
import pytest
import torch

import synth
from gpu_util import bf16_ulp_diff, dev, host
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_router_known_answers(q4t, gpu_lib):
    """Tie and near-tie vectors of the reference's router contract
    (tools/verify/moe_replay_gpu.cu:24-69)."""
    E, k, T = 512, 3, 4
    logits = np.zeros((T, E), np.uint16)
    logits[1, 0], logits[1, 511], logits[1, 5] = 0x3F80, 0x3F81, 0x3F7F
    logits[2, 5], logits[2, 511] = 0xC000, 0x4000
    logits[3, 511], logits[3, 5] = 0x42C8, 0xC2C8
    ids, w = q4t.router_topk(dev(logits), k)
    ids, w = host(ids), host(w)
    assert ids[0].tolist() == [0, 1, 2]
    assert ids[1].tolist() == [511, 0, 5]
    for t in range(T):
        v = O.bf16_to_f32(logits[t, ids[t]]).astype(np.float64)
        p = np.exp(v - v.max())
        assert np.abs(w[t] - p / p.sum()).max() <= 2e-6


@pytest.mark.parametrize("T,E,k", [(1, 512, 10), (16, 512, 10), (257, 512, 16), (5, 64, 4), (3, 100, 1)])
def test_router_topk_matches_oracle(q4t, gpu_lib, T, E, k):
    rng = np.random.default_rng(T + E)
    logits = O.f32_to_bf16(rng.standard_normal((T, E)).astype(np.float32))
    logits[0, : E // 2] = logits[0, 0]          # many exact ties -> lowest ids first
    ids, w = q4t.router_topk(dev(logits), k)
    want_ids, want_w = O.router_topk(logits, k)
    assert np.array_equal(host(ids), want_ids)
    assert np.abs(host(w) - want_w).max() <= 2e-6


@pytest.mark.parametrize("M", [1, 2, 8])
def test_small_m_linear_bit_exact(q4t, gpu_lib, M):
    """M <= 8 follows the reference GEMV accumulation order exactly."""
    rng = np.random.default_rng(M)
    for N, K in [(512, 2048), (1024, 2048), (2048, 512)]:
        x = O.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
        w = O.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
        got = host(q4t.bf16_linear(dev(x), dev(w)))
        assert np.array_equal(got, O.bf16_linear(x, w, 1))


@pytest.mark.parametrize("M,N,K", [(16, 512, 2048), (128, 2048, 512), (300, 1024, 2048), (9, 640, 2560)])
def test_tensor_core_linear(q4t, gpu_lib, M, N, K):
    rng = np.random.default_rng(M + N)
    x = O.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    w = O.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    got = host(q4t.bf16_linear(dev(x), dev(w)))
    xf, wf = O.bf16_to_f32(x).astype(np.float64), O.bf16_to_f32(w).astype(np.float64)
    ref = xf @ wf.T
    # one bf16 rounding (2^-9 relative) on top of fp32 accumulation noise, which
    # is bounded relative to the sum of the terms' magnitudes, not to the result
    tol = 2.0 ** -8 * np.abs(ref) + 1e-5 * (np.abs(xf) @ np.abs(wf).T)
    err = np.abs(O.bf16_to_f32(got).astype(np.float64) - ref)
    assert np.all(err <= tol), f"worst excess {np.max(err - tol)}"
    ulp = bf16_ulp_diff(got, O.f32_to_bf16(ref.astype(np.float32)))
    assert (ulp > 0).mean() < 0.02


@pytest.mark.parametrize("M,N,K", [(9, 512, 2048), (16, 512, 2048), (33, 512, 2048), (128, 512, 2048), (128, 2048, 512),
                                   (100, 640, 2560), (17, 64, 64), (40, 128, 832)])
def test_linear_of_one_row_tile_equals_the_general_kernel(q4t, gpu_lib, M, N, K):
    """Batches of 9..128 rows run on the kernel that loads four k-blocks per TMA operation
    (K = 832 and 2560/64 = 40 end in a short or exact group, K = 64 is a single k-block); the
    same rows inside a 300-row batch run on the general GEMM kernel.  Same MMA sequence over K,
    so the same bits: a token's logits do not depend on the size of the batch it arrives in."""
    rng = np.random.default_rng(M + N + K)
    x = O.f32_to_bf16(rng.standard_normal((300, K)).astype(np.float32))
    w = O.f32_to_bf16((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    big = host(q4t.bf16_linear(dev(x), dev(w)))
    small = host(q4t.bf16_linear(dev(np.ascontiguousarray(x[:M])), dev(w)))
    assert small.shape == (M, N)
    assert np.array_equal(small, big[:M])


@pytest.mark.parametrize("T,k,E", [(1, 10, 512), (16, 10, 512), (700, 10, 512), (37, 4, 64)])
def test_permutation_tables(q4t, gpu_lib, T, k, E):
    """Stable order (expert ascending, then (token,slot) ascending), read back
    from the workspace of a routed forward."""
    L = synth.make_layer(E=E, hs=256, moe_is=128, shared_is=128, seed=3)
    dl = q4t.DeviceLayer.from_host(L)
    ids, rw = synth.random_routing(T, k, E, seed=T)
    if T > 4:
        ids[3, 1] = -1            # skipped like the reference does (moe_gemm.cu:140)
        ids[4, 0] = E
    x = synth.make_x(T, L.hs)
    rf = q4t.RoutedForward(dl, T, k)
    y = torch.zeros((T, L.hs), dtype=torch.float32, device="cuda")
    rf(dev(x), dev(ids), dev(rw), y, flags=4)     # the grouped path also for decode-sized batches
    rf.status()
    counts, offsets, rof, fofr = O.permutation(ids, E)
    R = T * k
    assert np.array_equal(host(rf.region("counts", torch.int32, E)), counts)
    assert np.array_equal(host(rf.region("offsets", torch.int32, E + 1)), offsets)
    assert np.array_equal(host(rf.region("row_of_flat", torch.int32, R)), rof)
    n = offsets[-1]
    assert np.array_equal(host(rf.region("flat_of_row", torch.int32, R))[:n], fofr[:n])
    nt = int(host(rf.region("ntiles", torch.int32, 1))[0])
    tiles = (counts + 127) // 128
    # batches that run as CTA pairs pad every expert to an even number of row tiles
    # (the extra tile is empty); smaller batches have no empty tiles
    paired = nt != int(tiles.sum())
    if paired:
        assert nt == int(((tiles + 1) // 2 * 2).sum())
    row0 = host(rf.region("tile_row0", torch.int32, nt))
    nrows = host(rf.region("tile_nrows", torch.int32, nt))
    exp = host(rf.region("tile_expert", torch.int32, nt))
    assert np.all(nrows >= (0 if paired else 1)) and np.all(nrows <= 128)
    if paired:
        assert np.array_equal(exp[0::2], exp[1::2]), "both tiles of a pair belong to one expert"
    real = nrows > 0
    assert int(real.sum()) == int(tiles.sum())
    assert np.array_equal(row0[real], np.concatenate([[0], np.cumsum(nrows[real])[:-1]]))
    assert np.all(offsets[exp[real]] <= row0[real]) and np.all((row0 + nrows)[real] <= offsets[exp[real] + 1])
