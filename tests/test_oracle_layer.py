"""CPU tests of the oracle's layer-level restatement: router known answers
(tools/verify/moe_replay_gpu.cu:12-107 of the reference), permutation
properties, and consistency between the 'test twin' and 'device order' modes."""
import numpy as np
import pytest

import synth
from oracle import oracle as O


def test_router_known_answers():
    E, k, T = 512, 3, 4
    logits = np.zeros((T, E), np.uint16)
    logits[1, 0] = 0x3F80
    logits[1, 511] = 0x3F81
    logits[1, 5] = 0x3F7F
    logits[2, 5] = 0xC000
    logits[2, 511] = 0x4000
    logits[3, 511] = 0x42C8
    logits[3, 5] = 0xC2C8
    ids, w = O.router_topk(logits, k)
    assert ids[0].tolist() == [0, 1, 2]          # all-equal row: lowest ids
    assert ids[1].tolist() == [511, 0, 5]        # adjacent bf16 values, unsorted positions
    assert ids[2, 0] == 511 and ids[3, 0] == 511
    for t in range(T):
        v = O.bf16_to_f32(logits[t, ids[t]]).astype(np.float64)
        p = np.exp(v - v.max())
        p /= p.sum()
        assert np.abs(w[t] - p).max() <= 2e-6
    assert np.allclose(w.sum(axis=1), 1.0, atol=1e-6)


def test_router_rejects_nothing_and_orders_by_value():
    rng = np.random.default_rng(3)
    logits = O.f32_to_bf16(rng.standard_normal((7, 64)).astype(np.float32))
    ids, w = O.router_topk(logits, 10)
    v = O.bf16_to_f32(logits)
    for t in range(7):
        order = sorted(range(64), key=lambda e: (-v[t, e], e))[:10]
        assert ids[t].tolist() == order
        assert np.all(np.diff(w[t]) <= 0)


def test_permutation_stable_and_total():
    T, k, E = 37, 10, 64
    ids, _ = synth.random_routing(T, k, E)
    ids[3, 2] = -1          # dropped (out of range), src/quant/moe_gemm.cu:140
    ids[5, 0] = E
    counts, offsets, rof, fofr = O.permutation(ids, E)
    flat = ids.reshape(-1)
    valid = (flat >= 0) & (flat < E)
    assert counts.sum() == valid.sum() == offsets[-1]
    assert np.array_equal(np.bincount(flat[valid], minlength=E), counts)
    n = offsets[-1]
    rows = fofr[:n]
    # grouped by expert ascending, flat index ascending inside each expert
    assert np.all(np.diff(flat[rows]) >= 0)
    for e in range(E):
        seg = rows[offsets[e]:offsets[e + 1]]
        assert np.all(np.diff(seg) > 0)
    assert np.array_equal(rof[rows], np.arange(n))
    assert np.all(rof[~valid] == -1)


@pytest.fixture(scope="module")
def small_layer():
    return synth.make_layer(E=16, hs=512, moe_is=256, shared_is=128, seed=11,
                            per_expert_input_scale=True)


def test_routed_modes_agree(small_layer):
    L = small_layer
    T, k = 9, 4
    x = synth.make_x(T, L.hs, seed=5)
    ids, rw = synth.random_routing(T, k, L.E, seed=6)
    y0 = O.routed_forward(x, ids, rw, L, 0)
    y1, taps = O.routed_forward(x, ids, rw, L, 1, want_taps=True)
    scale = np.abs(y0).max()
    assert scale > 0
    # The device order rounds gu_out to bf16 before SwiGLU; that flips a few
    # intermediate FP4 codes, so the two conventions agree only loosely (the
    # reference accepts l2 < 2e-2 between them, tests/model_moe_test.cpp:433).
    assert np.abs(y1 - y0).max() / scale < 0.1
    assert np.linalg.norm(y1 - y0) / np.linalg.norm(y0) < 3e-2
    # taps: input codes equal a direct quantisation of the gathered rows
    counts, offsets, rof, fofr = O.permutation(ids, L.E)
    for r in range(T * k):
        t, e = fofr[r] // k, ids.reshape(-1)[fofr[r]]
        p, s = O.quantize_f32(O.bf16_to_f32(x[t:t + 1]), float(L.gu_input_scale[e]))
        assert np.array_equal(p[0], taps["a_packed"][r])
        assert np.array_equal(s[0], taps["a_sf"][r])


def test_routed_accumulates_into_y(small_layer):
    L = small_layer
    x = synth.make_x(3, L.hs, seed=7)
    ids, rw = synth.random_routing(3, 2, L.E, seed=8)
    base = np.full((3, L.hs), 0.5, np.float32)
    y = O.routed_forward(x, ids, rw, L, 1, y0=base)
    z = O.routed_forward(x, ids, rw, L, 1)
    assert np.array_equal(y, z + base)


def test_routed_invalid_dims(small_layer):
    with pytest.raises(ValueError):
        O.routed_forward(np.zeros((0, small_layer.hs), np.uint16), np.zeros((0, 2), np.int32),
                         np.zeros((0, 2), np.float32), small_layer, 1)


def test_moe_forward_modes_agree(small_layer):
    L = small_layer
    x = synth.make_x(5, L.hs, seed=9)
    a = O.moe_forward(x, L, 4, logits_mode=0, routed_mode=0, linear_mode=0)
    b = O.moe_forward(x, L, 4, logits_mode=1, routed_mode=1, linear_mode=1)
    ya, yb = O.bf16_to_f32(a["y"]), O.bf16_to_f32(b["y"])
    same_routing = np.array_equal(a["ids"], b["ids"])
    if same_routing:
        assert np.abs(ya - yb).max() / np.abs(ya).max() < 0.1
    # logits of the two accumulation orders agree to bf16 rounding
    la, lb = O.bf16_to_f32(a["logits"]), O.bf16_to_f32(b["logits"])
    assert np.abs(la - lb).max() <= 2.0 ** -7 * np.abs(la).max()
    with pytest.raises(ValueError):
        O.moe_forward(x, L, 17)


def test_gemv_order_matches_float64_closely():
    rng = np.random.default_rng(4)
    x = O.f32_to_bf16(rng.standard_normal((2, 2048)).astype(np.float32))
    w = O.f32_to_bf16(rng.standard_normal((8, 2048)).astype(np.float32) * 0.02)
    y = O.bf16_to_f32(O.bf16_linear(x, w, 1))
    ref = O.bf16_to_f32(x).astype(np.float64) @ O.bf16_to_f32(w).astype(np.float64).T
    assert np.abs(y - ref).max() <= 2.0 ** -8 * np.abs(ref).max() + 1e-6


def test_rmsnorm():
    x = synth.make_x(4, 256, seed=10)
    out = O.bf16_to_f32(O.rmsnorm_bf16(x))
    xf = O.bf16_to_f32(x).astype(np.float64)
    ref = xf / np.sqrt((xf ** 2).mean(axis=1, keepdims=True) + 1e-6)
    assert np.abs(out - ref).max() < 2.0 ** -7 * np.abs(ref).max()


def test_exact_gemm_against_float64_numpy():
    """The integer dot of mode 1 equals a float64 evaluation of the same sum."""
    rng = np.random.default_rng(12)
    N, K, M = 24, 256, 3
    w = rng.standard_normal((N, K)).astype(np.float32)
    a = rng.standard_normal((M, K)).astype(np.float32) * 3
    iw, ia = np.float32(0.013), np.float32(0.0021)
    wp, ws = O.quantize_f32(w, float(iw))
    ap, as_ = O.quantize_f32(a, float(ia))
    got = O.fp4_gemm(wp, O.swizzle_sf(ws, N, K), ap, O.swizzle_sf(as_, M, K), M, N, K,
                     float(iw), float(ia), 1)
    wd = O.dequant_to_f32(wp, ws, 1.0).astype(np.float64)   # codes * block scale, exact in f32
    ad = O.dequant_to_f32(ap, as_, 1.0).astype(np.float64)
    alpha = np.float64(np.float32(iw * ia))
    want = ((ad @ wd.T) * alpha).astype(np.float32)
    assert np.array_equal(got, want)


def test_rmsnorm_matches_float64_and_residual_step():
    """RMSNorm restated in the reference's summation order agrees with a float64
    evaluation to bf16 rounding, and the residual step is exactly bf16(x + y)."""
    rng = np.random.default_rng(5)
    for hs in (256, 2048, 2560):
        x = O.f32_to_bf16(rng.standard_normal((7, hs), dtype=np.float32) * np.float32(3.0))
        y = O.f32_to_bf16(rng.standard_normal((7, hs), dtype=np.float32))
        h = O.bf16_to_f32(O.rmsnorm_bf16(x))
        xf = O.bf16_to_f32(x).astype(np.float64)
        ref = xf / np.sqrt((xf * xf).mean(axis=1, keepdims=True) + 1e-6)
        assert np.max(np.abs(h - ref) / np.maximum(np.abs(ref), 1e-3)) < 2.0 ** -7.5
        x2, h2 = O.residual_rmsnorm_bf16(x, y)
        assert np.array_equal(x2, O.f32_to_bf16(O.bf16_to_f32(x) + O.bf16_to_f32(y)))
        assert np.array_equal(h2, O.rmsnorm_bf16(x2))
        x3, h3 = O.residual_rmsnorm_bf16(x, None)
        assert np.array_equal(x3, x) and np.array_equal(h3, O.rmsnorm_bf16(x))


def test_bf16_routed_experts_match_float64():
    """The MTP draft layer's BF16 experts: the oracle's chain of bf16 roundings stays within
    bf16 rounding of an unrounded float64 evaluation, skips invalid ids and accumulates."""
    rng = np.random.default_rng(8)
    E, hs, is_, T, k = 6, 128, 64, 5, 2
    gu = O.f32_to_bf16(rng.standard_normal((E, 2 * is_, hs), dtype=np.float32) * np.float32(0.05))
    down = O.f32_to_bf16(rng.standard_normal((E, hs, is_), dtype=np.float32) * np.float32(0.05))
    x = O.f32_to_bf16(rng.standard_normal((T, hs), dtype=np.float32))
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    ids[2, 1] = -1
    rw = rng.random((T, k), dtype=np.float32)
    y = O.moe_bf16_routed_forward(x, ids, rw, gu, down)
    xf, gf, df = (O.bf16_to_f32(a).astype(np.float64) for a in (x, gu, down))
    ref = np.zeros((T, hs))
    for t in range(T):
        for s in range(k):
            e = ids[t, s]
            if e < 0:
                continue
            h = gf[e] @ xf[t]
            g, u = h[:is_], h[is_:]
            ref[t] += rw[t, s] * (df[e] @ ((g / (1 + np.exp(-g))) * u))
    assert np.abs(y - ref).max() <= 2.0 ** -6 * np.abs(ref).max()
    y2 = O.moe_bf16_routed_forward(x, ids, rw, gu, down, y0=y)
    assert np.allclose(y2, 2 * y, rtol=1e-6, atol=1e-7)


def test_gated_residual_write_matches_float64():
    """out = bf16(R + y * gate) with one rounding (a fused multiply-add): equal to the float64
    evaluation rounded once to bf16, since products of two bf16 values plus a bf16 are exact
    in float64 (src/model/hyperconnection.cu:286-305)."""
    rng = np.random.default_rng(5)
    T, hc, hs = 7, 4, 96
    y = O.f32_to_bf16(rng.standard_normal((T, hs)).astype(np.float32))
    res = O.f32_to_bf16(rng.standard_normal((T, hc * hs)).astype(np.float32) * 3)
    gate = O.f32_to_bf16((2.0 / (1.0 + np.exp(-rng.standard_normal((T, hc))))).astype(np.float32))
    got = O.gated_residual_write(y, res, gate)
    yf, rf, gf = (O.bf16_to_f32(a).astype(np.float64) for a in (y, res, gate))
    want64 = rf.reshape(T, hc, hs) + yf[:, None, :] * gf[:, :, None]
    # float64 -> float32 -> bf16 would round twice; go through the exact value's bf16 neighbours
    want = O.f32_to_bf16(want64.reshape(T, hc * hs).astype(np.float32))
    diff = (got != want)
    # double rounding can only matter where the float32 rounding lands exactly on a bf16 tie
    assert diff.mean() < 1e-3
    assert np.abs(O.bf16_to_f32(got).astype(np.float64) - want64.reshape(T, -1)).max() <= 2.0 ** -8 * np.abs(want64).max()
