"""Seeded synthetic MoE layers and activations with the shapes and value
distributions of the benchmark configurations (weights ~ N(0, 0.02) quantised
to NVFP4 with global scale amax/(6*448); activations ~ N(0, 1) in bf16).
Weight quantisation goes through the CPU oracle, so this module is test
infrastructure, like the oracle itself."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def _quant_weight(w: np.ndarray, ws2: float):
    packed, sf = O.quantize_f32(w, ws2)
    return packed, O.swizzle_sf(sf, w.shape[0], w.shape[1])


def make_layer(E=512, hs=2048, moe_is=512, shared_is=512, seed=20260921, gu_input_scale=None,
               per_expert_input_scale=False, w_std=0.02) -> O.Layer:
    rng = np.random.default_rng(seed)
    gu_packed = np.empty((E * 2 * moe_is, hs // 2), np.uint8)
    dn_packed = np.empty((E * hs, moe_is // 2), np.uint8)
    gu_blk = O.sf_buffer_size(2 * moe_is, hs)
    dn_blk = O.sf_buffer_size(hs, moe_is)
    gu_sf = np.empty(E * gu_blk, np.uint8)
    dn_sf = np.empty(E * dn_blk, np.uint8)
    gu_ws2 = np.empty(E, np.float32)
    dn_ws2 = np.empty(E, np.float32)
    for e in range(E):
        wgu = rng.standard_normal((2 * moe_is, hs), dtype=np.float32) * np.float32(w_std)
        wdn = rng.standard_normal((hs, moe_is), dtype=np.float32) * np.float32(w_std)
        # gate and up share one global scale (amax over both), as in the checkpoint
        gu_ws2[e] = np.float32(np.abs(wgu).max() / np.float32(6.0 * 448.0))
        dn_ws2[e] = np.float32(np.abs(wdn).max() / np.float32(6.0 * 448.0))
        p, s = _quant_weight(wgu, float(gu_ws2[e]))
        gu_packed[e * 2 * moe_is:(e + 1) * 2 * moe_is] = p
        gu_sf[e * gu_blk:(e + 1) * gu_blk] = s
        p, s = _quant_weight(wdn, float(dn_ws2[e]))
        dn_packed[e * hs:(e + 1) * hs] = p
        dn_sf[e * dn_blk:(e + 1) * dn_blk] = s
    # activation global scales: x ~ N(0,1) has amax around 4.5-5; intermediate
    # values of a random expert are small (|g*sig(g)*u| << 1)
    base_in = np.float32(5.0 / (6.0 * 448.0)) if gu_input_scale is None else np.float32(gu_input_scale)
    gu_in = np.full(E, base_in, np.float32)
    dn_in = np.full(E, np.float32(2.0 / (6.0 * 448.0)), np.float32)
    if per_expert_input_scale:
        gu_in = (gu_in * (1.0 + 0.25 * rng.random(E, dtype=np.float32))).astype(np.float32)
        dn_in = (dn_in * (1.0 + 0.5 * rng.random(E, dtype=np.float32))).astype(np.float32)
    gate = O.f32_to_bf16(rng.standard_normal((E, hs), dtype=np.float32) * np.float32(w_std))
    sgu = O.f32_to_bf16(rng.standard_normal((2 * shared_is, hs), dtype=np.float32) * np.float32(w_std))
    sdn = O.f32_to_bf16(rng.standard_normal((hs, shared_is), dtype=np.float32) * np.float32(w_std))
    sgs = O.f32_to_bf16(rng.standard_normal((hs,), dtype=np.float32) * np.float32(w_std))
    return O.Layer(E, hs, moe_is, shared_is, gu_packed=gu_packed, gu_sf=gu_sf, dn_packed=dn_packed,
                   dn_sf=dn_sf, gu_w_scale2=gu_ws2, gu_input_scale=gu_in, dn_w_scale2=dn_ws2,
                   dn_input_scale=dn_in, gate=gate, shared_gu=sgu, shared_down=sdn,
                   shared_gate_scalar=sgs)


def make_x(T, hs, seed=1) -> np.ndarray:
    rng = np.random.default_rng(seed)
    return O.f32_to_bf16(rng.standard_normal((T, hs), dtype=np.float32))


def random_routing(T, k, E, seed=2):
    """Distinct experts per token, weights that sum to 1 (softmax of normals)."""
    rng = np.random.default_rng(seed)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    z = rng.standard_normal((T, k)).astype(np.float32)
    w = np.exp(z - z.max(axis=1, keepdims=True))
    w = (w / w.sum(axis=1, keepdims=True)).astype(np.float32)
    return ids, w
