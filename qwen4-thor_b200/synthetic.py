"""Seeded synthetic MoE layers built directly in HBM, with the shapes and
value distributions of the benchmark configurations: expert and shared
weights ~ N(0, 0.02), expert weights quantised to NVFP4 per expert and per
projection with global scale amax/(6*448) (gate and up share one scale),
activations ~ N(0, 1) in bf16, router weights ~ N(0, 0.02).

Only torch (device buffers, random numbers) and this library's own quantiser
are used, so full-size layers (906 MB at E=512, hs=2048, is=512) are built in
a second or two without touching the host."""
from __future__ import annotations

import math


def device_layer(q4t, E=512, hs=2048, moe_is=512, shared_is=512, seed=0, device="cuda",
                 zipf_s: float | None = None, zipf_strength: float = 1.0):
    """Returns a q4t.DeviceLayer.  With zipf_s set, router column 0 carries a
    per-expert bias b_e = -zipf_s * ln(rank_e) (rank a seeded permutation of the
    experts), which skews expert popularity when the activations hold 1.0 in
    column 0 (see make_x)."""
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    t = {}

    def projection(rows_per_expert, K):
        w = (torch.randn((E, rows_per_expert, K), device=device, generator=g) * 0.02).to(torch.bfloat16)
        amax = w.float().abs().amax(dim=(1, 2))
        gs = (amax / (6.0 * 448.0)).float()
        gs_host = gs.cpu().tolist()
        packed = torch.empty((E * rows_per_expert, K // 2), dtype=torch.uint8, device=device)
        blk = q4t.load().q4t_sf_buffer_size(rows_per_expert, K)
        sf = torch.zeros(E * blk, dtype=torch.uint8, device=device)
        for e in range(E):
            p, s = q4t.quantize_activation_fp4(w[e], gs_host[e])
            packed[e * rows_per_expert:(e + 1) * rows_per_expert] = p
            sf[e * blk:(e + 1) * blk] = s
        return packed, sf, gs.contiguous()

    t["gu_packed"], t["gu_sf"], t["gu_w_scale2"] = projection(2 * moe_is, hs)
    t["dn_packed"], t["dn_sf"], t["dn_w_scale2"] = projection(hs, moe_is)
    t["gu_input_scale"] = torch.full((E,), 5.0 / (6 * 448), dtype=torch.float32, device=device)
    t["dn_input_scale"] = torch.full((E,), 2.0 / (6 * 448), dtype=torch.float32, device=device)
    for n, shape in (("gate", (E, hs)), ("shared_gu", (2 * shared_is, hs)), ("shared_down", (hs, shared_is)),
                     ("shared_gate_scalar", (hs,))):
        t[n] = (torch.randn(shape, device=device, generator=g) * 0.02).to(torch.bfloat16)
    if zipf_s is not None:
        rank = torch.randperm(E, device=device, generator=g).float() + 1.0
        bias = -zipf_s * torch.log(rank) * zipf_strength
        t["gate"][:, 0] = bias.to(torch.bfloat16)
    return q4t.DeviceLayer(E, hs, moe_is, shared_is, t)


def make_x(T, hs, seed=1, device="cuda", bias_column: bool = False):
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn((T, hs), device=device, generator=g).to(torch.bfloat16)
    if bias_column:
        x[:, 0] = 1.0
    return x


def expected_unique_experts(T, k=10, E=512) -> float:
    return E * (1.0 - math.pow((E - k) / E, T))
