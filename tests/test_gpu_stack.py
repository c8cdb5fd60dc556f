"""The decode-stack harness: x <- bf16(x + MoE_l(RMSNorm(x))) over several layers.
The residual + RMSNorm step is bit-exact against the oracle; the stack equals the
layer-by-layer composition of the same entry points bit for bit and follows the oracle's
stack within the layer tolerance."""
import numpy as np
import pytest
import torch

import synth
from gpu_util import dev, host
from oracle import oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("T,hs", [(1, 256), (5, 2048), (130, 2560), (9, 8192)])
def test_residual_rmsnorm_bit_exact(q4t, gpu_lib, T, hs):
    rng = np.random.default_rng(T + hs)
    x = O.f32_to_bf16(rng.standard_normal((T, hs), dtype=np.float32) * np.float32(2.0))
    y = O.f32_to_bf16(rng.standard_normal((T, hs), dtype=np.float32))
    for with_y in (True, False):
        xd, yd = dev(x), dev(y)
        hd = torch.empty_like(xd)
        q4t.residual_rmsnorm(xd, yd if with_y else None, hd)
        torch.cuda.synchronize()
        x_ref, h_ref = O.residual_rmsnorm_bf16(x, y if with_y else None)
        assert np.array_equal(host(xd).view(np.uint16), x_ref)
        assert np.array_equal(host(hd).view(np.uint16), h_ref)


def test_residual_rmsnorm_rejects_bad_dims(q4t, gpu_lib):
    x = torch.zeros((2, 100), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(q4t.Q4TError, match="multiple of 8"):
        q4t.residual_rmsnorm(x, None, torch.empty_like(x))


def test_stack_equals_composition_and_oracle(q4t, gpu_lib):
    E, hs, is_, sis, k, T, nl = 32, 512, 256, 128, 4, 24, 3
    layers = [synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=70 + i) for i in range(nl)]
    dls = [q4t.DeviceLayer.from_host(L) for L in layers]
    x0 = synth.make_x(T, hs, seed=8)
    # the stack in one go
    xs = dev(x0).view(torch.bfloat16).clone()
    q4t.DecodeStack(dls, T, k)(xs)
    # the same entry points, layer by layer
    xc = dev(x0).view(torch.bfloat16).clone()
    h = torch.empty_like(xc)
    y = torch.empty_like(xc)
    for i, dl in enumerate(dls):
        q4t.residual_rmsnorm(xc, y if i else None, h)
        q4t.MoEForward(dl, T, k)(h, y)
    q4t.residual_rmsnorm(xc, y, h)
    torch.cuda.synchronize()
    assert torch.equal(xs.view(torch.int16), xc.view(torch.int16))
    # the oracle's stack (device-order arithmetic; fp32 logits order differs from the tensor cores',
    # so a near-tie in one router can move one token: compare in the layer tolerance)
    xo = x0.copy()
    yo = None
    for L in layers:
        xo, ho = O.residual_rmsnorm_bf16(xo, yo)
        yo = O.moe_forward(ho, L, k)["y"]
    xo, _ = O.residual_rmsnorm_bf16(xo, yo)
    got, ref = O.bf16_to_f32(host(xs).view(np.uint16)), O.bf16_to_f32(xo)
    assert np.max(np.abs(got - ref)) <= 2e-3 * np.max(np.abs(ref)) + 2.0 ** -8 * np.max(np.abs(ref))


@pytest.mark.parametrize("T", [1, 9, 130])
def test_gated_residual_write_fused_into_combine(q4t, gpu_lib, T):
    """The layer's gated residual write (GatedResidualFrame::Write after MoEForward,
    src/model/decoder_layer.cu:708 of the reference) fused into the final combine: y is
    unchanged and out equals the oracle's bf16(R + y * gate) bit for bit."""
    E, hs, is_, sis, k, hc = 64, 1024, 256, 256, 6, 4
    L = synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=5)
    dl = q4t.DeviceLayer.from_host(L)
    x = dev(synth.make_x(T, hs, seed=T))
    rng = np.random.default_rng(T)
    res = O.f32_to_bf16(rng.standard_normal((T, hc * hs)).astype(np.float32))
    gate = O.f32_to_bf16((2.0 / (1.0 + np.exp(-rng.standard_normal((T, hc))))).astype(np.float32))
    fwd = q4t.MoEForward(dl, T, k)
    y0 = torch.empty((T, hs), dtype=torch.bfloat16, device="cuda")
    fwd(x, y0)
    y1 = torch.empty_like(y0)
    out = torch.zeros((T, hc * hs), dtype=torch.bfloat16, device="cuda")
    fwd(x, y1, hc_write=(dev(res).view(torch.bfloat16), dev(gate).view(torch.bfloat16), out))
    fwd.status()
    assert torch.equal(y0.view(torch.int16), y1.view(torch.int16))
    want = O.gated_residual_write(host(y1), res, gate)
    assert np.array_equal(host(out), want)


@pytest.mark.parametrize("T,hs", [(1, 1024), (9, 512), (70, 2560), (130, 512)])
def test_stack_with_the_norm_step_fused_into_the_combine(q4t, gpu_lib, T, hs):
    """x <- bf16(x + y), h <- RMSNorm(x) between two layers: as a launch of its own and fused into
    the layer's final combine (q4t_forward_options.norm_*): the same bits in x after three layers."""
    E, is_, sis, k, nl = 32, 256, 128, 4, 3
    layers = [synth.make_layer(E=E, hs=hs, moe_is=is_, shared_is=sis, seed=40 + i) for i in range(nl)]
    dls = [q4t.DeviceLayer.from_host(L) for L in layers]
    x0 = synth.make_x(T, hs, seed=T)
    xa = dev(x0).view(torch.bfloat16).clone()
    xb = dev(x0).view(torch.bfloat16).clone()
    q4t.DecodeStack(dls, T, k, fused=False)(xa)
    q4t.DecodeStack(dls, T, k, fused=True)(xb)
    torch.cuda.synchronize()
    assert torch.equal(xa.view(torch.int16), xb.view(torch.int16))


def test_norm_write_rejects_bad_arguments(q4t, gpu_lib):
    L = synth.make_layer(E=8, hs=256, moe_is=128, shared_is=128, seed=1)
    dl = q4t.DeviceLayer.from_host(L)
    T, k = 4, 2
    fwd = q4t.MoEForward(dl, T, k)
    x = dev(synth.make_x(T, 256, seed=2))
    y = torch.empty((T, 256), dtype=torch.bfloat16, device="cuda")
    res = torch.zeros((T, 256), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(q4t.Q4TError, match="two distinct"):
        fwd(x, y, norm_write=(res, res, 1e-6))
    with pytest.raises(q4t.Q4TError, match="two distinct"):
        fwd(x, y, norm_write=(res, None, 1e-6))
