"""GPU parity: number formats, activation quantiser, dequantiser — bit-exact
against the oracle and the reference's golden vectors, through the C ABI."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_hw_encoders_equal_reference_encoders_exhaustively(q4t, gpu_lib):
    """Every float bit pattern: the kernels' hardware e2m1 / ue4m3 converters
    against the compare-chain restatement of the reference's format.h."""
    bad, first = q4t.selftest_encoders(0, 0, 1 << 32)
    assert bad == 0, f"e2m1: {bad} mismatches, first at bits 0x{first:08x}"
    bad, first = q4t.selftest_encoders(1, 0, 1 << 31)
    assert bad == 0, f"ue4m3: {bad} mismatches, first at bits 0x{first:08x}"
    # the SwiGLU epilogue's branch-free reciprocal equals IEEE 1/x on its whole domain
    bad, first = q4t.selftest_encoders(2, 0x3F800000, 0x7E800000 - 0x3F800000)
    assert bad == 0, f"reciprocal: {bad} mismatches, first at bits 0x{first:08x}"


def test_act_quant_reference_golden(q4t, gpu_lib, golden):
    x = dev(golden["actq_x_bf16"])
    packed, sf = q4t.quantize_activation_fp4(x, 0.00167)
    assert np.array_equal(host(packed), golden["actq_packed"])
    assert np.array_equal(O.unswizzle_sf(host(sf), 5, 64), golden["actq_sf_rm"])


@pytest.mark.parametrize("M,K,gs", [(1, 2048, 0.0019), (16, 2048, 0.0017), (130, 512, 0.0008),
                                    (7, 48, 0.01), (300, 640, 1e-5), (33, 2560, 1e3)])
def test_act_quant_bit_exact(q4t, gpu_lib, M, K, gs):
    rng = np.random.default_rng(M * 1000 + K)
    xf = rng.standard_normal((M, K)).astype(np.float32)
    xf[0, :16] = 0.0                       # all-zero group -> block scale 1
    xf[min(1, M - 1), 16:32] *= 1e4        # saturating values
    xf[0, 32:48] = -0.0
    if K >= 64:
        xf[0, 48:64] = np.float32(1e-30)   # values that underflow against the scale
    x = O.f32_to_bf16(xf)
    x[0, 33] = 0x8000                      # bf16 negative zero
    packed, sf = q4t.quantize_activation_fp4(dev(x), gs)
    want_p, want_sf = O.quantize_bf16(x, gs)
    assert np.array_equal(host(packed), want_p)
    got_rm = O.unswizzle_sf(host(sf), M, K)
    assert np.array_equal(got_rm, O.unswizzle_sf(want_sf, M, K))


def test_act_quant_empty_and_errors(q4t, gpu_lib):
    x = torch.zeros((0, 64), dtype=torch.int16, device="cuda")
    packed, sf = q4t.quantize_activation_fp4(x, 1.0)
    assert packed.numel() == 0
    with pytest.raises(q4t.Q4TError):
        q4t.quantize_activation_fp4(torch.zeros((2, 40), dtype=torch.int16, device="cuda"), 1.0)


def test_dequant_bit_exact(q4t, gpu_lib):
    rng = np.random.default_rng(5)
    for N, K, inv in [(2, 32, 0.37), (64, 2048, 0.0013), (5, 640, 11.0)]:
        packed = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
        scale = rng.integers(0, 128, (N, K // 16), dtype=np.uint8)
        got = host(q4t.dequant_fp4_to_bf16(dev(packed), dev(scale), inv))
        want = O.dequant_to_bf16(packed, scale, inv)
        # -0.0 and +0.0 products carry the sign of the code; compare bit patterns
        assert np.array_equal(got, want)
