"""GPU parity of the NVFP4 tensor-core GEMM (the Fp4Gemm replacement): the
reference's own test cases and tolerance, bit-level comparison with the
oracle's exact mode, and the CUDA-core verification kernel at larger sizes."""
import numpy as np
import pytest
import torch

from gpu_util import bf16_ulp_diff, dev, host
from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _quant_pair(rng, M, N, K, iw, ia, a_scale=1.0):
    w = rng.standard_normal((N, K)).astype(np.float32)
    a = (rng.standard_normal((M, K)) * a_scale).astype(np.float32)
    wp, ws = O.quantize_f32(w, iw)
    ap, as_ = O.quantize_f32(a, ia)
    return wp, O.swizzle_sf(ws, N, K), ap, O.swizzle_sf(as_, M, K)


@pytest.mark.parametrize("s,N,K", [(0, 640, 2560), (1, 2560, 640)])
@pytest.mark.parametrize("M", [1, 8, 64, 256])
def test_fp4_gemm_reference_cases(q4t, gpu_lib, golden, s, N, K, M):
    """tests/quant_fp4_test.cpp:367-471 of the reference: seed 1234 operands, all four M,
    abs(got-want)/max(1,abs(want)) < 0.02 against its CPU dequant GEMM (the M = 256
    fixture stores every eighth row of the expected output)."""
    args = [dev(golden[f"gemm{s}_w_packed"]), dev(golden[f"gemm{s}_w_sf_swz"]),
            dev(golden[f"gemm{s}_m{M}_a_packed"]), dev(golden[f"gemm{s}_m{M}_a_sf_swz"])]
    step = 8 if M == 256 else 1
    got = host(q4t.fp4_gemm(*args, M, N, K, 0.29, 0.41))[::step]
    want = golden[f"gemm{s}_m{M}_out_rows8" if step == 8 else f"gemm{s}_m{M}_out"]
    rel = np.abs(got - want) / np.maximum(1.0, np.abs(want))
    assert rel.max() < 0.02, f"max_rel {rel.max()}"
    assert rel.max() < 1e-3   # in fact only fp32 summation noise apart


@pytest.mark.parametrize("M,N,K", [(1, 1024, 2048), (8, 2048, 512), (64, 1024, 2048), (256, 2048, 512),
                                   (320, 1024, 2048), (129, 640, 2560), (5, 2560, 640), (200, 256, 64)])
def test_fp4_gemm_vs_exact_oracle(q4t, gpu_lib, M, N, K):
    rng = np.random.default_rng(M * 7 + N)
    iw, ia = 0.0137, 0.0019
    wp, ws, ap, as_ = _quant_pair(rng, M, N, K, iw, ia, a_scale=3.0)
    d = [dev(t) for t in (wp, ws, ap, as_)]
    want = O.fp4_gemm(wp, ws, ap, as_, M, N, K, iw, ia, 1)          # float(exact * alpha)
    got32 = host(q4t.fp4_gemm(*d, M, N, K, iw, ia))
    chk = host(q4t.fp4_gemm(*d, M, N, K, iw, ia, check_kernel=True))
    assert np.array_equal(chk, want), "CUDA-core verification kernel must equal the CPU oracle bit for bit"
    scale = np.abs(want).max()
    assert np.abs(got32 - want).max() <= 2e-6 * scale + 1e-30, (
        f"fp32 out: max abs diff {np.abs(got32 - want).max()} vs scale {scale}")
    got16 = host(q4t.fp4_gemm(*d, M, N, K, iw, ia, out_bf16=True))
    want16 = O.f32_to_bf16(want)
    ulp = bf16_ulp_diff(got16, want16)
    mism = int((ulp > 0).sum())
    print(f"[fp4_gemm {M}x{N}x{K}] bf16 outputs differing from bf16(exact*alpha): {mism} of {ulp.size}, max ulp {ulp.max()}")
    assert ulp.max() <= 1
    assert mism <= max(2, ulp.size // 2000)


def test_fp4_gemm_large_vs_verification_kernel(q4t, gpu_lib):
    """Sizes beyond the CPU oracle: tensor cores against exact CUDA-core arithmetic."""
    rng = np.random.default_rng(99)
    M, N, K = 2048, 1024, 2048
    iw, ia = 0.011, 0.0023
    wp, ws, ap, as_ = _quant_pair(rng, M, N, K, iw, ia, a_scale=2.0)
    d = [dev(t) for t in (wp, ws, ap, as_)]
    got = host(q4t.fp4_gemm(*d, M, N, K, iw, ia, out_bf16=True))
    chk = O.f32_to_bf16(host(q4t.fp4_gemm(*d, M, N, K, iw, ia, check_kernel=True)))
    ulp = bf16_ulp_diff(got, chk)
    assert ulp.max() <= 1 and (ulp > 0).mean() < 1e-3, f"max ulp {ulp.max()} mismatch rate {(ulp > 0).mean()}"
