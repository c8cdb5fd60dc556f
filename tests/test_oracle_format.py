"""CPU tests: the oracle's format / layout primitives against the reference's
known-answer vectors (tests/quant_fp4_test.cpp:127-244 of the reference),
against golden tables produced by the reference's own header code, and, when
the pinning shim oracle/_ref is present, bit-for-bit against those headers."""
import numpy as np
import pytest

from oracle import oracle as O


def test_e2m1_decode_table():
    expect = [0, .5, 1, 1.5, 2, 3, 4, 6, -0., -.5, -1, -1.5, -2, -3, -4, -6]
    L = O.lib()
    for c, v in enumerate(expect):
        got = L.q4o_e2m1_to_float(c)
        assert got == v and np.signbit(got) == np.signbit(np.float32(v))


def test_e2m1_encode_known_answers():
    L = O.lib()
    for v, c in zip([.5, 1, 1.5, 2, 3, 4, 6, 0], [1, 2, 3, 4, 5, 6, 7, 0]):
        assert L.q4o_float_to_e2m1(v) == c
    ties = {0.25: 0, 0.75: 2, 1.25: 2, 1.75: 4, 2.5: 4, 3.5: 6, 5.0: 6}
    for v, c in ties.items():
        assert L.q4o_float_to_e2m1(v) == c
        assert L.q4o_float_to_e2m1(-v) == (c | 8)
    assert L.q4o_float_to_e2m1(100.0) == 7
    assert L.q4o_float_to_e2m1(-100.0) == 15
    assert L.q4o_float_to_e2m1(-1.0) == 10
    assert L.q4o_float_to_e2m1(-0.0) == 0          # -0.0 does not compare below zero
    assert L.q4o_float_to_e2m1(-0.1) == 8          # negative input that rounds to 0 keeps its sign


def test_e4m3_known_answers():
    L = O.lib()
    for v in [0.0, .5, 1, 1.5, 2, 3, 4, 6, 448, 0.015625, 0.03125, 128, .75, 2.25, .0625]:
        assert L.q4o_e4m3_to_float(L.q4o_float_to_e4m3(v)) == v
    assert L.q4o_float_to_e4m3(5.0 * 0.001953125) == 5
    assert L.q4o_e4m3_to_float(L.q4o_float_to_e4m3(1000.0)) == 448.0
    assert L.q4o_e4m3_to_float(0x7F) == 0.0
    prev = 0.0
    for i in range(1000):
        d = L.q4o_e4m3_to_float(L.q4o_float_to_e4m3(0.001 + i * 0.5))
        assert d >= prev - 1e-6
        prev = d


def test_swizzle_known_answers():
    assert O.lib().q4o_sf_num_gtiles(128) == 2
    for (r, g, nt), want in {(0, 0, 2): 0, (0, 1, 2): 1, (0, 3, 2): 3, (0, 4, 2): 512,
                             (0, 7, 2): 515, (1, 0, 2): 16, (31, 0, 2): 496, (32, 0, 2): 4,
                             (127, 7, 2): 1023, (128, 0, 2): 1024, (128, 0, 40): 20480}.items():
        assert O.sf_offset(r, g, nt) == want
    assert O.lib().q4o_sf_num_gtiles(2560) == 40
    for (rows, K), want in {(1, 2560): 20480, (8, 640): 5120, (128, 640): 5120,
                            (129, 640): 10240, (640, 2560): 102400}.items():
        assert O.sf_buffer_size(rows, K) == want


def test_swizzle_roundtrip():
    rows, K = 300, 640
    rng = np.random.default_rng(0)
    rm = rng.integers(0, 128, (rows, K // 16), dtype=np.uint8)
    sw = O.swizzle_sf(rm, rows, K)
    assert sw.size == O.sf_buffer_size(rows, K)
    assert np.array_equal(O.unswizzle_sf(sw, rows, K), rm)
    # padding bytes are zero
    assert int(sw.astype(np.int64).sum()) == int(rm.astype(np.int64).sum())


def test_encoder_tables_match_reference_golden(golden):
    bits = np.arange(65536, dtype=np.uint32)
    f = (bits << 16).view(np.float32)
    finite = ~np.isnan(f)
    out = np.empty(65536, np.uint8)
    import ctypes as C
    O.lib().q4o_float_to_e2m1_bulk(f.ctypes.data_as(C.POINTER(C.c_float)), C.c_size_t(65536),
                                   out.ctypes.data_as(C.POINTER(C.c_uint8)))
    assert np.array_equal(out[finite], golden["e2m1_of_bf16"][finite])
    O.lib().q4o_float_to_e4m3_bulk(f.ctypes.data_as(C.POINTER(C.c_float)), C.c_size_t(32768),
                                   out.ctypes.data_as(C.POINTER(C.c_uint8)))
    assert np.array_equal(out[:32768][finite[:32768]], golden["e4m3_of_bf16"][finite[:32768]])


def test_act_quant_golden(golden):
    """Reference act-quant case (M=5, K=64, seed 7, global scale 0.00167)."""
    packed, sf = O.quantize_bf16(golden["actq_x_bf16"], 0.00167)
    assert np.array_equal(packed, golden["actq_packed"])
    assert np.array_equal(sf, golden["actq_sf_swz"])
    assert np.array_equal(O.unswizzle_sf(sf, 5, 64), golden["actq_sf_rm"])


@pytest.mark.parametrize("s,N,K", [(0, 640, 2560), (1, 2560, 640)])
@pytest.mark.parametrize("M", [1, 8, 64, 256])
def test_fp4_gemm_golden(golden, s, N, K, M):
    """Reference W4A4 GEMM cases (all four M of tests/quant_fp4_test.cpp:367-471); mode 0 must
    reproduce the reference's CPU check value exactly, mode 1 (exact arithmetic) within its
    0.02 bound.  The M = 256 fixture stores every eighth row of the expected output."""
    args = (golden[f"gemm{s}_w_packed"], golden[f"gemm{s}_w_sf_swz"],
            golden[f"gemm{s}_m{M}_a_packed"], golden[f"gemm{s}_m{M}_a_sf_swz"], M, N, K, 0.29, 0.41)
    step = 8 if M == 256 else 1
    want = golden[f"gemm{s}_m{M}_out_rows8" if step == 8 else f"gemm{s}_m{M}_out"]
    got0 = O.fp4_gemm(*args, 0)[::step]
    assert np.array_equal(got0, want)
    got1 = O.fp4_gemm(*args, 1)[::step]
    rel = np.abs(got1 - want) / np.maximum(1.0, np.abs(want))
    assert rel.max() < 0.02
    # the exact mode differs from the fp32 sequential sum only by rounding noise
    assert rel.max() < 1e-3


def test_pinned_against_reference_headers():
    """Bit-for-bit against the reference's own inline functions (oracle/_ref).
    Sampled here (every special value plus two million random bit patterns); the GPU test of the
    encoders sweeps every float bit pattern against the same compare chain."""
    R = O.ref_lib()
    if R is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    import ctypes as C
    L = O.lib()
    for c in range(256):
        assert L.q4o_e4m3_to_float(c) == R.ref_e4m3_to_float(c)
        assert L.q4o_e2m1_to_float(c & 15) == R.ref_e2m1_to_float(c & 15)
    rng = np.random.default_rng(1)
    bits = np.concatenate([
        rng.integers(0, 2**32, 2_000_000, dtype=np.uint64).astype(np.uint32),
        (np.arange(65536, dtype=np.uint32) << 16),
        np.arange(0x3B000000, 0x44000000, 4099, dtype=np.uint32),  # dense over the e4m3 range
    ])
    f = bits.view(np.float32)
    f = f[~np.isnan(f)]
    n = f.size
    a = np.empty(n, np.uint8)
    b = np.empty(n, np.uint8)
    fp, ap, bp = (x.ctypes.data_as(C.c_void_p) for x in (f, a, b))
    L.q4o_float_to_e4m3_bulk(fp, C.c_size_t(n), ap)
    R.ref_float_to_e4m3_bulk(fp, C.c_size_t(n), bp)
    assert np.array_equal(a, b)
    L.q4o_float_to_e2m1_bulk(fp, C.c_size_t(n), ap)
    R.ref_float_to_e2m1_bulk(fp, C.c_size_t(n), bp)
    assert np.array_equal(a, b)
    for rows, K in [(1, 2560), (8, 640), (129, 640), (640, 2560), (1024, 2048), (300, 64)]:
        assert O.sf_buffer_size(rows, K) == R.ref_sf_buffer_size(rows, K)
        nt = L.q4o_sf_num_gtiles(K)
        assert nt == R.ref_sf_num_gtiles(K)
        for r in range(0, rows, 7):
            for g in range(0, K // 16, 3):
                assert O.sf_offset(r, g, nt) == R.ref_sf_offset(r, g, nt)
