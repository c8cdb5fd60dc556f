"""Second oracle: the REFERENCE's own GPU code on the same B200.

oracle/_ref/libq4t_ref_gpu.so is the reference's MoERoutedForward (src/quant/moe_gemm.cu:314-621:
gather-quantise, per-expert cuBLASLt NVFP4 GEMMs, SwiGLU-quantise, combine) and Fp4Gemm
(include/q4t/quant/fp4_gemm.h:58-213), compiled for sm_100a from the reference tree by
`make -C oracle ref_gpu`.  Running it beside this repository's kernels on the same inputs turns
the tolerance-level GEMM parity into a bit-level statement: bf16 outputs of the tensor-core
GEMMs, the grouped down-projection rows of the routed experts and the fp32 routed sum are
compared bit for bit.

The same library holds the reference's BF16 routed experts of the MTP draft layer
(src/mtp/moe_bf16.cu:271-426, cuBLASLt / GEMV projections): its output pins both the CPU
oracle's restatement of that path and the tensor-core kernels, at the tolerance three bf16
roundings over differently ordered fp32 sums allow.

Skipped where the library was not built (no reference tree at build time) or where cuBLASLt
offers no NVFP4 algorithm."""
import ctypes as C
import importlib
import os

import numpy as np
import pytest
import torch

from gpu_util import bf16_ulp_diff, dev, host
from oracle import oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libq4t_ref_gpu.so")


@pytest.fixture(scope="module")
def ref_gpu(gpu_lib):
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libq4t_ref_gpu.so not built (make -C oracle ref_gpu needs the reference tree)")
    R = C.CDLL(REF_SO)
    R.ref_gpu_last_error.restype = C.c_char_p
    R.ref_gpu_workspace_bytes.restype = C.c_size_t
    R.ref_gpu_workspace_bytes.argtypes = [C.c_int] * 4
    R.ref_gpu_workspace_regions.argtypes = [C.c_int] * 4 + [C.POINTER(C.c_size_t * 4)]
    vp = C.c_void_p
    R.ref_gpu_moe_routed_forward.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int] + [vp] * 8 + [vp] * 4 + \
        [vp, vp, C.c_size_t, C.c_int, C.c_int, vp]
    R.ref_gpu_fp4_gemm.argtypes = [vp, vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, vp,
                                   C.c_size_t, C.POINTER(C.c_int), vp]
    R.ref_gpu_quantize_activation.argtypes = [vp, vp, vp, C.c_int, C.c_int, C.c_float, vp]
    if hasattr(R, "ref_gpu_moe_bf16_routed_forward"):
        R.ref_gpu_moe_bf16_workspace_bytes.restype = C.c_size_t
        R.ref_gpu_moe_bf16_workspace_bytes.argtypes = [C.c_int] * 5
        R.ref_gpu_moe_bf16_routed_forward.argtypes = [vp, vp, vp, vp, C.c_int, C.c_int, C.c_int, vp, vp, vp, vp,
                                                      C.c_size_t, C.c_int, C.c_int, vp]
    return R


@pytest.fixture(scope="module")
def gemm_ws():
    return torch.empty(32 << 20, dtype=torch.uint8, device="cuda")


def _ref_gemm(R, gemm_ws, d, M, N, K, iw, ia, bf16=True):
    out = torch.empty((M, N), dtype=torch.bfloat16 if bf16 else torch.float32, device="cuda")
    algo = C.c_int(0)
    st = R.ref_gpu_fp4_gemm(d[0].data_ptr(), d[1].data_ptr(), d[2].data_ptr(), d[3].data_ptr(), out.data_ptr(),
                            1 if bf16 else 0, M, N, K, iw, ia, gemm_ws.data_ptr(), gemm_ws.numel(), C.byref(algo), None)
    torch.cuda.synchronize()
    if st != 0 or not algo.value:
        pytest.skip(f"cuBLASLt returned no NVFP4 algorithm here (status {st}, has_algo {algo.value})")
    return host(out)


@pytest.mark.parametrize("s,N,K", [(0, 640, 2560), (1, 2560, 640)])
@pytest.mark.parametrize("M", [1, 8, 64, 256])
def test_fp4_gemm_equals_reference_cublaslt(q4t, ref_gpu, gemm_ws, golden, s, N, K, M):
    """The reference's unit-test operands (tests/quant_fp4_test.cpp:367-471) through its own
    Fp4Gemm<uint16_t> (cuBLASLt) and through the tcgen05 kernel: equal bf16 bits."""
    d = [dev(golden[f"gemm{s}_w_packed"]), dev(golden[f"gemm{s}_w_sf_swz"]),
         dev(golden[f"gemm{s}_m{M}_a_packed"]), dev(golden[f"gemm{s}_m{M}_a_sf_swz"])]
    want = _ref_gemm(ref_gpu, gemm_ws, d, M, N, K, 0.29, 0.41)
    got = host(q4t.fp4_gemm(*d, M, N, K, 0.29, 0.41, out_bf16=True))
    ulp = bf16_ulp_diff(got, want)
    n_bad = int((ulp > 0).sum())
    print(f"[vs cuBLASLt {M}x{N}x{K}] bf16 outputs differing: {n_bad} of {ulp.size}, max ulp {ulp.max()}")
    assert n_bad == 0


def test_exact_oracle_equals_reference_cublaslt(q4t, ref_gpu, gemm_ws):
    """The CPU oracle's exact mode (bf16 of the exactly rounded product) against the reference's
    cuBLASLt GEMM: what the reference's audits report, re-measured here."""
    rng = np.random.default_rng(77)
    M, N, K = 96, 1024, 2048
    iw, ia = 0.0137, 0.0019
    w = rng.standard_normal((N, K)).astype(np.float32)
    a = (rng.standard_normal((M, K)) * 3.0).astype(np.float32)
    wp, ws = O.quantize_f32(w, iw)
    ap, as_ = O.quantize_f32(a, ia)
    d = [dev(t) for t in (wp, O.swizzle_sf(ws, N, K), ap, O.swizzle_sf(as_, M, K))]
    want = _ref_gemm(ref_gpu, gemm_ws, d, M, N, K, iw, ia)
    exact = O.f32_to_bf16(O.fp4_gemm(wp, O.swizzle_sf(ws, N, K), ap, O.swizzle_sf(as_, M, K), M, N, K, iw, ia, 1))
    got = host(q4t.fp4_gemm(*d, M, N, K, iw, ia, out_bf16=True))
    print(f"[{M}x{N}x{K}] cuBLASLt vs bf16(exact): {int((want != exact).sum())} differ; tcgen05 kernel vs cuBLASLt: "
          f"{int((got != want).sum())} differ; of {want.size}")
    assert int((want != exact).sum()) == 0
    assert int((got != want).sum()) == 0


def _sorted_rows(a, offsets):
    """Rows of each expert's segment sorted bytewise: the reference fills an expert's rows in the
    order its atomics landed, so segments are compared as sets of rows."""
    out = a.copy()
    for e in range(len(offsets) - 1):
        lo, hi = int(offsets[e]), int(offsets[e + 1])
        if hi - lo > 1:
            seg = out[lo:hi]
            order = np.lexsort(seg.T[::-1])
            out[lo:hi] = seg[order]
    return out


@pytest.mark.parametrize("E,hs,is_,T,k", [(512, 2048, 512, 16, 10), (64, 2560, 640, 40, 10), (32, 1024, 256, 300, 4),
                                          (256, 2560, 640, 1, 10), (256, 2560, 640, 8, 10)])
def test_routed_forward_equals_reference_gpu(q4t, ref_gpu, gemm_ws, E, hs, is_, T, k):
    """MoERoutedForward of the reference (per-expert cuBLASLt loop) and q4t_moe_routed_forward on
    the same seeded layer and routing: the grouped down-projection rows (as per-expert sets of
    rows) and the fp32 routed sum."""
    syn = importlib.import_module("qwen4-thor_b200.synthetic")
    import synth
    dl = syn.device_layer(q4t, E, hs, is_, 128, seed=11 + T)
    x = syn.make_x(T, hs, seed=5 + T)
    ids_h, rw_h = synth.random_routing(T, k, E, seed=T)
    ids, rw = dev(ids_h), dev(rw_h)
    R = T * k
    # reference
    ws = torch.zeros(ref_gpu.ref_gpu_workspace_bytes(T, k, hs, is_) + 256, dtype=torch.uint8, device="cuda")
    y_ref = torch.zeros((T, hs), dtype=torch.float32, device="cuda")
    t = dl.t
    hostf = {n: t[n].cpu().numpy().astype(np.float32) for n in ("gu_w_scale2", "gu_input_scale", "dn_w_scale2", "dn_input_scale")}
    rc = ref_gpu.ref_gpu_moe_routed_forward(
        x.data_ptr(), ids.data_ptr(), rw.data_ptr(), y_ref.data_ptr(), E, hs, is_,
        t["gu_packed"].data_ptr(), t["gu_sf"].data_ptr(), t["dn_packed"].data_ptr(), t["dn_sf"].data_ptr(),
        t["gu_w_scale2"].data_ptr(), t["gu_input_scale"].data_ptr(), t["dn_w_scale2"].data_ptr(),
        t["dn_input_scale"].data_ptr(),
        hostf["gu_w_scale2"].ctypes.data, hostf["gu_input_scale"].ctypes.data, hostf["dn_w_scale2"].ctypes.data,
        hostf["dn_input_scale"].ctypes.data, ws.data_ptr(), gemm_ws.data_ptr(), gemm_ws.numel(), T, k, None)
    torch.cuda.synchronize()
    if rc != 0:
        msg = ref_gpu.ref_gpu_last_error().decode()
        if "algo" in msg.lower() or "cublas" in msg.lower():
            pytest.skip(f"the reference's cuBLASLt path is unavailable here: {msg}")
        raise AssertionError(f"reference MoERoutedForward failed: {msg}")
    reg = (C.c_size_t * 4)()
    ref_gpu.ref_gpu_workspace_regions(T, k, hs, is_, C.byref(reg))
    # Of the reference's workspace only dn_out is a grouped [R, hs] buffer: a_packed, a_sf and
    # gu_out are per-expert scratch that the next expert overwrites (src/quant/moe_gemm.cu:
    # 540-600).  dn_out depends on every earlier stage (input codes and scales, the gate/up
    # GEMM, its bf16 rounding, SwiGLU with the exp intrinsic, requantisation, the down GEMM),
    # so its equality pins the whole chain.
    r_dn = host(ws[reg[3]:reg[3] + R * hs * 2].view(torch.int16)).reshape(R, -1)
    # this library
    rf = q4t.RoutedForward(dl, T, k)
    y = torch.zeros((T, hs), dtype=torch.float32, device="cuda")
    rf(x, ids, rw, y, flags=q4t.FLAG_GENERAL_PATH)
    rf.status()
    offsets = host(rf.region("offsets", torch.int32, E + 1))
    o_dn = host(rf.region("dn_out", torch.int16, R * hs)).reshape(R, -1)
    dn_bad = int((_sorted_rows(o_dn, offsets) != _sorted_rows(r_dn, offsets)).sum())
    y_bad = int((host(y) != host(y_ref)).sum())
    print(f"[vs reference GPU E={E} hs={hs} is={is_} T={T} k={k}] differing from the reference's own GPU code: "
          f"dn_out bf16 values {dn_bad} of {o_dn.size}, routed fp32 values {y_bad} of {y.numel()}")
    assert dn_bad == 0
    assert y_bad == 0
    if T <= 128:
        # the decode-sized path (rows in (token,slot) order) against the same reference output
        fofr = host(rf.region("flat_of_row", torch.int32, R))[:offsets[-1]]
        y2 = torch.zeros((T, hs), dtype=torch.float32, device="cuda")
        rf(x, ids, rw, y2, flags=q4t.FLAG_DECODE_PATH)
        rf.status()
        assert np.array_equal(host(rf.region("row_of_flat", torch.int32, R)), np.arange(R))
        s_dn = host(rf.region("dn_out", torch.int16, R * hs)).reshape(R, -1)[fofr]
        dn_bad = int((_sorted_rows(s_dn, offsets) != _sorted_rows(r_dn, offsets)).sum())
        y_bad = int((host(y2) != host(y_ref)).sum())
        print(f"    decode-sized path: dn_out bf16 values differing {dn_bad}, routed fp32 values differing {y_bad}")
        assert dn_bad == 0 and y_bad == 0


# The reference's own fixture for this path (tests/mtp_moe_path_test.cpp:29-38, 153-170): activations
# ((c*37 + row*113 + 17) mod 509 - 254) / 128, first-row experts and binary-fraction router weights.
_MTP_FIRST_IDS = [37, 3, 91, 7, 211, 19, 401, 23, 127, 53]
_MTP_ROUTER_W = [0.25, 0.125, 0.125, 0.125, 0.0625, 0.0625, 0.0625, 0.0625, 0.0625, 0.0625]


def _mtp_fixture(rows, hs, k, E):
    c = np.arange(hs, dtype=np.int64)[None, :]
    r = np.arange(rows, dtype=np.int64)[:, None]
    x = O.f32_to_bf16((((c * 37 + r * 113 + 17) % 509 - 254).astype(np.float32) / np.float32(128.0)))
    ids = np.empty((rows, k), np.int32)
    ids[0] = _MTP_FIRST_IDS[:k]
    for row in range(1, rows):
        ids[row] = (260 + row * k + np.arange(k)) % E
    rw = np.tile(np.array(_MTP_ROUTER_W[:k], np.float32), (rows, 1))
    return x, ids, rw


@pytest.mark.parametrize("E,hs,is_,T,k,fixture", [(512, 2560, 640, 4, 10, True), (512, 2560, 640, 1, 10, True),
                                                  (64, 1024, 256, 40, 6, False)])
def test_mtp_bf16_experts_vs_reference_gpu(q4t, ref_gpu, gemm_ws, E, hs, is_, T, k, fixture):
    """MoeBf16RoutedForward of the reference, q4t_moe_bf16_routed_forward and the CPU oracle's
    restatement on the same weights and routing."""
    if not hasattr(ref_gpu, "ref_gpu_moe_bf16_routed_forward"):
        pytest.skip("oracle/_ref/libq4t_ref_gpu.so was built without the BF16 experts")
    g = torch.Generator(device="cuda").manual_seed(E + T)
    gu = (torch.randn((E, 2 * is_, hs), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    down = (torch.randn((E, hs, is_), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
    if fixture:
        x_h, ids_h, rw_h = _mtp_fixture(T, hs, k, E)
    else:
        import synth
        x_h = synth.make_x(T, hs, seed=3)
        ids_h, rw_h = synth.random_routing(T, k, E, seed=5)
    x, ids, rw = dev(x_h), dev(ids_h), dev(rw_h)
    # the reference
    ws = torch.zeros(ref_gpu.ref_gpu_moe_bf16_workspace_bytes(T, k, hs, is_, E) + 256, dtype=torch.uint8, device="cuda")
    y_ref = torch.zeros((T, hs), dtype=torch.float32, device="cuda")
    rc = ref_gpu.ref_gpu_moe_bf16_routed_forward(x.data_ptr(), ids.data_ptr(), rw.data_ptr(), y_ref.data_ptr(), E, hs, is_,
                                                 gu.data_ptr(), down.data_ptr(), ws.data_ptr(), gemm_ws.data_ptr(),
                                                 gemm_ws.numel(), T, k, None)
    torch.cuda.synchronize()
    if rc != 0:
        msg = ref_gpu.ref_gpu_last_error().decode()
        if "GEMM failed" in msg:
            pytest.skip(f"the reference's cuBLASLt BF16 path is unavailable here: {msg}")
        raise AssertionError(f"reference MoeBf16RoutedForward failed: {msg}")
    want = host(y_ref)
    # this library
    moe = q4t.Bf16MoE(gu, down, None, T, k)
    y = torch.zeros((T, hs), dtype=torch.float32, device="cuda")
    moe.routed(x, ids, rw, y)
    torch.cuda.synchronize()
    got = host(y)
    # the CPU oracle on the experts that are used (ids renumbered into the compacted set)
    used, inv = np.unique(ids_h, return_inverse=True)
    sel = torch.from_numpy(used.astype(np.int64)).cuda()
    gu_h = host(gu[sel].view(torch.int16)).view(np.uint16)
    down_h = host(down[sel].view(torch.int16)).view(np.uint16)
    orc = O.moe_bf16_routed_forward(x_h, inv.reshape(ids_h.shape).astype(np.int32), rw_h, gu_h, down_h)
    scale = np.abs(want).max()

    def dist(a):
        return float(np.sqrt(((a - want) ** 2).sum() / (want ** 2).sum())), float(np.abs(a - want).max() / scale)

    (l2_k, mx_k), (l2_o, mx_o) = dist(got), dist(orc)
    print(f"[MTP bf16 experts vs reference GPU E={E} hs={hs} is={is_} T={T} k={k}] kernels: relative_l2 {l2_k:.3e} "
          f"max|diff|/max {mx_k:.3e}; CPU oracle: relative_l2 {l2_o:.3e} max|diff|/max {mx_o:.3e}")
    # one bf16 step of the largest output and 0.4 % L2, the bounds of the oracle comparison
    assert l2_k <= 4e-3 and mx_k <= 2.0 ** -7
    assert l2_o <= 4e-3 and mx_o <= 2.0 ** -7
