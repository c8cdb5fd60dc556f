"""CPU tests of the C-ABI library: it loads without a GPU, exports every
symbol the header declares, and its host-only entry points (layout helpers,
expert packer, workspace sizing, argument checks that precede any device
work) behave like the reference's."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib(q4t):
    if not os.path.exists(q4t.LIB_PATH):
        import importlib.util
        spec = importlib.util.spec_from_file_location("q4t_build", os.path.join(ROOT, "qwen4-thor_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    return q4t.load()


def test_exports_match_header(lib, q4t):
    text = open(os.path.join(ROOT, "include", "q4t_moe_b200.h")).read()
    declared = set(re.findall(r"\b(q4t_[a-z0-9_]+)\s*\(", text))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert declared == set(q4t.EXPORTS)


def test_check_library_is_separate(lib, q4t):
    """The device-side checkers the GPU tests use live in their own shared object: the product
    library exports none of them, the companion exports exactly what its header declares."""
    text = open(os.path.join(ROOT, "include", "q4t_moe_b200_check.h")).read()
    declared = set(re.findall(r"\b(q4t_[a-z0-9_]+)\s*\(", text))
    assert declared == set(q4t.CHECK_EXPORTS)
    chk = q4t.load_check()
    for name in declared:
        assert hasattr(chk, name), f"{name} declared in the check header but not exported"
        assert not hasattr(lib, name), f"{name} is test-only and must not be exported by the product library"


def test_sf_helpers_match_oracle(lib):
    for rows, K in [(1, 2560), (8, 640), (129, 640), (640, 2560), (1024, 2048), (2048, 512)]:
        assert lib.q4t_sf_buffer_size(rows, K) == O.sf_buffer_size(rows, K)
        nt = lib.q4t_sf_num_gtiles(K)
        for r in range(0, rows, 13):
            for g in range(0, K // 16, 5):
                assert lib.q4t_sf_offset(r, g, nt) == O.sf_offset(r, g, nt)


def test_pack_expert_host_matches_loader_layout(lib, q4t):
    hs, is_ = 256, 128
    rng = np.random.default_rng(0)
    gate_w = rng.integers(0, 256, (is_, hs // 2), dtype=np.uint8)
    up_w = rng.integers(0, 256, (is_, hs // 2), dtype=np.uint8)
    down_w = rng.integers(0, 256, (hs, is_ // 2), dtype=np.uint8)
    gate_s = rng.integers(0, 127, (is_, hs // 16), dtype=np.uint8)
    up_s = rng.integers(0, 127, (is_, hs // 16), dtype=np.uint8)
    down_s = rng.integers(0, 127, (hs, is_ // 16), dtype=np.uint8)
    gu_p = np.zeros((2 * is_, hs // 2), np.uint8)
    dn_p = np.zeros((hs, is_ // 2), np.uint8)
    gu_sf = np.full(O.sf_buffer_size(2 * is_, hs), 0xAA, np.uint8)
    dn_sf = np.full(O.sf_buffer_size(hs, is_), 0xAA, np.uint8)
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    rc = lib.q4t_pack_expert_host(p(gate_w), p(up_w), p(down_w), p(gate_s), p(up_s), p(down_s), hs, is_,
                                  p(gu_p), p(gu_sf), p(dn_p), p(dn_sf))
    assert rc == 0
    # codes unchanged, gate rows then up rows (src/quant/moe_weights.cpp:176-190 of the reference)
    assert np.array_equal(gu_p, np.concatenate([gate_w, up_w]))
    assert np.array_equal(dn_p, down_w)
    # scales: gate|up concatenated, then swizzled; down swizzled (moe_weights.cpp:222-226)
    assert np.array_equal(gu_sf, O.swizzle_sf(np.concatenate([gate_s, up_s]), 2 * is_, hs))
    assert np.array_equal(dn_sf, O.swizzle_sf(down_s, hs, is_))
    assert np.array_equal(O.unswizzle_sf(gu_sf, 2 * is_, hs)[is_:], up_s)
    # divisibility rules of the loader (moe_weights.cpp:49-57)
    assert lib.q4t_pack_expert_host(p(gate_w), p(up_w), p(down_w), p(gate_s), p(up_s), p(down_s), 200, is_,
                                    p(gu_p), p(gu_sf), p(dn_p), p(dn_sf)) != 0
    assert b"multiples of" in lib.q4t_last_error()


def test_workspace_sizes(lib, q4t):
    # the four reference regions keep the reference's order and sizes
    M, k, hs, is_, E = 16, 10, 2048, 512, 512
    L = q4t.routed_ws_layout(M, k, hs, is_, E)
    R = M * k
    assert L.a_packed == 0
    assert L.a_sf == R * hs // 2
    assert L.gu_out == L.a_sf + O.sf_buffer_size(R, hs)
    assert L.dn_out == L.gu_out + R * 2 * is_ * 2
    ref_total = 163840 + 32768 + 327680 + 655360   # reference RequiredBytes at these dims
    assert L.dn_out + R * hs * 2 == ref_total
    assert L.total >= ref_total
    assert lib.q4t_moe_routed_workspace_bytes(M, k, hs, is_, E) == L.total
    F = q4t.forward_ws_layout(M, k, hs, is_, 512, E)
    assert F.routed_ws == 0 and F.logits >= L.total
    order = [F.logits, F.expert_ids, F.router_w, F.routed, F.shared_gu, F.shared_act, F.shared_down, F.total]
    assert order == sorted(order)
    assert lib.q4t_moe_forward_workspace_bytes(M, k, hs, is_, 512, E) == F.total
    assert lib.q4t_moe_routed_workspace_bytes(0, k, hs, is_, E) == 0


def test_argument_errors_before_device_work(lib, q4t):
    rw = q4t.RoutedWeights(512, 2048, 512, 0)
    ex = q4t.ExtraWeights(512, 2048, 512)
    dummy = C.c_void_p(256)
    # T <= 0 is a no-op (src/model/moe.cu:442)
    assert lib.q4t_moe_forward(dummy, C.byref(rw), C.byref(ex), dummy, 0, 10, dummy, 0, None, 0, None) == 0
    # k out of range (moe.cu:443)
    assert lib.q4t_moe_forward(dummy, C.byref(rw), C.byref(ex), dummy, 2, 17, dummy, 1 << 30, None, 0, None) != 0
    assert lib.q4t_last_error() == b"k out of range"
    # workspace too small (moe.cu:444-447)
    assert lib.q4t_moe_forward(dummy, C.byref(rw), C.byref(ex), dummy, 2, 10, dummy, 1024, None, 0, None) != 0
    assert lib.q4t_last_error() == b"workspace too small"
    # invalid dims (src/quant/moe_gemm.cu:321-323)
    assert lib.q4t_moe_routed_forward(dummy, dummy, dummy, dummy, C.byref(rw), dummy, 1 << 30, 0, 10, 0, None) != 0
    assert lib.q4t_last_error() == b"invalid MoE forward dims"
    assert lib.q4t_router_topk(dummy, dummy, dummy, 4, 512, 17, None) != 0
    assert lib.q4t_last_error() == b"k out of range"
    assert lib.q4t_quantize_activation_fp4(dummy, dummy, dummy, 4, 40, 1.0, None) != 0


def test_ep_sync_entry_points_check_arguments(lib, q4t):
    """The collective-free exchange of the expert-parallel step: sizing and the argument checks
    that precede any device work."""
    assert lib.q4t_ep_sync_buffer_bytes(8, 4096, 10) == 256 + 8 * 4096 * 10 * 4
    assert lib.q4t_ep_sync_buffer_bytes(9, 4096, 10) == 0 and lib.q4t_ep_sync_buffer_bytes(2, 0, 10) == 0
    table = q4t.EpPeerTable()
    table.world, table.rank, table.tokens_per_rank = 2, 0, 8
    assert lib.q4t_ep_wait(C.byref(table), 0, 1, None) != 0
    assert lib.q4t_last_error() == b"peer table has no sync buffers"
    assert lib.q4t_ep_post_rows(C.byref(table), 1, None) != 0
    assert lib.q4t_ep_post_ids(None, C.byref(table), 2, 1, None) != 0
    table.world = 9
    assert lib.q4t_ep_sync_status(C.byref(table)) != 0
    assert b"invalid peer table" in lib.q4t_last_error()
