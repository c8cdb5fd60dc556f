"""Python binding of libq4t_moe_b200.so (C ABI in include/q4t_moe_b200.h).

PyTorch is used only for plumbing: device buffers, streams and (in the
benchmark) torch.distributed.  Every compute call goes through the C ABI into
the hand-written sm_100a kernels; there is no eager/PyTorch fallback, and the
calls raise if the shared library or a B200-class device is missing.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("Q4T_LIB_PATH", os.path.join(_HERE, "libq4t_moe_b200.so"))


class Q4TError(RuntimeError):
    pass


class RoutedWeights(C.Structure):
    """q4t_routed_weights: POD image of MoEWeightLayout."""
    _fields_ = [("E", C.c_int32), ("hs", C.c_int32), ("moe_is", C.c_int32), ("slot_mode", C.c_int32),
                ("gu_packed", C.c_void_p), ("gu_sf", C.c_void_p), ("dn_packed", C.c_void_p),
                ("dn_sf", C.c_void_p), ("gu_w_scale2", C.c_void_p), ("gu_input_scale", C.c_void_p),
                ("dn_w_scale2", C.c_void_p), ("dn_input_scale", C.c_void_p),
                ("gu_input_scale_uniform", C.c_float), ("reserved", C.c_int32)]


class ExtraWeights(C.Structure):
    """q4t_extra_weights: POD image of MoEExtraWeights."""
    _fields_ = [("E", C.c_int32), ("hs", C.c_int32), ("shared_is", C.c_int32),
                ("gate", C.c_void_p), ("shared_gu", C.c_void_p), ("shared_down", C.c_void_p),
                ("shared_gate_scalar", C.c_void_p)]


class RoutedWsLayout(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in (
        "a_packed", "a_sf", "gu_out", "dn_out", "counts", "offsets", "row_of_flat", "flat_of_row",
        "row_tile", "ntiles", "tile_expert", "tile_row0", "tile_nrows", "a_sf_tiles", "xq_packed", "xq_sf", "inter_packed",
        "inter_sf_tiles", "status", "max_tiles", "total")]


class Bf16ExpertWeights(C.Structure):
    """q4t_bf16_expert_weights: the MTP draft layer's BF16 routed experts."""
    _fields_ = [("E", C.c_int32), ("hs", C.c_int32), ("moe_is", C.c_int32), ("reserved", C.c_int32),
                ("gu", C.c_void_p), ("down", C.c_void_p)]


class EpPeerTable(C.Structure):
    """q4t_ep_peer_table: who publishes what, for the pull/push expert-parallel path."""
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("tokens_per_rank", C.c_int32),
                ("expert_map", C.c_int32), ("xq_packed", C.c_void_p * 8), ("xq_sf", C.c_void_p * 8),
                ("dn_rows", C.c_void_p * 8), ("placement", C.c_void_p), ("experts_total", C.c_int32),
                ("reserved", C.c_int32), ("expert_owner", C.c_void_p), ("sync", C.c_void_p * 8)]


class ForwardWsLayout(C.Structure):
    _fields_ = [(n, C.c_size_t) for n in (
        "routed_ws", "logits", "expert_ids", "router_w", "routed", "shared_gu", "shared_act",
        "shared_down", "slot_ids", "total")]


class ForwardOptions(C.Structure):
    """q4t_forward_options: the replay table, the router-trace observer and the slot-mode table."""
    _fields_ = [("fixed_ids", C.c_void_p), ("trace_ids_out", C.c_void_p), ("slot_of_expert", C.c_void_p),
                ("flags", C.c_uint32), ("hc_count", C.c_int32), ("hc_residual", C.c_void_p),
                ("hc_inject_gate", C.c_void_p), ("hc_out", C.c_void_p), ("norm_residual", C.c_void_p),
                ("norm_out", C.c_void_p), ("norm_eps", C.c_float)]


EXPORTS = [
    "q4t_last_error", "q4t_version", "q4t_set_pair_min_rows", "q4t_sf_num_gtiles", "q4t_sf_buffer_size", "q4t_sf_offset",
    "q4t_pack_expert_host", "q4t_quantize_activation_fp4", "q4t_dequant_fp4_to_bf16", "q4t_fp4_gemm",
    "q4t_router_topk", "q4t_bf16_linear", "q4t_moe_routed_workspace_bytes",
    "q4t_moe_routed_workspace_layout", "q4t_moe_routed_forward", "q4t_moe_forward_workspace_bytes",
    "q4t_moe_forward_workspace_layout", "q4t_moe_forward", "q4t_moe_forward_ex", "q4t_moe_workspace_status",
    "q4t_moe_noalloc_status",
    "q4t_stage_timing_enable", "q4t_stage_timing_read",
    "q4t_moe_routed_forward_noalloc", "q4t_ep_dispatch_workspace_bytes", "q4t_ep_dispatch",
    "q4t_moe_expert_rows", "q4t_moe_finish_workspace_bytes", "q4t_moe_finish",
    "q4t_moe_shared_expert", "q4t_moe_combine", "q4t_residual_rmsnorm_bf16",
    "q4t_moe_bf16_workspace_bytes", "q4t_moe_bf16_routed_forward", "q4t_moe_bf16_forward_workspace_bytes",
    "q4t_moe_bf16_forward",
    "q4t_peer_buffer_alloc", "q4t_peer_buffer_free", "q4t_peer_buffer_export", "q4t_peer_buffer_open",
    "q4t_peer_buffer_close", "q4t_ep_publish", "q4t_ep_publish_selected", "q4t_ep_route_publish", "q4t_ep_combine", "q4t_moe_expert_peer_workspace_bytes", "q4t_moe_expert_peer", "q4t_ep_flat_rows",
    "q4t_ep_sync_buffer_bytes", "q4t_ep_post_ids", "q4t_ep_post_rows", "q4t_ep_wait", "q4t_ep_sync_status",
]
# libq4t_moe_b200_check.so (include/q4t_moe_b200_check.h): device-side checkers for the GPU tests only.
CHECK_EXPORTS = ["q4t_check_last_error", "q4t_fp4_gemm_check", "q4t_selftest_encoders"]
CHECK_LIB_PATH = os.path.join(_HERE, "libq4t_moe_b200_check.so")
# q4t_moe_forward / q4t_moe_routed_forward flags
FLAG_DUMP_GATE_UP = 1      # materialise the bf16 gate|up projections
FLAG_ROUTED_F32 = 2        # materialise the fp32 routed sum (q4t_moe_forward)
FLAG_GENERAL_PATH = 4      # decode-sized batches (at most 64 tokens): take the grouped path of larger batches anyway
FLAG_DECODE_PATH = 8       # take the decode-sized path up to its limit of 128 tokens
EP_MAX_RANKS = 8
PEER_HANDLE_BYTES = 64
EP_SYNC_IDS_OFFSET = 256
EP_REPLICATED = 1 << 30
NOALLOC_SCRATCH_BYTES = 3 << 20

_lib = None


def load():
    """Loads the shared library (no device needed for this step)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise Q4TError(f"{LIB_PATH} is missing: build it with `python qwen4-thor_b200/build.py` "
                       "(there is no fallback path)")
    L = C.CDLL(LIB_PATH)
    L.q4t_last_error.restype = C.c_char_p
    L.q4t_version.restype = C.c_char_p
    L.q4t_set_pair_min_rows.argtypes = [C.c_int64]
    L.q4t_sf_num_gtiles.restype = C.c_int32
    L.q4t_sf_buffer_size.restype = C.c_size_t
    L.q4t_sf_buffer_size.argtypes = [C.c_int32, C.c_int32]
    L.q4t_sf_offset.restype = C.c_size_t
    L.q4t_sf_offset.argtypes = [C.c_int32, C.c_int32, C.c_int32]
    L.q4t_moe_routed_workspace_bytes.restype = C.c_size_t
    L.q4t_moe_routed_workspace_bytes.argtypes = [C.c_int32] * 5
    L.q4t_moe_forward_workspace_bytes.restype = C.c_size_t
    L.q4t_moe_forward_workspace_bytes.argtypes = [C.c_int32] * 6
    vp, i32, f32, u32, sz = C.c_void_p, C.c_int32, C.c_float, C.c_uint32, C.c_size_t
    L.q4t_pack_expert_host.argtypes = [vp] * 6 + [i32, i32] + [vp] * 4
    L.q4t_quantize_activation_fp4.argtypes = [vp, vp, vp, i32, i32, f32, vp]
    L.q4t_dequant_fp4_to_bf16.argtypes = [vp, vp, vp, f32, i32, i32, vp]
    L.q4t_fp4_gemm.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, f32, f32, vp]
    L.q4t_router_topk.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    L.q4t_bf16_linear.argtypes = [vp, vp, vp, i32, i32, i32, vp]
    L.q4t_moe_routed_workspace_layout.argtypes = [i32] * 5 + [C.POINTER(RoutedWsLayout)]
    L.q4t_moe_routed_forward.argtypes = [vp, vp, vp, vp, C.POINTER(RoutedWeights), vp, sz, i32, i32, u32, vp]
    L.q4t_moe_routed_forward_noalloc.argtypes = [vp, vp, vp, vp, C.POINTER(RoutedWeights), i32, i32, u32, vp]
    L.q4t_ep_dispatch_workspace_bytes.restype = C.c_size_t
    L.q4t_ep_dispatch_workspace_bytes.argtypes = [i32, i32, i32]
    L.q4t_ep_dispatch.argtypes = [vp, vp, i32, i32, i32, i32, i32, vp, vp, vp, vp, vp, sz, vp]
    L.q4t_moe_expert_rows.argtypes = [vp, vp, vp, C.POINTER(RoutedWeights), vp, sz, i32, u32, vp]
    L.q4t_moe_finish_workspace_bytes.restype = C.c_size_t
    L.q4t_moe_finish_workspace_bytes.argtypes = [i32, i32, i32]
    L.q4t_moe_finish.argtypes = [vp, vp, vp, vp, C.POINTER(ExtraWeights), vp, i32, i32, vp, sz, vp]
    L.q4t_peer_buffer_alloc.argtypes = [sz, C.POINTER(C.c_void_p)]
    L.q4t_peer_buffer_free.argtypes = [vp]
    L.q4t_peer_buffer_export.argtypes = [vp, C.c_char_p]
    L.q4t_peer_buffer_open.argtypes = [C.c_char_p, C.POINTER(C.c_void_p)]
    L.q4t_peer_buffer_close.argtypes = [vp]
    L.q4t_moe_shared_expert.argtypes = [vp, C.POINTER(ExtraWeights), i32, vp, sz, vp]
    L.q4t_moe_combine.argtypes = [vp, vp, vp, vp, C.POINTER(ExtraWeights), vp, i32, i32, vp, sz, vp]
    L.q4t_moe_bf16_workspace_bytes.restype = C.c_size_t
    L.q4t_moe_bf16_workspace_bytes.argtypes = [i32] * 5
    L.q4t_moe_bf16_forward_workspace_bytes.restype = C.c_size_t
    L.q4t_moe_bf16_forward_workspace_bytes.argtypes = [i32] * 6
    L.q4t_moe_bf16_routed_forward.argtypes = [vp, vp, vp, vp, C.POINTER(Bf16ExpertWeights), vp, sz, i32, i32, vp]
    L.q4t_moe_bf16_forward.argtypes = [vp, C.POINTER(Bf16ExpertWeights), C.POINTER(ExtraWeights), vp, i32, i32, vp, sz,
                                       vp]
    L.q4t_residual_rmsnorm_bf16.argtypes = [vp, vp, vp, i32, i32, f32, vp]
    L.q4t_ep_route_publish.argtypes = [vp, C.POINTER(ExtraWeights), C.POINTER(EpPeerTable), i32, f32, vp, vp, vp, vp,
                                       sz, vp]
    L.q4t_ep_combine.argtypes = [vp, vp, vp, vp, C.POINTER(ExtraWeights), vp, i32, i32, vp, vp, sz, vp]
    L.q4t_ep_publish.argtypes = [vp, C.POINTER(EpPeerTable), i32, f32, vp]
    L.q4t_ep_publish_selected.argtypes = [vp, vp, C.POINTER(EpPeerTable), i32, i32, i32, f32, vp]
    L.q4t_ep_sync_buffer_bytes.restype = sz
    L.q4t_ep_sync_buffer_bytes.argtypes = [i32, i32, i32]
    L.q4t_ep_post_ids.argtypes = [vp, C.POINTER(EpPeerTable), i32, u32, vp]
    L.q4t_ep_post_rows.argtypes = [C.POINTER(EpPeerTable), u32, vp]
    L.q4t_ep_wait.argtypes = [C.POINTER(EpPeerTable), i32, u32, vp]
    L.q4t_ep_sync_status.argtypes = [C.POINTER(EpPeerTable)]
    L.q4t_moe_expert_peer_workspace_bytes.restype = C.c_size_t
    L.q4t_moe_expert_peer_workspace_bytes.argtypes = [i32] * 5
    L.q4t_moe_expert_peer.argtypes = [vp, C.POINTER(EpPeerTable), C.POINTER(RoutedWeights), i32, vp, sz, u32, vp]
    L.q4t_ep_flat_rows.argtypes = [vp, i32, i32, vp, vp]
    L.q4t_moe_forward_workspace_layout.argtypes = [i32] * 6 + [C.POINTER(ForwardWsLayout)]
    L.q4t_moe_forward.argtypes = [vp, C.POINTER(RoutedWeights), C.POINTER(ExtraWeights), vp, i32, i32,
                                  vp, sz, vp, u32, vp]
    L.q4t_moe_forward_ex.argtypes = [vp, C.POINTER(RoutedWeights), C.POINTER(ExtraWeights), vp, i32, i32,
                                     vp, sz, C.POINTER(ForwardOptions), vp]
    L.q4t_moe_workspace_status.argtypes = [vp, i32, i32, i32, i32, i32]
    L.q4t_moe_noalloc_status.argtypes = [i32] * 5
    _lib = L
    return L


_check_lib = None


def load_check():
    """Loads the test-only companion library (exact CUDA-core GEMM, encoder sweeps)."""
    global _check_lib
    if _check_lib is None:
        if not os.path.exists(CHECK_LIB_PATH):
            raise Q4TError(f"{CHECK_LIB_PATH} is missing: build it with `python qwen4-thor_b200/build.py`")
        L = C.CDLL(CHECK_LIB_PATH)
        vp, i32, f32 = C.c_void_p, C.c_int32, C.c_float
        L.q4t_check_last_error.restype = C.c_char_p
        L.q4t_fp4_gemm_check.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, f32, f32, vp]
        L.q4t_selftest_encoders.argtypes = [i32, C.c_uint64, C.c_uint64, C.POINTER(C.c_uint64),
                                            C.POINTER(C.c_uint32), vp]
        _check_lib = L
    return _check_lib


def _check_rc(rc: int) -> None:
    if rc != 0:
        raise Q4TError(f"[{rc}] {load_check().q4t_check_last_error().decode()}")


def check(rc: int) -> None:
    if rc != 0:
        raise Q4TError(f"[{rc}] {load().q4t_last_error().decode()}")


def _stream_ptr(stream=None):
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


# --------------------------------------------------------------------- layouts
def routed_ws_layout(M, k, hs, moe_is, E) -> RoutedWsLayout:
    L = RoutedWsLayout()
    check(load().q4t_moe_routed_workspace_layout(M, k, hs, moe_is, E, C.byref(L)))
    return L


def forward_ws_layout(T, k, hs, moe_is, shared_is, E) -> ForwardWsLayout:
    F = ForwardWsLayout()
    check(load().q4t_moe_forward_workspace_layout(T, k, hs, moe_is, shared_is, E, C.byref(F)))
    return F


# ------------------------------------------------------------- device weights
class DeviceLayer:
    """One MoE layer resident in HBM, in the reference's device layout.

    Built from any object with the oracle Layer's attributes (numpy arrays) or
    directly from torch CUDA tensors."""

    ROUTED = ("gu_packed", "gu_sf", "dn_packed", "dn_sf", "gu_w_scale2", "gu_input_scale",
              "dn_w_scale2", "dn_input_scale")
    EXTRA = ("gate", "shared_gu", "shared_down", "shared_gate_scalar")

    def __init__(self, E, hs, moe_is, shared_is, tensors: dict, E_router=None):
        """E_router: experts the router chooses among when this object holds only some of
        them (one rank of an expert-parallel layer); defaults to E."""
        self.E, self.hs, self.moe_is, self.shared_is = E, hs, moe_is, shared_is
        self.E_router = E if E_router is None else E_router
        self.t = tensors  # keeps the device buffers alive
        gis = tensors.get("gu_input_scale")
        uniform = 0.0
        if gis is not None and gis.numel() > 0:   # one host read at construction time
            lo, hi = float(gis.min()), float(gis.max())
            uniform = lo if lo == hi and lo > 0 else 0.0
        self.routed = RoutedWeights(E, hs, moe_is, 0, *[self._p(n) for n in self.ROUTED], uniform, 0)
        self.extra = ExtraWeights(self.E_router, hs, shared_is, *[self._p(n) for n in self.EXTRA])

    def _p(self, name):
        t = self.t.get(name)
        return None if t is None else t.data_ptr()

    @classmethod
    def from_host(cls, layer, device="cuda"):
        import numpy as np
        import torch
        tensors = {}
        for n in cls.ROUTED + cls.EXTRA:
            a = getattr(layer, n, None)
            if a is None:
                continue
            if a.dtype == np.uint16:   # bf16 bit patterns
                tensors[n] = torch.from_numpy(a.view(np.int16)).to(device)
            else:
                tensors[n] = torch.from_numpy(a).to(device)
        return cls(layer.E, layer.hs, layer.moe_is, layer.shared_is, tensors)


# ------------------------------------------------------------------ operators
def quantize_activation_fp4(x_bf16, global_scale: float, stream=None):
    """x: CUDA tensor [M, K] of bf16 (torch.bfloat16 or int16 bit patterns)."""
    import torch
    M, K = x_bf16.shape
    packed = torch.empty((M, K // 2), dtype=torch.uint8, device=x_bf16.device)
    sf = torch.zeros(load().q4t_sf_buffer_size(M, K), dtype=torch.uint8, device=x_bf16.device)
    check(load().q4t_quantize_activation_fp4(_ptr(x_bf16), _ptr(packed), _ptr(sf), M, K,
                                             float(global_scale), _stream_ptr(stream)))
    return packed, sf


def dequant_fp4_to_bf16(packed, group_scale, inv_global: float, stream=None):
    import torch
    N, K2 = packed.shape
    out = torch.empty((N, K2 * 2), dtype=torch.bfloat16, device=packed.device)
    check(load().q4t_dequant_fp4_to_bf16(_ptr(packed), _ptr(group_scale), _ptr(out), float(inv_global),
                                         N, K2 * 2, _stream_ptr(stream)))
    return out


def fp4_gemm(w_packed, w_sf, a_packed, a_sf, M, N, K, inv_w, inv_a, out_bf16=False, check_kernel=False,
             stream=None):
    import torch
    dt = torch.bfloat16 if out_bf16 else torch.float32
    out = torch.empty((M, N), dtype=dt, device=w_packed.device)
    if check_kernel:
        _check_rc(load_check().q4t_fp4_gemm_check(_ptr(w_packed), _ptr(w_sf), _ptr(a_packed), _ptr(a_sf),
                                                  _ptr(out), M, N, K, float(inv_w), float(inv_a),
                                                  _stream_ptr(stream)))
    else:
        check(load().q4t_fp4_gemm(_ptr(w_packed), _ptr(w_sf), _ptr(a_packed), _ptr(a_sf), _ptr(out),
                                  1 if out_bf16 else 0, M, N, K, float(inv_w), float(inv_a),
                                  _stream_ptr(stream)))
    return out


def router_topk(logits_bf16, k: int, stream=None):
    import torch
    T, E = logits_bf16.shape
    ids = torch.empty((T, k), dtype=torch.int32, device=logits_bf16.device)
    w = torch.empty((T, k), dtype=torch.float32, device=logits_bf16.device)
    check(load().q4t_router_topk(_ptr(logits_bf16), _ptr(ids), _ptr(w), T, E, k, _stream_ptr(stream)))
    return ids, w


def bf16_linear(x, w, stream=None):
    import torch
    M, K = x.shape
    N = w.shape[0]
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    check(load().q4t_bf16_linear(_ptr(x), _ptr(w), _ptr(y), M, N, K, _stream_ptr(stream)))
    return y


class RoutedForward:
    """MoERoutedForward with a caller-owned workspace (allocated once here)."""

    def __init__(self, layer: DeviceLayer, M: int, k: int, device="cuda"):
        import torch
        self.layer, self.M, self.k = layer, M, k
        self.layout = routed_ws_layout(M, k, layer.hs, layer.moe_is, layer.E)
        self.ws = torch.empty(self.layout.total, dtype=torch.uint8, device=device)

    def __call__(self, x, ids, rw, y, flags=0, stream=None):
        check(load().q4t_moe_routed_forward(_ptr(x), _ptr(ids), _ptr(rw), _ptr(y), C.byref(self.layer.routed),
                                            _ptr(self.ws), self.layout.total, self.M, self.k, flags,
                                            _stream_ptr(stream)))
        return y

    def region(self, name, dtype, count):
        import torch
        off = getattr(self.layout, name)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        return self.ws[off:off + nbytes].view(dtype)

    def status(self):
        import torch
        torch.cuda.synchronize()
        check(load().q4t_moe_workspace_status(_ptr(self.ws), self.M, self.k, self.layer.hs,
                                              self.layer.moe_is, self.layer.E))


def routed_forward_noalloc(layer: DeviceLayer, x, ids, rw, y, flags=0, stream=None):
    """MoERoutedForward on the library's built-in scratch: no workspace, no
    device allocation.  Small batches only (see NOALLOC_SCRATCH_BYTES)."""
    M, k = ids.shape
    check(load().q4t_moe_routed_forward_noalloc(_ptr(x), _ptr(ids), _ptr(rw), _ptr(y), C.byref(layer.routed),
                                                M, k, flags, _stream_ptr(stream)))
    return y


def noalloc_status(layer: DeviceLayer, M: int, k: int):
    """Raises if a bounded device-side wait ran out during the last no-allocation call of
    these dimensions (synchronises the device first)."""
    import torch
    torch.cuda.synchronize()
    check(load().q4t_moe_noalloc_status(M, k, layer.hs, layer.moe_is, layer.E))


class MoEForward:
    """MoEForward (router + routed experts + shared expert + gated combine)."""

    def __init__(self, layer: DeviceLayer, T: int, k: int, device="cuda"):
        import torch
        self.layer, self.T, self.k = layer, T, k
        # the workspace is sized by the experts the router chooses among (more than layer.E in slot mode)
        self.layout = forward_ws_layout(T, k, layer.hs, layer.moe_is, layer.shared_is, layer.E_router)
        self.routed_layout = routed_ws_layout(T, k, layer.hs, layer.moe_is, layer.E_router)
        self.ws = torch.empty(self.layout.total, dtype=torch.uint8, device=device)

    def __call__(self, x, y, fixed_ids=None, flags=0, stream=None, trace_ids_out=None, slot_of_expert=None,
                 hc_write=None, norm_write=None):
        """trace_ids_out: CUDA int32 [T,k] that receives the selected expert ids (the router-trace
        observer); slot_of_expert: CUDA int32 [E] expert -> resident slot table (slot mode: the
        layer's routed weights then hold layer.E slots, the router chooses among layer.E_router);
        hc_write: (residual bf16 [T, hc*hs], inject_gate bf16 [T, hc], out bf16 [T, hc*hs]), the
        layer's gated residual write fused into the final combine; norm_write: (residual bf16 [T, hs]
        read and written, out bf16 [T, hs], eps): residual <- bf16(residual + y), out <- RMSNorm(residual),
        the step between two layers of a stack fused into the final combine."""
        if trace_ids_out is None and slot_of_expert is None and hc_write is None and norm_write is None:
            check(load().q4t_moe_forward(_ptr(x), C.byref(self.layer.routed), C.byref(self.layer.extra), _ptr(y),
                                         self.T, self.k, _ptr(self.ws), self.layout.total, _ptr(fixed_ids),
                                         flags, _stream_ptr(stream)))
            return y
        hc, res, gate, out = 0, None, None, None
        if hc_write is not None:
            res, gate, out = hc_write
            hc = gate.shape[1]
        nres, nout, neps = norm_write if norm_write is not None else (None, None, 0.0)
        opt = ForwardOptions(_ptr(fixed_ids), _ptr(trace_ids_out), _ptr(slot_of_expert), flags, hc, _ptr(res),
                             _ptr(gate), _ptr(out), _ptr(nres), _ptr(nout), float(neps))
        check(load().q4t_moe_forward_ex(_ptr(x), C.byref(self.layer.routed), C.byref(self.layer.extra), _ptr(y),
                                        self.T, self.k, _ptr(self.ws), self.layout.total, C.byref(opt),
                                        _stream_ptr(stream)))
        return y

    def region(self, name, dtype, count):
        import torch
        off = getattr(self.layout, name)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        return self.ws[off:off + nbytes].view(dtype)

    def routed_region(self, name, dtype, count):
        import torch
        off = self.layout.routed_ws + getattr(self.routed_layout, name)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        return self.ws[off:off + nbytes].view(dtype)

    def status(self):
        import torch
        torch.cuda.synchronize()
        ws = self.ws[self.layout.routed_ws:]
        check(load().q4t_moe_workspace_status(_ptr(ws), self.T, self.k, self.layer.hs, self.layer.moe_is,
                                              self.layer.E_router))


STAGES = ("router_logits", "topk", "permutation", "gather_quantise", "gate_up_gemm", "down_gemm",
          "shared_expert", "combine")


class Bf16MoE:
    """The MTP draft layer's MoE: BF16 routed experts (gu [E, 2*moe_is, hs], down [E, hs, moe_is],
    CUDA bf16 tensors) with the router and shared expert of `extra_layer` (a DeviceLayer whose
    EXTRA tensors are set)."""

    def __init__(self, gu, down, extra_layer, T: int, k: int, device="cuda"):
        import torch
        E, two_is, hs = gu.shape
        self.gu, self.down, self.extra_layer, self.T, self.k = gu, down, extra_layer, T, k
        self.E, self.hs, self.moe_is = E, hs, two_is // 2
        self.w = Bf16ExpertWeights(E, hs, self.moe_is, 0, gu.data_ptr(), down.data_ptr())
        lib = load()
        self.routed_bytes = lib.q4t_moe_bf16_workspace_bytes(T, k, hs, self.moe_is, E)
        sis = extra_layer.shared_is if extra_layer is not None else 128
        self.forward_bytes = lib.q4t_moe_bf16_forward_workspace_bytes(T, k, hs, self.moe_is, sis, E)
        self.ws = torch.empty(max(self.routed_bytes, self.forward_bytes), dtype=torch.uint8, device=device)

    def routed(self, x, ids, rw, y, stream=None):
        check(load().q4t_moe_bf16_routed_forward(_ptr(x), _ptr(ids), _ptr(rw), _ptr(y), C.byref(self.w), _ptr(self.ws),
                                                 self.ws.numel(), self.T, self.k, _stream_ptr(stream)))
        return y

    def forward(self, x, y, stream=None):
        check(load().q4t_moe_bf16_forward(_ptr(x), C.byref(self.w), C.byref(self.extra_layer.extra), _ptr(y), self.T,
                                          self.k, _ptr(self.ws), self.ws.numel(), _stream_ptr(stream)))
        return y


def residual_rmsnorm(x, y, h, eps: float = 1e-6, stream=None):
    """x <- bf16(x + y) in place (y may be None), h <- RMSNorm(x): the step between two
    layers of a decode stack.  x, y, h: CUDA bf16 [T, hs]."""
    T, hs = x.shape
    check(load().q4t_residual_rmsnorm_bf16(_ptr(x), _ptr(y), _ptr(h), T, hs, float(eps), _stream_ptr(stream)))
    return h


class DecodeStack:
    """L MoE layers applied as x <- bf16(x + MoE_l(RMSNorm(x))), the decode-stack harness
    (eps 1e-6, no norm weight).  One workspace is shared by all layers."""

    def __init__(self, layers, T: int, k: int, eps: float = 1e-6, device="cuda", fused: bool = True):
        import torch
        self.layers, self.T, self.k, self.eps, self.fused = layers, T, k, eps, fused
        self.fwd = MoEForward(layers[0], T, k, device)
        hs = layers[0].hs
        self.h = torch.empty((T, hs), dtype=torch.bfloat16, device=device)
        self.h2 = torch.empty((T, hs), dtype=torch.bfloat16, device=device)
        self.y = torch.empty((T, hs), dtype=torch.bfloat16, device=device)

    def __call__(self, x, stream=None):
        """Runs the stack in place on x (bf16 [T, hs]); returns x.  fused (default): one residual +
        RMSNorm launch in front of the first layer, after that every layer's combine adds its output
        to x and writes the next layer's normalised input itself (same bits either way)."""
        L = load()
        sp = _stream_ptr(stream)
        fw = self.fwd
        if self.fused:
            check(L.q4t_residual_rmsnorm_bf16(_ptr(x), None, _ptr(self.h), self.T, self.layers[0].hs, float(self.eps), sp))
            h_in, h_out = self.h, self.h2
            for layer in self.layers:
                opt = ForwardOptions(None, None, None, 0, 0, None, None, None, _ptr(x), _ptr(h_out), float(self.eps))
                check(L.q4t_moe_forward_ex(_ptr(h_in), C.byref(layer.routed), C.byref(layer.extra), _ptr(self.y), self.T,
                                           self.k, _ptr(fw.ws), fw.ws.numel(), C.byref(opt), sp))
                h_in, h_out = h_out, h_in
            return x
        for i, layer in enumerate(self.layers):
            check(L.q4t_residual_rmsnorm_bf16(_ptr(x), _ptr(self.y) if i else None, _ptr(self.h), self.T,
                                              layer.hs, float(self.eps), sp))
            check(L.q4t_moe_forward(_ptr(self.h), C.byref(layer.routed), C.byref(layer.extra), _ptr(self.y), self.T,
                                    self.k, _ptr(fw.ws), fw.ws.numel(), None, 0, sp))
        # the last layer's output joins the residual stream
        check(L.q4t_residual_rmsnorm_bf16(_ptr(x), _ptr(self.y), _ptr(self.h), self.T, self.layers[0].hs,
                                          float(self.eps), sp))
        return x


def stage_timing(enable: bool) -> None:
    check(load().q4t_stage_timing_enable(1 if enable else 0))


def stage_timing_read() -> dict:
    ms = (C.c_float * len(STAGES))()
    check(load().q4t_stage_timing_read(ms))
    return dict(zip(STAGES, [float(v) for v in ms]))


def selftest_encoders(which: int, first: int, count: int):
    m = C.c_uint64(0)
    b = C.c_uint32(0)
    _check_rc(load_check().q4t_selftest_encoders(which, first, count, C.byref(m), C.byref(b), _stream_ptr()))
    return m.value, b.value
