"""ctypes/numpy front end of the CPU oracle (oracle/q4t_oracle.c).

TEST INFRASTRUCTURE ONLY.  The tests, the smoke check and the benchmark's
CPU-baseline leg import this module; the CUDA library never does.  bf16 data
is carried as uint16 arrays throughout.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libq4t_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libq4t_ref.so")


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference pinning shim when the reference
    tree is present) with the Makefile beside this file."""
    if force or not os.path.exists(_LIB_PATH) or (
        os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "q4t_oracle.c"))
    ):
        subprocess.run(["make", "-C", _HERE], check=True, capture_output=True)


def build_ref_gpu() -> bool:
    """Compile the reference's own GPU implementation of the routed experts into
    oracle/_ref/libq4t_ref_gpu.so (the second oracle of the GPU tests) when the reference tree
    and nvcc are present; returns whether the library exists afterwards.  A failure to build is
    not an error: the tests that use it skip."""
    try:
        subprocess.run(["make", "-C", _HERE, "ref_gpu"], check=True, capture_output=True, timeout=900)
    except (subprocess.SubprocessError, OSError):
        pass
    return os.path.exists(os.path.join(_HERE, "_ref", "libq4t_ref_gpu.so"))


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


class _Layer(C.Structure):
    _fields_ = [("E", C.c_int), ("hs", C.c_int), ("moe_is", C.c_int), ("shared_is", C.c_int),
                ("gu_packed", C.c_void_p), ("gu_sf", C.c_void_p),
                ("dn_packed", C.c_void_p), ("dn_sf", C.c_void_p),
                ("gu_w_scale2", C.c_void_p), ("gu_input_scale", C.c_void_p),
                ("dn_w_scale2", C.c_void_p), ("dn_input_scale", C.c_void_p),
                ("gate", C.c_void_p), ("shared_gu", C.c_void_p),
                ("shared_down", C.c_void_p), ("shared_gate_scalar", C.c_void_p)]


class _Taps(C.Structure):
    _fields_ = [("a_packed", C.c_void_p), ("a_sf", C.c_void_p), ("gu_out", C.c_void_p),
                ("i_packed", C.c_void_p), ("i_sf", C.c_void_p), ("dn_out", C.c_void_p)]


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_LIB_PATH)
        L.q4o_e2m1_to_float.restype = C.c_float
        L.q4o_e2m1_to_float.argtypes = [C.c_uint8]
        L.q4o_float_to_e2m1.restype = C.c_int
        L.q4o_float_to_e2m1.argtypes = [C.c_float]
        L.q4o_e4m3_to_float.restype = C.c_float
        L.q4o_e4m3_to_float.argtypes = [C.c_uint8]
        L.q4o_float_to_e4m3.restype = C.c_uint8
        L.q4o_float_to_e4m3.argtypes = [C.c_float]
        L.q4o_sf_offset.restype = C.c_size_t
        L.q4o_sf_offset.argtypes = [C.c_int, C.c_int, C.c_int]
        L.q4o_sf_num_gtiles.restype = C.c_int
        L.q4o_sf_buffer_size.restype = C.c_size_t
        L.q4o_sf_buffer_size.argtypes = [C.c_int, C.c_int]
        L.q4o_routed_forward.restype = C.c_int
        L.q4o_moe_forward.restype = C.c_int
        L.q4o_num_threads.restype = C.c_int
        _lib = L
    return _lib


def ref_lib():
    """The reference's own header functions (oracle/_ref), or None if that
    shim has not been built (no reference tree on this machine)."""
    if not os.path.exists(_REF_PATH):
        return None
    R = C.CDLL(_REF_PATH)
    R.ref_e2m1_to_float.restype = C.c_float
    R.ref_e2m1_to_float.argtypes = [C.c_uint8]
    R.ref_float_to_e2m1.restype = C.c_int
    R.ref_float_to_e2m1.argtypes = [C.c_float]
    R.ref_e4m3_to_float.restype = C.c_float
    R.ref_e4m3_to_float.argtypes = [C.c_uint8]
    R.ref_float_to_e4m3.restype = C.c_uint8
    R.ref_float_to_e4m3.argtypes = [C.c_float]
    R.ref_sf_offset.restype = C.c_size_t
    R.ref_sf_offset.argtypes = [C.c_int, C.c_int, C.c_int]
    R.ref_sf_num_gtiles.restype = C.c_int
    R.ref_sf_buffer_size.restype = C.c_size_t
    R.ref_sf_buffer_size.argtypes = [C.c_int, C.c_int]
    return R


# ----------------------------------------------------------------- bf16 utils
def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------ primitives
def sf_buffer_size(rows: int, K: int) -> int:
    return int(lib().q4o_sf_buffer_size(rows, K))


def sf_offset(row: int, group: int, nt: int) -> int:
    return int(lib().q4o_sf_offset(row, group, nt))


def swizzle_sf(sf_rm: np.ndarray, rows: int, K: int) -> np.ndarray:
    sf_rm = np.ascontiguousarray(sf_rm, dtype=np.uint8)
    out = np.empty(sf_buffer_size(rows, K), np.uint8)
    lib().q4o_swizzle_sf(_p(sf_rm, C.c_uint8), C.c_int(rows), C.c_int(K), _p(out, C.c_uint8))
    return out


def unswizzle_sf(sf_swz: np.ndarray, rows: int, K: int) -> np.ndarray:
    """Row-major [rows, K/16] view of a swizzled buffer (inverse of swizzle_sf)."""
    groups = K // 16
    nt = (groups + 3) // 4
    r = np.arange(rows)[:, None]
    g = np.arange(groups)[None, :]
    off = (r % 32) * 16 + ((r % 128) // 32) * 4 + (g % 4) + (g // 4) * 512 + (r // 128) * nt * 512
    return np.asarray(sf_swz, dtype=np.uint8)[off]


def quantize_f32(v: np.ndarray, global_scale: float):
    v = np.ascontiguousarray(v, dtype=np.float32)
    rows, K = v.shape
    packed = np.empty((rows, K // 2), np.uint8)
    sf = np.empty((rows, K // 16), np.uint8)
    lib().q4o_quantize_f32(_p(v, C.c_float), C.c_int(rows), C.c_int(K), C.c_float(global_scale),
                           _p(packed, C.c_uint8), _p(sf, C.c_uint8))
    return packed, sf


def quantize_bf16(x: np.ndarray, global_scale: float):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    rows, K = x.shape
    packed = np.empty((rows, K // 2), np.uint8)
    sf = np.empty(sf_buffer_size(rows, K), np.uint8)
    lib().q4o_quantize_bf16(_p(x, C.c_uint16), C.c_int(rows), C.c_int(K), C.c_float(global_scale),
                            _p(packed, C.c_uint8), _p(sf, C.c_uint8))
    return packed, sf


def dequant_to_bf16(packed, sf_rm, inv_global: float):
    packed = np.ascontiguousarray(packed, np.uint8)
    sf_rm = np.ascontiguousarray(sf_rm, np.uint8)
    N, K2 = packed.shape
    out = np.empty((N, K2 * 2), np.uint16)
    lib().q4o_dequant_to_bf16(_p(packed, C.c_uint8), _p(sf_rm, C.c_uint8), C.c_int(N),
                              C.c_int(K2 * 2), C.c_float(inv_global), _p(out, C.c_uint16))
    return out


def dequant_to_f32(packed, sf_rm, global_scale: float):
    packed = np.ascontiguousarray(packed, np.uint8)
    sf_rm = np.ascontiguousarray(sf_rm, np.uint8)
    N, K2 = packed.shape
    out = np.empty((N, K2 * 2), np.float32)
    lib().q4o_dequant_to_f32(_p(packed, C.c_uint8), _p(sf_rm, C.c_uint8), C.c_int(N),
                             C.c_int(K2 * 2), C.c_float(global_scale), _p(out, C.c_float))
    return out


def fp4_gemm(w_packed, w_sf, a_packed, a_sf, M, N, K, inv_w, inv_a, mode):
    out = np.empty((M, N), np.float32)
    args = [np.ascontiguousarray(t, np.uint8) for t in (w_packed, w_sf, a_packed, a_sf)]
    lib().q4o_fp4_gemm(*[_p(t, C.c_uint8) for t in args], _p(out, C.c_float), C.c_int(M),
                       C.c_int(N), C.c_int(K), C.c_float(inv_w), C.c_float(inv_a), C.c_int(mode))
    return out


def bf16_linear(x, w, mode: int):
    x = np.ascontiguousarray(x, np.uint16)
    w = np.ascontiguousarray(w, np.uint16)
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), np.uint16)
    lib().q4o_bf16_linear(_p(x, C.c_uint16), _p(w, C.c_uint16), _p(y, C.c_uint16), C.c_int(M),
                          C.c_int(N), C.c_int(K), C.c_int(mode))
    return y


def router_topk(logits, k: int):
    logits = np.ascontiguousarray(logits, np.uint16)
    T, E = logits.shape
    ids = np.empty((T, k), np.int32)
    w = np.empty((T, k), np.float32)
    lib().q4o_router_topk(_p(logits, C.c_uint16), C.c_int(T), C.c_int(E), C.c_int(k),
                          _p(ids, C.c_int32), _p(w, C.c_float))
    return ids, w


def permutation(ids, E: int):
    ids = np.ascontiguousarray(ids, np.int32)
    T, k = ids.shape
    counts = np.empty(E, np.int32)
    offsets = np.empty(E + 1, np.int32)
    rof = np.empty(T * k, np.int32)
    fofr = np.empty(T * k, np.int32)
    lib().q4o_permutation(_p(ids, C.c_int32), C.c_int(T), C.c_int(k), C.c_int(E),
                          _p(counts, C.c_int32), _p(offsets, C.c_int32), _p(rof, C.c_int32),
                          _p(fofr, C.c_int32))
    return counts, offsets, rof, fofr


class Layer:
    """Host copy of one MoE layer in the reference's device layout."""

    FIELDS = ("gu_packed", "gu_sf", "dn_packed", "dn_sf", "gu_w_scale2", "gu_input_scale",
              "dn_w_scale2", "dn_input_scale", "gate", "shared_gu", "shared_down",
              "shared_gate_scalar")

    def __init__(self, E, hs, moe_is, shared_is, **arrays):
        self.E, self.hs, self.moe_is, self.shared_is = E, hs, moe_is, shared_is
        for f in self.FIELDS:
            a = arrays.get(f)
            setattr(self, f, None if a is None else np.ascontiguousarray(a))

    def cstruct(self) -> _Layer:
        s = _Layer(self.E, self.hs, self.moe_is, self.shared_is)
        for f in self.FIELDS:
            a = getattr(self, f)
            setattr(s, f, None if a is None else a.ctypes.data)
        return s


def routed_forward(x, ids, rw, layer: Layer, mode: int, want_taps: bool = False, y0=None):
    x = np.ascontiguousarray(x, np.uint16)
    ids = np.ascontiguousarray(ids, np.int32)
    rw = np.ascontiguousarray(rw, np.float32)
    T, k = ids.shape
    hs, is_ = layer.hs, layer.moe_is
    R = T * k
    y = np.zeros((T, hs), np.float32) if y0 is None else np.array(y0, np.float32, order="C")
    taps = None
    tp = None
    if want_taps:
        taps = dict(a_packed=np.zeros((R, hs // 2), np.uint8), a_sf=np.zeros((R, hs // 16), np.uint8),
                    gu_out=np.zeros((R, 2 * is_), np.uint16), i_packed=np.zeros((R, is_ // 2), np.uint8),
                    i_sf=np.zeros((R, is_ // 16), np.uint8), dn_out=np.zeros((R, hs), np.uint16))
        tp = _Taps(*[taps[n].ctypes.data for n, _ in _Taps._fields_])
    ls = layer.cstruct()
    rc = lib().q4o_routed_forward(_p(x, C.c_uint16), _p(ids, C.c_int32), _p(rw, C.c_float),
                                  _p(y, C.c_float), C.byref(ls), C.c_int(T), C.c_int(k),
                                  C.c_int(mode), C.byref(tp) if tp is not None else None)
    if rc != 0:
        raise ValueError("invalid MoE forward dims")
    return (y, taps) if want_taps else y


def combine_rows(rows, row_of_flat, rw, T, k):
    rows = np.ascontiguousarray(rows, np.uint16)
    rof = np.ascontiguousarray(row_of_flat, np.int32)
    rw = np.ascontiguousarray(rw, np.float32)
    hs = rows.shape[1]
    y = np.zeros((T, hs), np.float32)
    lib().q4o_combine_rows(_p(rows, C.c_uint16), _p(rof, C.c_int32), _p(rw, C.c_float), C.c_int(T), C.c_int(k),
                           C.c_int(hs), _p(y, C.c_float))
    return y


def shared_combine(x, routed, layer: Layer, linear_mode: int):
    x = np.ascontiguousarray(x, np.uint16)
    routed = np.ascontiguousarray(routed, np.float32)
    T = x.shape[0]
    y = np.empty((T, layer.hs), np.uint16)
    ls = layer.cstruct()
    lib().q4o_shared_combine(_p(x, C.c_uint16), _p(routed, C.c_float), C.byref(ls), C.c_int(T),
                             C.c_int(linear_mode), _p(y, C.c_uint16))
    return y


def moe_forward(x, layer: Layer, k: int, logits_mode=0, routed_mode=1, linear_mode=0):
    x = np.ascontiguousarray(x, np.uint16)
    T = x.shape[0]
    y = np.empty((T, layer.hs), np.uint16)
    logits = np.empty((T, layer.E), np.uint16)
    ids = np.empty((T, k), np.int32)
    rw = np.empty((T, k), np.float32)
    routed = np.empty((T, layer.hs), np.float32)
    ls = layer.cstruct()
    rc = lib().q4o_moe_forward(_p(x, C.c_uint16), C.byref(ls), C.c_int(T), C.c_int(k),
                               C.c_int(logits_mode), C.c_int(routed_mode), C.c_int(linear_mode),
                               _p(y, C.c_uint16), _p(logits, C.c_uint16), _p(ids, C.c_int32),
                               _p(rw, C.c_float), _p(routed, C.c_float))
    if rc != 0:
        raise ValueError("k out of range")
    return dict(y=y, logits=logits, ids=ids, rw=rw, routed=routed)


def rmsnorm_bf16(x, eps: float = 1e-6):
    x = np.ascontiguousarray(x, np.uint16)
    T, hs = x.shape
    out = np.empty_like(x)
    lib().q4o_rmsnorm_bf16(_p(x, C.c_uint16), C.c_int(T), C.c_int(hs), C.c_float(eps),
                           _p(out, C.c_uint16))
    return out


def residual_rmsnorm_bf16(x, y, eps: float = 1e-6):
    """Returns (bf16(x + y), RMSNorm of that); y may be None (norm only).  Follows
    q4o_residual_rmsnorm_bf16."""
    x = np.array(x, np.uint16, copy=True, order="C")
    T, hs = x.shape
    h = np.empty_like(x)
    yp = None if y is None else _p(np.ascontiguousarray(y, np.uint16), C.c_uint16)
    lib().q4o_residual_rmsnorm_bf16(_p(x, C.c_uint16), yp, C.c_int(T), C.c_int(hs), C.c_float(eps),
                                    _p(h, C.c_uint16))
    return x, h


def gated_residual_write(y, residual, gate):
    """out[t, b, :] = bf16(residual[t, b, :] + y[t, :] * gate[t, b]) on bf16 bit patterns
    (q4o_gated_residual_write); y [T, hs], residual [T, hc*hs], gate [T, hc]."""
    y = np.ascontiguousarray(y, np.uint16)
    residual = np.ascontiguousarray(residual, np.uint16)
    gate = np.ascontiguousarray(gate, np.uint16)
    T, hs = y.shape
    hc = gate.shape[1]
    out = np.empty_like(residual)
    lib().q4o_gated_residual_write(_p(y, C.c_uint16), _p(residual, C.c_uint16), _p(gate, C.c_uint16), C.c_int(T),
                                   C.c_int(hc), C.c_int(hs), _p(out, C.c_uint16))
    return out


def moe_bf16_routed_forward(x, ids, rw, gu, down, y0=None):
    """The MTP draft layer's BF16 routed experts (q4o_moe_bf16_routed_forward): gu [E, 2*is, hs],
    down [E, hs, is] bf16 bit patterns; returns fp32 [T, hs] (added to y0 when given)."""
    x = np.ascontiguousarray(x, np.uint16)
    ids = np.ascontiguousarray(ids, np.int32)
    rw = np.ascontiguousarray(rw, np.float32)
    gu = np.ascontiguousarray(gu, np.uint16)
    down = np.ascontiguousarray(down, np.uint16)
    T, hs = x.shape
    k = ids.shape[1]
    E, two_is, _ = gu.shape
    y = np.zeros((T, hs), np.float32) if y0 is None else np.array(y0, np.float32, copy=True, order="C")
    lib().q4o_moe_bf16_routed_forward(_p(x, C.c_uint16), _p(ids, C.c_int32), _p(rw, C.c_float), _p(gu, C.c_uint16),
                                      _p(down, C.c_uint16), C.c_int(T), C.c_int(k), C.c_int(E), C.c_int(hs),
                                      C.c_int(two_is // 2), _p(y, C.c_float))
    return y


def set_num_threads(n: int) -> None:
    lib().q4o_set_num_threads(C.c_int(int(n)))


def num_threads() -> int:
    return int(lib().q4o_num_threads())
