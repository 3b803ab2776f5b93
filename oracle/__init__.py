"""ctypes loader for the CPU oracle (``libperegrine_oracle.so``).

TEST INFRASTRUCTURE ONLY.  Importable from ``tests/``, from
``__graft_entry__.smoke()`` and from ``bench.py``'s CPU-baseline / reference
arm; the product package never imports it.

All array arguments are NumPy arrays; shapes follow the reference engine's
conventions (weights row-major ``[O, ceil(I/2)]`` packed nibbles, activations
``[S, I]``).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libperegrine_oracle.so")


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc only)."""
    src = os.path.join(_HERE, "peregrine_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libperegrine_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


class PoWeight(C.Structure):
    _fields_ = [
        ("q", C.c_void_p),
        ("scale", C.c_void_p),
        ("fmt", C.c_int32),
        ("gs", C.c_int32),
        ("i_n", C.c_int32),
        ("o_n", C.c_int32),
    ]


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        sz, vp, i32, f32 = C.c_size_t, C.c_void_p, C.c_int32, C.c_float
        L.po_lcg_next.restype = C.c_uint64
        L.po_lcg_next.argtypes = [vp]
        for n in ("po_lcg_fill_f32", "po_lcg_fill_i8_127", "po_lcg_fill_nib"):
            getattr(L, n).argtypes = [vp, vp, sz]
            getattr(L, n).restype = None
        L.po_pack_i4.argtypes = [vp, sz, vp]
        L.po_qrow_i8.argtypes = [vp, vp, sz]
        L.po_qrow_i8.restype = f32
        for n in ("po_dot_i4i8_scalar", "po_dot_i4i8"):
            getattr(L, n).argtypes = [vp, vp, sz]
            getattr(L, n).restype = i32
        for n in ("po_dot_i4i8_grouped_scalar", "po_dot_i4i8_grouped"):
            getattr(L, n).argtypes = [vp, vp, vp, sz, sz]
            getattr(L, n).restype = f32
        L.po_matmul_f32.argtypes = [vp, vp, vp, sz, sz, sz]
        L.po_matmul_i4_idot.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, vp]
        L.po_matmul_i4g_idot.argtypes = [vp, vp, vp, vp, vp, sz, sz, sz, sz, vp]
        L.po_weight_apply.argtypes = [vp, vp, sz, vp]
        L.po_sigmoidf.argtypes = [f32]
        L.po_sigmoidf.restype = f32
        L.po_siluf.argtypes = [f32]
        L.po_siluf.restype = f32
        L.po_silu_mul.argtypes = [vp, vp, sz]
        L.po_rmsnorm.argtypes = [vp, vp, vp, sz, f32]
        L.po_argmax.argtypes = [vp, sz]
        L.po_argmax.restype = i32
        L.po_swiglu.argtypes = [vp, vp, vp, vp, sz, vp, vp]
        L.po_route.argtypes = [vp, vp, vp, sz, sz, sz, sz, C.c_int, f32, vp, vp, vp, vp]
        L.po_batch_union.argtypes = [vp, vp, sz, sz, sz, vp]
        L.po_batch_union.restype = sz
        L.po_reduce_layout.argtypes = [vp, sz, sz, vp, vp]
        L.po_reduce_layout.restype = C.c_int
        L.po_moe_forward.argtypes = [vp, vp, vp, vp, sz, vp, sz, sz, sz, C.c_int, f32, C.c_int, vp, vp, vp, vp, vp, vp]
        L.po_quant_i4.argtypes = [vp, sz, sz, vp, vp]
        L.po_quant_i4_grouped.argtypes = [vp, sz, sz, sz, vp, vp]
        L.po_set_exp_mode.argtypes = [C.c_int]
        L.po_force_simd.argtypes = [C.c_int]
        L.po_simd_tier.restype = C.c_int
        L.po_max_threads.restype = C.c_int
        _lib = L
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _c(a, dt):
    a = np.ascontiguousarray(a, dtype=dt)
    return a


# ---------------------------------------------------------------- fixtures
class Lcg:
    """The reference's 64-bit LCG (testkit.rs:10-16, idot.rs:558-572)."""

    def __init__(self, seed: int):
        self.state = C.c_uint64(seed & 0xFFFFFFFFFFFFFFFF)

    def next(self) -> int:
        return int(lib().po_lcg_next(C.byref(self.state)))

    def f32(self, n: int) -> np.ndarray:
        out = np.empty(n, np.float32)
        lib().po_lcg_fill_f32(C.byref(self.state), _p(out), n)
        return out

    def i8_127(self, n: int) -> np.ndarray:
        out = np.empty(n, np.int8)
        lib().po_lcg_fill_i8_127(C.byref(self.state), _p(out), n)
        return out

    def nib(self, n: int) -> np.ndarray:
        out = np.empty(n, np.int32)
        lib().po_lcg_fill_nib(C.byref(self.state), _p(out), n)
        return out


def pack_i4(vals) -> np.ndarray:
    vals = _c(vals, np.int32)
    out = np.zeros((vals.size + 1) // 2, np.uint8)
    lib().po_pack_i4(_p(vals), vals.size, _p(out))
    return out


# ------------------------------------------------------------------ kernels
def qrow_i8(x):
    x = _c(x, np.float32)
    q = np.empty(x.size, np.int8)
    s = lib().po_qrow_i8(_p(x), _p(q), x.size)
    return q, np.float32(s)


def dot_i4i8_scalar(w4, x, n):
    w4, x = _c(w4, np.uint8), _c(x, np.int8)
    return int(lib().po_dot_i4i8_scalar(_p(w4), _p(x), n))


def dot_i4i8(w4, x, n):
    w4, x = _c(w4, np.uint8), _c(x, np.int8)
    return int(lib().po_dot_i4i8(_p(w4), _p(x), n))


def dot_i4i8_grouped(w4, x, scales, n, gs, scalar=False):
    w4, x, scales = _c(w4, np.uint8), _c(x, np.int8), _c(scales, np.float32)
    f = lib().po_dot_i4i8_grouped_scalar if scalar else lib().po_dot_i4i8_grouped
    return np.float32(f(_p(w4), _p(x), _p(scales), n, gs))


def matmul_f32(x, w, s_n, d_n, o_n):
    x, w = _c(x, np.float32), _c(w, np.float32)
    y = np.empty((s_n, o_n), np.float32)
    lib().po_matmul_f32(_p(y), _p(x), _p(w), s_n, d_n, o_n)
    return y


def matmul_i4_idot(xq, sx, q4, scale, s_n, i_n, o_n, want_acc=False):
    xq, sx, q4, scale = _c(xq, np.int8), _c(sx, np.float32), _c(q4, np.uint8), _c(scale, np.float32)
    y = np.empty((s_n, o_n), np.float32)
    acc = np.empty((s_n, o_n), np.int32) if want_acc else None
    lib().po_matmul_i4_idot(_p(y), _p(xq), _p(sx), _p(q4), _p(scale), s_n, i_n, o_n, _p(acc))
    return (y, acc) if want_acc else y


def matmul_i4g_idot(xq, sx, q4, scale, s_n, i_n, o_n, gs, want_blocks=False):
    xq, sx, q4, scale = _c(xq, np.int8), _c(sx, np.float32), _c(q4, np.uint8), _c(scale, np.float32)
    ng = (i_n + gs - 1) // gs
    y = np.empty((s_n, o_n), np.float32)
    blocks = np.empty((s_n, o_n, ng), np.int32) if want_blocks else None
    lib().po_matmul_i4g_idot(_p(y), _p(xq), _p(sx), _p(q4), _p(scale), s_n, i_n, o_n, gs, _p(blocks))
    return (y, blocks) if want_blocks else y


def sigmoidf(x):
    return np.float32(lib().po_sigmoidf(np.float32(x)))


def siluf(x):
    return np.float32(lib().po_siluf(np.float32(x)))


def silu_mul(g, u):
    g = np.array(g, np.float32, copy=True)
    u = _c(u, np.float32)
    lib().po_silu_mul(_p(g), _p(u), g.size)
    return g


def rmsnorm(x, w, eps):
    x, w = _c(x, np.float32), _c(w, np.float32)
    out = np.empty_like(x)
    lib().po_rmsnorm(_p(out), _p(x), _p(w), x.size, np.float32(eps))
    return out


def argmax(lo):
    lo = _c(lo, np.float32)
    return int(lib().po_argmax(_p(lo), lo.size))


def quant_i4(w, o, i):
    w = _c(w, np.float32)
    q = np.zeros(o * ((i + 1) // 2), np.uint8)
    sc = np.empty(o, np.float32)
    lib().po_quant_i4(_p(w), o, i, _p(q), _p(sc))
    return q, sc


def quant_i4_grouped(w, o, i, gs):
    w = _c(w, np.float32)
    q = np.zeros(o * ((i + 1) // 2), np.uint8)
    sc = np.empty(o * ((i + gs - 1) // gs), np.float32)
    lib().po_quant_i4_grouped(_p(w), o, i, gs, _p(q), _p(sc))
    return q, sc


def set_exp_mode(mode: int):
    lib().po_set_exp_mode(mode)


def force_simd(tier: int):
    lib().po_force_simd(tier)


def simd_tier() -> int:
    return int(lib().po_simd_tier())


def max_threads() -> int:
    return int(lib().po_max_threads())


# ----------------------------------------------------------------- weights
@dataclass
class Weight:
    """One quantised matrix as the reference's QtWeight holds it.

    fmt 2: per-row int4 (``scale[O]``); fmt 4: grouped int4 (``scale[O*ng]``,
    ``gs``); fmt 0: f32 ``[O, I]`` in ``q``.
    """

    q: np.ndarray
    scale: np.ndarray | None
    fmt: int
    gs: int
    i_n: int
    o_n: int

    def c(self) -> PoWeight:
        return PoWeight(
            self.q.ctypes.data,
            0 if self.scale is None else self.scale.ctypes.data,
            self.fmt,
            self.gs,
            self.i_n,
            self.o_n,
        )

    def apply(self, x, s_n):
        x = _c(x, np.float32)
        y = np.empty((s_n, self.o_n), np.float32)
        w = self.c()
        lib().po_weight_apply(C.byref(w), _p(x), s_n, _p(y))
        return y


def _weights_array(ws):
    arr = (PoWeight * len(ws))()
    for i, w in enumerate(ws):
        arr[i] = w.c()
    return arr


def swiglu(gate: Weight, up: Weight, down: Weight, x, s_n, want_h=False):
    x = _c(x, np.float32)
    y = np.empty((s_n, down.o_n), np.float32)
    h = np.empty((s_n, gate.o_n), np.float32) if want_h else None
    g, u, d = gate.c(), up.c(), down.c()
    lib().po_swiglu(C.byref(g), C.byref(u), C.byref(d), _p(x), s_n, _p(y), _p(h))
    return (y, h) if want_h else y


def route(x, router_w, router_bias, s_n, d_n, e_n, k, norm_topk, routed_scale, want_logits=False):
    x, router_w, router_bias = _c(x, np.float32), _c(router_w, np.float32), _c(router_bias, np.float32)
    idx = np.zeros((s_n, k), np.int32)
    w = np.zeros((s_n, k), np.float32)
    keff = np.zeros(s_n, np.int32)
    logits = np.empty((s_n, e_n), np.float32) if want_logits else None
    lib().po_route(_p(x), _p(router_w), _p(router_bias), s_n, d_n, e_n, k, int(bool(norm_topk)),
                   np.float32(routed_scale), _p(idx), _p(w), _p(keff), _p(logits))
    return (idx, w, keff, logits) if want_logits else (idx, w, keff)


def batch_union(idx, keff, s_n, k, e_n):
    idx, keff = _c(idx, np.int32), _c(keff, np.int32)
    out = np.empty(e_n + 1, np.int32)
    n = lib().po_batch_union(_p(idx), _p(keff), s_n, k, e_n, _p(out))
    return out[:n].copy()


def reduce_layout(dst, s_n):
    dst = _c(dst, np.int32)
    row_ptr = np.zeros(s_n + 1, np.int32)
    row_idx = np.zeros(dst.size, np.int32)
    ok = lib().po_reduce_layout(_p(dst), dst.size, s_n, _p(row_ptr), _p(row_idx))
    return (row_ptr, row_idx) if ok else None


def moe_forward(x, router_w, router_bias, experts, shared, s_n, hidden, k, norm_topk, routed_scale, threads=1,
                want_routing=False):
    """experts: list of (gate, up, down) Weight triples; shared: triple or None."""
    x, router_w, router_bias = _c(x, np.float32), _c(router_w, np.float32), _c(router_bias, np.float32)
    e_n = len(experts)
    flat = _weights_array([w for tri in experts for w in tri])
    sh = _weights_array(list(shared)) if shared is not None else None
    out = np.empty((s_n, hidden), np.float32)
    idx = np.zeros((s_n, k), np.int32)
    w = np.zeros((s_n, k), np.float32)
    keff = np.zeros(s_n, np.int32)
    uni = np.zeros(e_n + 1, np.int32)
    nu = C.c_int32(0)
    lib().po_moe_forward(_p(x), _p(router_w), _p(router_bias), C.cast(flat, C.c_void_p), e_n,
                         C.cast(sh, C.c_void_p) if sh is not None else None, s_n, hidden, k, int(bool(norm_topk)),
                         np.float32(routed_scale), threads, _p(out), _p(idx), _p(w), _p(keff), _p(uni),
                         C.cast(C.byref(nu), C.c_void_p))
    if want_routing:
        return out, idx, w, keff, uni[: nu.value].copy()
    return out
