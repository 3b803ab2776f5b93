"""ctypes access to libpgb_hostcheck.so (host mirror of the tile-stream walk)."""
import ctypes as C

import numpy as np

import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "peregrine_b200", "csrc")
HOSTCHECK = os.path.join(HERE, "libpgb_hostcheck.so")


def build_hostcheck(force: bool = False) -> str:
    """Host-only helper library of the CPU tests: the tile-stream walk compiled from the same
    layout header and repacker the CUDA backend uses."""
    srcs = [os.path.join(HERE, "w4_hostcheck.cpp"), os.path.join(CSRC, "w4_host.cpp")]
    deps = srcs + [os.path.join(CSRC, "w4_layout.h"), os.path.join(CSRC, "w4_host.h")]
    stale = force or not os.path.exists(HOSTCHECK) or any(
        os.path.getmtime(p) > os.path.getmtime(HOSTCHECK) for p in deps)
    if stale:
        subprocess.check_call(["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-pthread",
                               "-I", CSRC, "-o", HOSTCHECK] + srcs)
    return HOSTCHECK

_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build_hostcheck())
        vp, i = C.c_void_p, C.c_int
        L.pgb_hc_layout.argtypes = [i, i, i, i, vp]
        L.pgb_hc_repack.argtypes = [vp, vp, i, i, i, i, vp, vp, i]
        L.pgb_hc_nibble.argtypes = [vp, i, i, i, i, i, i]
        L.pgb_hc_qrow.argtypes = [vp, i, i, i, vp, vp, vp]
        L.pgb_hc_qrow.restype = None
        L.pgb_hc_walk.argtypes = [vp, vp, i, i, i, i, vp, vp, vp, i, vp, vp]
        _lib = L
    return _lib


FIELDS = ["O", "K", "grouped", "gs", "bpg", "ng_src", "nblk", "ntile", "chunk_bytes", "gpc", "nchunk", "kp",
          "tile_bytes", "total_bytes"]


def layout(O, K, grouped, gs):
    out = np.zeros(14, np.int64)
    if not lib().pgb_hc_layout(O, K, int(grouped), gs, out.ctypes.data):
        return None
    return dict(zip(FIELDS, [int(v) for v in out]))


def repack(q, scales, O, K, grouped, gs, threads=1):
    L = layout(O, K, grouped, gs)
    stream = np.zeros(L["total_bytes"], np.uint8)
    rs = np.zeros(L["ntile"] * 16, np.float32)
    q = np.ascontiguousarray(q, np.uint8)
    scales = np.ascontiguousarray(scales, np.float32)
    assert lib().pgb_hc_repack(q.ctypes.data, scales.ctypes.data, O, K, int(grouped), gs, stream.ctypes.data,
                               rs.ctypes.data, threads)
    return stream, rs, L


def nibble(stream, O, K, grouped, gs, o, k):
    return lib().pgb_hc_nibble(stream.ctypes.data, O, K, int(grouped), gs, o, k)


def qrow(x, L):
    x = np.ascontiguousarray(x, np.float32)
    xq = np.zeros(L["kp"], np.int8)
    sx = np.zeros(1, np.float32)
    cs = np.zeros(L["nblk"], np.int32)
    lib().pgb_hc_qrow(x.ctypes.data, x.size, L["kp"], L["nblk"], xq.ctypes.data, sx.ctypes.data, cs.ctypes.data)
    return xq, sx[0], cs


def walk(stream, rs, L, xq, cs, sx, nrows, want_tap=False):
    O = L["O"]
    y = np.zeros((nrows, O), np.float32)
    tap = np.zeros((nrows, O, L["ng_src"] if L["grouped"] else 1), np.int32) if want_tap else None
    xq = np.ascontiguousarray(xq, np.int8)
    cs = np.ascontiguousarray(cs, np.int32)
    sx = np.ascontiguousarray(sx, np.float32)
    assert lib().pgb_hc_walk(stream.ctypes.data, rs.ctypes.data, O, L["K"], L["grouped"], L["gs"], xq.ctypes.data,
                             cs.ctypes.data, sx.ctypes.data, nrows, y.ctypes.data,
                             None if tap is None else tap.ctypes.data)
    return (y, tap) if want_tap else y
