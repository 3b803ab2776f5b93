"""Host-side mirror of ``crates/peregrine-cuda/src/lib.rs`` over the C ABI.

Names and behaviour follow the reference crate: ``init``/``shutdown``/
``mem_info`` (lib.rs:161-255), ``GpuExpert.upload``/``upload_int4``
(lib.rs:257-347), ``expert_group`` / ``expert_group_tiled`` /
``expert_group_reduce`` (lib.rs:420-679), ``ReduceLayout.build``
(lib.rs:563-610), ``GroupArm`` (lib.rs:436-461), ``group_stats`` /
``graph_cache_stats`` (lib.rs:686-740).  Failures raise ``CudaError`` where the
reference returns ``Err(Error::Format(..))``.

There is no CPU fallback: if the shared library is missing or does not load the
import of this module's ``lib()`` fails loudly.
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("PEREGRINE_B200_LIB") or os.path.join(_HERE, "libcoli_cuda_backend.so")

# every symbol include/peregrine_b200.h declares
SYMBOLS = [
    "coli_cuda_init", "coli_cuda_shutdown", "coli_cuda_device_count", "coli_cuda_probe_device_count",
    "coli_cuda_device_at", "coli_cuda_mem_info", "coli_cuda_stats", "coli_cuda_group_stats",
    "coli_cuda_tensor_upload", "coli_cuda_tensor_update", "coli_cuda_tensor_free", "coli_cuda_tensor_bytes",
    "coli_cuda_tensor_device", "coli_cuda_matmul", "coli_cuda_expert_mlp", "coli_cuda_shared_mlp_w4a16",
    "coli_cuda_expert_group", "coli_cuda_expert_group_tiled", "coli_cuda_expert_group_reduce",
    "coli_cuda_attention_absorb", "coli_cuda_attention_absorb_batch", "coli_cuda_attention_project_batch",
    "coli_cuda_attention_project_batch_dev", "coli_cuda_attention_absorb_batch_dev",
    "coli_cuda_attention_absorb_kvdev", "coli_cuda_attention_project_batch_dev_out",
    "coli_cuda_pipe_scratch", "coli_cuda_pipe_alloc", "coli_cuda_pipe_free", "coli_cuda_pipe_upload",
    "coli_cuda_pipe_download", "coli_cuda_pipe_rmsnorm", "coli_cuda_pipe_rmsnorm_s", "coli_cuda_pipe_rope",
    "coli_cuda_pipe_rope_base", "coli_cuda_pipe_silu_mul", "coli_cuda_pipe_add", "coli_cuda_pipe_rows_add",
    "coli_cuda_pipe_gemm", "coli_cuda_pipe_copy2d", "coli_cuda_pipe_peer_copy", "coli_cuda_pipe_sync",
    "coli_cuda_graph_begin", "coli_cuda_graph_end", "coli_cuda_graph_launch", "coli_cuda_graph_free",
    "coli_cuda_graph_cache_stats",
    # additive entry points
    "coli_cuda_tensor_upload_grouped", "coli_cuda_moe_layer_create", "coli_cuda_moe_layer_set_expert",
    "coli_cuda_moe_layer_free", "coli_cuda_moe_layer_forward_dev", "coli_cuda_moe_layer_forward",
    "coli_cuda_moe_layer_last_routing", "coli_cuda_moe_layer_enable_taps", "coli_cuda_moe_layer_set_spec",
    "coli_cuda_moe_layer_set_fused", "coli_cuda_int8_peak_probe", "coli_cuda_tensor_clone", "coli_cuda_moe_layer_set_bias", "coli_cuda_moe_layer_decode_timeline", "coli_cuda_moe_layer_host_times", "coli_cuda_graph_launch_async", "coli_cuda_moe_layer_last_pairs",
    "coli_cuda_moe_layer_read_taps", "coli_cuda_moe_layer_set_ep", "coli_cuda_ep_create",
    "coli_cuda_ep_block_bytes", "coli_cuda_ep_local_base", "coli_cuda_ep_export", "coli_cuda_ep_attach",
    "coli_cuda_ep_attach_ptr", "coli_cuda_ep_free", "coli_cuda_ep_reset", "coli_cuda_moe_layer_ep_route_dev",
    "coli_cuda_moe_layer_ep_dispatch_dev", "coli_cuda_moe_layer_ep_experts_dev", "coli_cuda_moe_layer_ep_finish_dev",
    "coli_cuda_moe_layer_ep_forward_dev", "coli_cuda_moe_layer_set_profile", "coli_cuda_moe_layer_profile",
    "coli_cuda_pipe_gemm_noalloc", "coli_cuda_pipe_embed", "coli_cuda_pipe_argmax", "coli_cuda_last_device_error", "coli_cuda_selftest_bounded_wait", "coli_cuda_kernel_launches", "coli_cuda_stream",
]


class CudaError(RuntimeError):
    pass


_lib = None


def lib():
    """Loads the backend; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise CudaError(f"{LIB_PATH} is missing: build it with `python -m peregrine_b200.build`")
        L = C.CDLL(LIB_PATH)
        vp, i, f, sz, u64 = C.c_void_p, C.c_int, C.c_float, C.c_size_t, C.c_uint64
        L.coli_cuda_init.argtypes = [vp, i]
        L.coli_cuda_shutdown.restype = None
        L.coli_cuda_device_at.argtypes = [i]
        L.coli_cuda_mem_info.argtypes = [i, vp, vp]
        L.coli_cuda_stats.argtypes = [i, vp, vp]
        L.coli_cuda_stats.restype = None
        L.coli_cuda_group_stats.argtypes = [vp] * 6
        L.coli_cuda_group_stats.restype = None
        L.coli_cuda_graph_cache_stats.argtypes = [vp] * 4
        L.coli_cuda_graph_cache_stats.restype = None
        L.coli_cuda_tensor_upload.argtypes = [vp, vp, vp, i, i, i, i]
        L.coli_cuda_tensor_upload_grouped.argtypes = [vp, vp, vp, i, i, i, i]
        L.coli_cuda_tensor_update.argtypes = [vp, vp, vp]
        L.coli_cuda_tensor_free.argtypes = [vp]
        L.coli_cuda_tensor_free.restype = None
        L.coli_cuda_tensor_bytes.argtypes = [vp]
        L.coli_cuda_tensor_bytes.restype = sz
        L.coli_cuda_tensor_device.argtypes = [vp]
        L.coli_cuda_matmul.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i]
        L.coli_cuda_expert_mlp.argtypes = [vp, vp, vp, vp, vp, i]
        L.coli_cuda_expert_group.argtypes = [vp, vp, vp, vp, i, vp, vp]
        L.coli_cuda_expert_group_tiled.argtypes = [vp, vp, vp, vp, i, vp, vp, i, i, i, vp]
        L.coli_cuda_expert_group_reduce.argtypes = [vp, vp, vp, vp, i, vp, vp, vp, i, vp, vp]
        L.coli_cuda_pipe_scratch.argtypes = [i, i, sz]
        L.coli_cuda_pipe_scratch.restype = vp
        L.coli_cuda_pipe_alloc.argtypes = [i, sz]
        L.coli_cuda_pipe_alloc.restype = vp
        L.coli_cuda_pipe_free.argtypes = [i, vp]
        L.coli_cuda_pipe_free.restype = None
        L.coli_cuda_pipe_upload.argtypes = [i, vp, vp, sz]
        L.coli_cuda_pipe_download.argtypes = [i, vp, vp, sz]
        L.coli_cuda_pipe_rmsnorm.argtypes = [i, vp, vp, vp, i, i, f]
        L.coli_cuda_pipe_rmsnorm_s.argtypes = [i, vp, vp, vp, i, i, f, i, i]
        L.coli_cuda_pipe_rope.argtypes = [i, vp, vp, i, i, i, i, i, f]
        L.coli_cuda_pipe_rope_base.argtypes = [i, vp, i, i, i, i, i, i, f]
        L.coli_cuda_pipe_silu_mul.argtypes = [i, vp, vp, sz]
        L.coli_cuda_pipe_add.argtypes = [i, vp, vp, sz]
        L.coli_cuda_pipe_rows_add.argtypes = [i, vp, vp, vp, i, i]
        L.coli_cuda_pipe_gemm.argtypes = [vp, vp, vp, i]
        L.coli_cuda_pipe_gemm_noalloc.argtypes = [vp, vp, vp, i]
        L.coli_cuda_pipe_embed.argtypes = [i, vp, vp, vp, i, i, i]
        L.coli_cuda_pipe_argmax.argtypes = [i, vp, vp, i, i]
        L.coli_cuda_pipe_copy2d.argtypes = [i, vp, i, vp, i, i, i]
        L.coli_cuda_pipe_peer_copy.argtypes = [i, vp, i, vp, sz]
        L.coli_cuda_pipe_sync.argtypes = [i]
        L.coli_cuda_graph_begin.argtypes = [i]
        L.coli_cuda_graph_end.argtypes = [i, vp]
        L.coli_cuda_graph_launch.argtypes = [vp]
        L.coli_cuda_graph_launch_async.argtypes = [vp]
        L.coli_cuda_graph_free.argtypes = [vp]
        L.coli_cuda_graph_free.restype = None
        L.coli_cuda_moe_layer_create.argtypes = [vp, i, i, i, i, i, i, f, vp, vp]
        L.coli_cuda_moe_layer_set_expert.argtypes = [vp, i, vp, vp, vp]
        L.coli_cuda_moe_layer_free.argtypes = [vp]
        L.coli_cuda_moe_layer_free.restype = None
        L.coli_cuda_moe_layer_forward_dev.argtypes = [vp, vp, vp, i]
        L.coli_cuda_moe_layer_forward.argtypes = [vp, vp, vp, i]
        L.coli_cuda_moe_layer_last_routing.argtypes = [vp, i, vp, vp, vp, vp, vp]
        L.coli_cuda_moe_layer_enable_taps.argtypes = [vp, i]
        L.coli_cuda_moe_layer_set_spec.argtypes = [vp, i]
        L.coli_cuda_moe_layer_set_fused.argtypes = [vp, i]
        L.coli_cuda_tensor_clone.argtypes = [vp, vp]
        L.coli_cuda_int8_peak_probe.argtypes = [i, i, i]
        L.coli_cuda_int8_peak_probe.restype = C.c_double
        L.coli_cuda_moe_layer_set_bias.argtypes = [vp, vp]
        L.coli_cuda_moe_layer_decode_timeline.argtypes = [vp, i, vp, i, vp, vp]
        L.coli_cuda_moe_layer_host_times.argtypes = [vp, vp, vp, i]
        L.coli_cuda_moe_layer_last_pairs.argtypes = [vp, vp, vp, vp, i]
        L.coli_cuda_moe_layer_read_taps.argtypes = [vp, vp, sz, vp, sz]
        L.coli_cuda_moe_layer_set_ep.argtypes = [vp, i, i]
        L.coli_cuda_ep_create.argtypes = [vp, i, i, i, i, i, i]
        L.coli_cuda_ep_block_bytes.argtypes = [vp]
        L.coli_cuda_ep_block_bytes.restype = sz
        L.coli_cuda_ep_local_base.argtypes = [vp]
        L.coli_cuda_ep_local_base.restype = vp
        L.coli_cuda_ep_export.argtypes = [vp, vp]
        L.coli_cuda_ep_attach.argtypes = [vp, i, vp]
        L.coli_cuda_ep_attach_ptr.argtypes = [vp, i, vp]
        L.coli_cuda_ep_reset.argtypes = [vp]
        L.coli_cuda_ep_free.argtypes = [vp]
        L.coli_cuda_ep_free.restype = None
        L.coli_cuda_moe_layer_ep_route_dev.argtypes = [vp, vp, vp]
        L.coli_cuda_moe_layer_ep_dispatch_dev.argtypes = [vp, vp]
        L.coli_cuda_moe_layer_ep_experts_dev.argtypes = [vp, vp]
        L.coli_cuda_moe_layer_ep_finish_dev.argtypes = [vp, vp, vp]
        L.coli_cuda_moe_layer_ep_forward_dev.argtypes = [vp, vp, vp, vp]
        L.coli_cuda_moe_layer_set_profile.argtypes = [vp, i]
        L.coli_cuda_moe_layer_profile.argtypes = [vp, vp, vp]
        L.coli_cuda_last_device_error.argtypes = [i]
        L.coli_cuda_selftest_bounded_wait.argtypes = [i, C.c_longlong]
        L.coli_cuda_kernel_launches.restype = u64
        L.coli_cuda_stream.argtypes = [i]
        L.coli_cuda_stream.restype = vp
        _lib = L
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ------------------------------------------------------------ lifecycle
def probe_device_count() -> int:
    return int(lib().coli_cuda_probe_device_count())


def init(devices) -> int:
    """Initialise contexts on the given CUDA ordinals; returns how many are up
    (0 on failure), as the reference's ``init`` does (lib.rs:161-190)."""
    arr = np.ascontiguousarray(devices, dtype=np.int32)
    if arr.size == 0:
        return 0
    if lib().coli_cuda_init(_ptr(arr), int(arr.size)) != 1:
        return 0
    return int(lib().coli_cuda_device_count())


def shutdown() -> None:
    lib().coli_cuda_shutdown()


def device_count() -> int:
    return int(lib().coli_cuda_device_count())


def mem_info(device: int):
    free, total = C.c_size_t(0), C.c_size_t(0)
    if lib().coli_cuda_mem_info(device, C.byref(free), C.byref(total)) != 1:
        raise CudaError(f"cuda mem_info(device={device}) failed")
    return free.value, total.value


@dataclass
class GroupStats:
    calls: int
    experts: int
    rows: int
    h2d_ms: float
    kernel_ms: float
    d2h_ms: float


def group_stats() -> GroupStats:
    a, b, c_ = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
    d, e, f = C.c_double(0), C.c_double(0), C.c_double(0)
    lib().coli_cuda_group_stats(C.byref(a), C.byref(b), C.byref(c_), C.byref(d), C.byref(e), C.byref(f))
    return GroupStats(a.value, b.value, c_.value, d.value, e.value, f.value)


@dataclass
class GraphCacheStats:
    captures: int
    replays: int
    invalidations: int
    uncacheable: int


def graph_cache_stats() -> GraphCacheStats:
    v = [C.c_uint64(0) for _ in range(4)]
    lib().coli_cuda_graph_cache_stats(*[C.byref(x) for x in v])
    return GraphCacheStats(*[x.value for x in v])


def int8_peak_probe(device: int, iters: int = 8192, launches: int = 20) -> float:
    """Measured int8 tensor throughput (tera-ops/s) of a bare tcgen05 kind::i8 loop, one CTA per SM."""
    return float(lib().coli_cuda_int8_peak_probe(device, iters, launches))


def kernel_launches() -> int:
    return int(lib().coli_cuda_kernel_launches())


def last_device_error(device: int) -> int:
    return int(lib().coli_cuda_last_device_error(device))


def selftest_bounded_wait(device: int, limit_cycles: int = 200_000) -> bool:
    """Runs the bounded-wait self-test kernel; the expired wait shows up in ``last_device_error``."""
    return lib().coli_cuda_selftest_bounded_wait(device, int(limit_cycles)) == 1


# ------------------------------------------------------------ residency
class Tensor:
    """One resident matrix (``ColiCudaTensor*``); freed on ``free()``/GC."""

    def __init__(self, handle, fmt, i_n, o_n, device):
        self.handle, self.fmt, self.i_n, self.o_n, self.device = handle, fmt, i_n, o_n, device

    @staticmethod
    def upload(device, weights, scales, fmt, i_n, o_n) -> "Tensor":
        h = C.c_void_p(None)
        w = np.ascontiguousarray(weights)
        s = None if scales is None else _f32(scales)
        ok = lib().coli_cuda_tensor_upload(C.byref(h), _ptr(w), _ptr(s), fmt, i_n, o_n, device)
        if ok != 1 or not h.value:
            raise CudaError(f"cuda tensor_upload failed (fmt={fmt}, i={i_n}, o={o_n})")
        return Tensor(h, fmt, i_n, o_n, device)

    @staticmethod
    def upload_grouped(device, weights, scales, i_n, o_n, gs) -> "Tensor":
        h = C.c_void_p(None)
        w = np.ascontiguousarray(weights, dtype=np.uint8)
        s = _f32(scales)
        ng = -(-i_n // gs)
        if w.size != o_n * ((i_n + 1) // 2) or s.size != o_n * ng:
            raise CudaError("grouped int4 upload: byte/scale length mismatch")
        ok = lib().coli_cuda_tensor_upload_grouped(C.byref(h), _ptr(w), _ptr(s), i_n, o_n, gs, device)
        if ok != 1 or not h.value:
            raise CudaError(f"cuda grouped tensor_upload failed (i={i_n}, o={o_n}, gs={gs})")
        return Tensor(h, 4, i_n, o_n, device)

    def clone(self) -> "Tensor":
        """A second resident copy (device-to-device)."""
        h = C.c_void_p()
        if lib().coli_cuda_tensor_clone(C.byref(h), self.handle) != 1:
            raise CudaError("cuda tensor_clone failed")
        return Tensor(h, self.fmt, self.i_n, self.o_n, self.device)

    def update(self, weights, scales):
        w = np.ascontiguousarray(weights)
        s = None if scales is None else _f32(scales)
        if lib().coli_cuda_tensor_update(self.handle, _ptr(w), _ptr(s)) != 1:
            raise CudaError("cuda tensor_update failed")

    def bytes(self) -> int:
        return int(lib().coli_cuda_tensor_bytes(self.handle))

    def free(self):
        if self.handle is not None and self.handle.value:
            lib().coli_cuda_tensor_free(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class GpuExpert:
    """gate/up/down of one expert resident in VRAM (lib.rs:257-347)."""

    def __init__(self, gate: Tensor, up: Tensor, down: Tensor):
        self.gate, self.up, self.down = gate, up, down

    @staticmethod
    def upload(device, gate, up, down, hidden, inter) -> "GpuExpert":
        gate, up, down = _f32(gate), _f32(up), _f32(down)
        if gate.size != inter * hidden or up.size != inter * hidden or down.size != hidden * inter:
            raise CudaError("gpu expert upload: weight length mismatch")
        g = Tensor.upload(device, gate, None, 0, hidden, inter)
        u = Tensor.upload(device, up, None, 0, hidden, inter)
        d = Tensor.upload(device, down, None, 0, inter, hidden)
        return GpuExpert(g, u, d)

    @staticmethod
    def upload_int4(device, gate, up, down, hidden, inter) -> "GpuExpert":
        """Each of gate/up/down is ``(packed_nibbles, per_row_scales)``."""

        def ok(t, o, i):
            return np.asarray(t[0]).size == o * ((i + 1) // 2) and np.asarray(t[1]).size == o

        if not (ok(gate, inter, hidden) and ok(up, inter, hidden) and ok(down, hidden, inter)):
            raise CudaError("gpu int4 expert upload: byte/scale length mismatch")
        g = Tensor.upload(device, np.asarray(gate[0], np.uint8), gate[1], 2, hidden, inter)
        u = Tensor.upload(device, np.asarray(up[0], np.uint8), up[1], 2, hidden, inter)
        d = Tensor.upload(device, np.asarray(down[0], np.uint8), down[1], 2, inter, hidden)
        return GpuExpert(g, u, d)

    @staticmethod
    def upload_int4_grouped(device, gate, up, down, hidden, inter, gs) -> "GpuExpert":
        """Additive: grouped int4 ``(packed_nibbles, scales[O*ng])`` per matrix."""
        g = Tensor.upload_grouped(device, gate[0], gate[1], hidden, inter, gs)
        u = Tensor.upload_grouped(device, up[0], up[1], hidden, inter, gs)
        d = Tensor.upload_grouped(device, down[0], down[1], inter, hidden, gs)
        return GpuExpert(g, u, d)

    def clone(self) -> "GpuExpert":
        return GpuExpert(self.gate.clone(), self.up.clone(), self.down.clone())

    def free(self):
        for t in (self.gate, self.up, self.down):
            t.free()


class GroupArm(enum.Enum):
    """Which kernel arm an ``expert_group`` call reported (lib.rs:436-461)."""

    Int4Tc = 0
    W4A16 = 1
    PackedW4 = 2
    Generic = 3

    @staticmethod
    def from_c(v: int) -> "GroupArm":
        return {0: GroupArm.Int4Tc, 1: GroupArm.W4A16, 2: GroupArm.PackedW4}.get(v, GroupArm.Generic)


def _handles(experts, which):
    arr = (C.c_void_p * len(experts))()
    for i, e in enumerate(experts):
        arr[i] = getattr(e, which).handle
    return arr


def _group_dispatch(experts, rows, x, hidden, tile, want_arm):
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    if len(experts) != rows.size:
        raise CudaError("expert_group: experts/rows length mismatch")
    if np.any(rows < 0):
        raise CudaError("expert_group: negative row count")
    total = int(rows.sum())
    x = _f32(x)
    if x.size != total * hidden:
        raise CudaError("expert_group: x length != sum(rows)*hidden")
    y = np.empty((total, hidden), np.float32)
    g, u, d = _handles(experts, "gate"), _handles(experts, "up"), _handles(experts, "down")
    if tile is None and not want_arm:
        ok = lib().coli_cuda_expert_group(g, u, d, _ptr(rows), len(experts), _ptr(y), _ptr(x))
        arm = -1
    else:
        tm, tn, tk = tile if tile is not None else (0, 0, 0)
        arm_c = C.c_int(-1)
        ok = lib().coli_cuda_expert_group_tiled(g, u, d, _ptr(rows), len(experts), _ptr(y), _ptr(x), tm, tn, tk,
                                                C.byref(arm_c))
        arm = arm_c.value
    if ok != 1:
        raise CudaError("cuda expert_group failed")
    return y, arm


def expert_group(experts, rows, x, hidden) -> np.ndarray:
    """lib.rs:420-431: ``experts[k]`` processes ``rows[k]`` consecutive rows of x."""
    return _group_dispatch(experts, rows, x, hidden, None, False)[0]


def expert_group_tiled(experts, rows, x, hidden, tile=None):
    """lib.rs:463-478: returns ``(y, GroupArm)``."""
    y, arm = _group_dispatch(experts, rows, x, hidden, tile, True)
    return y, GroupArm.from_c(arm)


@dataclass
class ReduceLayout:
    """CSR of the fused reduce (lib.rs:563-610)."""

    row_ptr: np.ndarray
    row_idx: np.ndarray

    @staticmethod
    def build(dst, s_n: int):
        """Counting sort of y-row indices by destination row: each output row's
        list comes out ascending.  ``None`` when a destination is out of range."""
        dst = np.asarray(dst, dtype=np.int64)
        if dst.size and (dst.min() < 0 or dst.max() >= s_n):
            return None
        counts = np.zeros(s_n + 1, np.int32)
        for s in dst:
            counts[s + 1] += 1
        row_ptr = np.cumsum(counts, dtype=np.int32)
        fill = row_ptr.copy()
        row_idx = np.zeros(dst.size, np.int32)
        for k, s in enumerate(dst):
            row_idx[fill[s]] = k
            fill[s] += 1
        return ReduceLayout(row_ptr.astype(np.int32), row_idx)


def expert_group_reduce(experts, rows, x, hidden, layout: ReduceLayout, rw, s_n) -> np.ndarray:
    """lib.rs:612-679, with the same pre-flight checks."""
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    if len(experts) != rows.size:
        raise CudaError("expert_group_reduce: experts/rows length mismatch")
    if np.any(rows < 0):
        raise CudaError("expert_group_reduce: negative row count")
    total = int(rows.sum())
    x, rw = _f32(x), _f32(rw)
    if x.size != total * hidden:
        raise CudaError("expert_group_reduce: x length != sum(rows)*hidden")
    if rw.size != total or layout.row_idx.size != total:
        raise CudaError("expert_group_reduce: weights/row_idx length != sum(rows)")
    if s_n == 0 or layout.row_ptr.size != s_n + 1:
        raise CudaError("expert_group_reduce: row_ptr length != s_n + 1")
    if layout.row_ptr[-1] != total or layout.row_ptr[0] != 0:
        raise CudaError("expert_group_reduce: row_ptr does not span [0, sum(rows)]")
    if np.any((layout.row_idx < 0) | (layout.row_idx >= total)):
        raise CudaError("expert_group_reduce: row_idx out of range")
    out = np.empty((s_n, hidden), np.float32)
    g, u, d = _handles(experts, "gate"), _handles(experts, "up"), _handles(experts, "down")
    rp = np.ascontiguousarray(layout.row_ptr, np.int32)
    ri = np.ascontiguousarray(layout.row_idx, np.int32)
    ok = lib().coli_cuda_expert_group_reduce(g, u, d, _ptr(rows), len(experts), _ptr(rp), _ptr(ri), _ptr(rw), s_n,
                                             _ptr(out), _ptr(x))
    if ok != 1:
        raise CudaError("cuda expert_group_reduce failed")
    return out


# ----------------------------------------------------- device-resident layer
class MoeLayer:
    """Router + routed experts (+ shared expert) resident on one device.

    Mirrors the arguments of the reference's ``moe_forward``
    (crates/peregrine-model/src/mlp.rs:46-57): ``forward(x)`` returns
    ``out[M, D]`` for host rows; ``forward_dev`` takes device pointers and does
    not synchronise."""

    def __init__(self, device, hidden, inter, n_experts, k, norm_topk, routed_scale, router_w, router_bias=None):
        self.device, self.hidden, self.inter, self.n_experts, self.k = device, hidden, inter, n_experts, k
        rw = _f32(router_w)
        if rw.size != n_experts * hidden:
            raise CudaError("moe layer: router weight length mismatch")
        rb = None if router_bias is None else _f32(router_bias)
        h = C.c_void_p(None)
        ok = lib().coli_cuda_moe_layer_create(C.byref(h), device, hidden, inter, n_experts, k, int(bool(norm_topk)),
                                              C.c_float(routed_scale), _ptr(rw), _ptr(rb))
        if ok != 1 or not h.value:
            raise CudaError("cuda moe_layer_create failed")
        self.handle = h
        self._experts = {}

    def set_expert(self, e: int, expert: GpuExpert):
        if lib().coli_cuda_moe_layer_set_expert(self.handle, e, expert.gate.handle, expert.up.handle,
                                                expert.down.handle) != 1:
            raise CudaError(f"cuda moe_layer_set_expert({e}) failed")
        self._experts[e] = expert  # keep the tensors alive

    def set_shared(self, expert: GpuExpert):
        self.set_expert(self.n_experts, expert)

    def forward(self, x, out: np.ndarray | None = None) -> np.ndarray:
        """Blocking layer step on host rows.  With ``out`` (C-contiguous fp32 of x's shape) and a
        C-contiguous fp32 ``x`` no array is allocated or converted on the way in."""
        if out is None or x.dtype != np.float32 or not x.flags.c_contiguous:
            x = _f32(x).reshape(-1, self.hidden)
            if out is None:
                out = np.empty_like(x)
        if out.dtype != np.float32 or not out.flags.c_contiguous or out.size != x.size:
            raise ValueError("moe layer forward: out must be C-contiguous fp32 of x's size")
        if lib().coli_cuda_moe_layer_forward(self.handle, out.ctypes.data, x.ctypes.data,
                                             x.size // self.hidden) != 1:
            raise CudaError("cuda moe_layer_forward failed")
        return out

    def host_times(self, reset: bool = True):
        """Mean host-side microseconds per blocking ``forward`` since the last reset, by part."""
        us = (C.c_double * 5)()
        n = C.c_uint64(0)
        lib().coli_cuda_moe_layer_host_times(self.handle, us, C.byref(n), int(reset))
        names = ("stage_x", "enqueue_upload", "enqueue_launches", "wait_device", "copy_out")
        return {k: us[j] / max(n.value, 1) for j, k in enumerate(names)}, int(n.value)

    def forward_dev(self, out_ptr: int, x_ptr: int, m: int):
        if lib().coli_cuda_moe_layer_forward_dev(self.handle, C.c_void_p(out_ptr), C.c_void_p(x_ptr), m) != 1:
            raise CudaError("cuda moe_layer_forward_dev failed")

    def last_routing(self, m: int):
        idx = np.zeros((m, self.k), np.int32)
        w = np.zeros((m, self.k), np.float32)
        keff = np.zeros(m, np.int32)
        uni = np.zeros(self.n_experts + 1, np.int32)
        nu = C.c_int(0)
        if lib().coli_cuda_moe_layer_last_routing(self.handle, m, _ptr(idx), _ptr(w), _ptr(keff), _ptr(uni),
                                                  C.byref(nu)) != 1:
            raise CudaError("cuda moe_layer_last_routing failed")
        return idx, w, keff, uni[: nu.value].copy()

    def enable_taps(self, on: bool = True):
        lib().coli_cuda_moe_layer_enable_taps(self.handle, int(on))

    def set_spec(self, mode: int):
        """Speculative routing of decode-sized batches: -1 default, 0 off, 1 on, 2 on with a wrong guess."""
        if lib().coli_cuda_moe_layer_set_spec(self.handle, int(mode)) != 1:
            raise CudaError("cuda moe_layer_set_spec failed")

    def set_bias(self, bias):
        b = _f32(bias)
        if b.size != self.n_experts or lib().coli_cuda_moe_layer_set_bias(self.handle, _ptr(b)) != 1:
            raise CudaError("cuda moe_layer_set_bias failed")

    def set_fused(self, mode: int):
        """-1 process default, 0 separate launches, 1 the single-launch decode step (one token)."""
        if lib().coli_cuda_moe_layer_set_fused(self.handle, mode) != 1:
            raise CudaError("cuda moe_layer_set_fused failed")

    def decode_timeline(self, enable: bool = True, read: bool = False):
        """Switches the timeline of the single-launch step on/off; with ``read`` returns
        ``(stamps [n_ctas, 16] uint64 ns, n_chain)`` of the last such step."""
        n, nc = C.c_int(0), C.c_int(0)
        if lib().coli_cuda_moe_layer_decode_timeline(self.handle, int(enable), None, 0, C.byref(n), C.byref(nc)) != 1:
            raise CudaError("cuda moe_layer_decode_timeline failed")
        if not read:
            return None
        out = np.zeros((n.value, 16), np.uint64)
        if lib().coli_cuda_moe_layer_decode_timeline(self.handle, int(enable), _ptr(out), n.value, None, None) != 1:
            raise CudaError("cuda moe_layer_decode_timeline read failed")
        return out, nc.value

    def last_pairs(self, m: int):
        cap = m * (self.k + 1)
        tok = np.zeros(cap, np.int32)
        exp = np.zeros(cap, np.int32)
        n = C.c_int(0)
        if lib().coli_cuda_moe_layer_last_pairs(self.handle, C.byref(n), _ptr(tok), _ptr(exp), cap) != 1:
            raise CudaError("cuda moe_layer_last_pairs failed")
        return tok[: n.value].copy(), exp[: n.value].copy()

    def read_taps(self, n_pairs: int, ng_gateup: int, ng_down: int):
        gu = np.zeros((n_pairs, 2, self.inter, ng_gateup), np.int32)
        dn = np.zeros((n_pairs, self.hidden, ng_down), np.int32)
        if lib().coli_cuda_moe_layer_read_taps(self.handle, _ptr(gu), gu.size, _ptr(dn), dn.size) != 1:
            raise CudaError("cuda moe_layer_read_taps failed")
        return gu, dn

    # ---- expert parallelism (see include/peregrine_b200.h)
    def set_ep(self, rank: int, world: int):
        if lib().coli_cuda_moe_layer_set_ep(self.handle, rank, world) != 1:
            raise CudaError("cuda moe_layer_set_ep failed")
        self.ep_rank, self.ep_world = rank, world

    def owned_experts(self):
        world, rank = getattr(self, "ep_world", 1), getattr(self, "ep_rank", 0)
        per = -(-self.n_experts // world)
        return range(min(rank * per, self.n_experts), min((rank + 1) * per, self.n_experts))

    # profile mode: names of the seven bracketed stages of a step made of separate launches.
    # "join_repair_or_qrow_h": with speculative routing the wait for the exact plan plus the repair
    # launch; otherwise the separate quantiser of h when the down launch cannot stage it itself
    STAGES = ("qrow_x_unfused", "route", "route_plan_unfused", "gemv_gateup", "join_repair_or_qrow_h", "gemv_down",
              "unused")

    def set_profile(self, on: bool):
        if lib().coli_cuda_moe_layer_set_profile(self.handle, int(on)) != 1:
            raise CudaError("cuda moe_layer_set_profile failed")

    def profile(self):
        """Accumulated device ms per stage and the number of profiled forwards."""
        ms = (C.c_double * 7)()
        n = C.c_uint64(0)
        lib().coli_cuda_moe_layer_profile(self.handle, ms, C.byref(n))
        return dict(zip(self.STAGES, list(ms))), n.value

    def free(self):
        if getattr(self, "handle", None) is not None and self.handle.value:
            lib().coli_cuda_moe_layer_free(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
