"""Caller-side contracts of the GPU lane, replayed through the C ABI:

* the shape-cache counters of the expert-group call under COLI_CUDA_GRAPH=1
  (crates/peregrine-cuda/src/lib.rs:963-1126),
* the tier's job-list calls (crates/peregrine-model/src/gpu.rs:1896-2090): results in job order for
  a mixed int4 / f32 residency, from a checkpoint written in the container format,
* the single-matrix device call coli_cuda_pipe_gemm against the oracle's Weight.apply.
"""
import ctypes as C

import numpy as np
import pytest

import oracle as po
from peregrine_b200 import cuda
from peregrine_b200.container import SafeTensors, expert_names, write_safetensors
from peregrine_b200.gpu_tier import GpuTier
from peregrine_b200.synth import synth_matrix
from tests.gpu_common import bits

pytestmark = pytest.mark.gpu


def lcg_floats(seed, n):
    """crates/peregrine-model/src/testkit.rs:10-16."""
    out = np.empty(n, np.float32)
    s = seed & 0xFFFFFFFFFFFFFFFF
    for i in range(n):
        s = (s * 6364136223846793005 + 1442695040888963407) & 0xFFFFFFFFFFFFFFFF
        out[i] = np.float32(np.float32(s >> 40) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0))
    return out


def int4_expert(dev, seed, hidden, inter):
    """crates/peregrine-cuda/src/lib.rs:950-960."""
    f = lcg_floats(seed, 3 * hidden * inter) * np.float32(0.1)
    g = po.quant_i4(f[:inter * hidden].reshape(inter, hidden), inter, hidden)
    u = po.quant_i4(f[inter * hidden:2 * inter * hidden].reshape(inter, hidden), inter, hidden)
    d = po.quant_i4(f[2 * inter * hidden:].reshape(hidden, inter), hidden, inter)
    return cuda.GpuExpert.upload_int4(dev, g, u, d, hidden, inter)


def group(monkeypatch, knob, experts, rows, x, hidden):
    monkeypatch.setenv("COLI_CUDA_GRAPH", "1" if knob else "0")
    return cuda.expert_group(experts, rows, x, hidden)


def test_graph_knob_first_call_captures_repeat_replays(dev, monkeypatch):
    hidden, inter, n = 64, 32, 2
    e = int4_expert(dev, 0x9001, hidden, inter)
    x = lcg_floats(0x51DE, n * hidden).reshape(n, hidden)
    eager = group(monkeypatch, False, [e], [n], x, hidden)
    before = cuda.graph_cache_stats()
    captured = group(monkeypatch, True, [e], [n], x, hidden)
    replayed = group(monkeypatch, True, [e], [n], x, hidden)
    after = cuda.graph_cache_stats()
    assert np.array_equal(bits(eager), bits(captured)) and np.array_equal(bits(eager), bits(replayed))
    assert after.captures > before.captures
    assert after.replays > before.replays
    e.free()


def test_grown_scratch_invalidates_cached_shapes(dev, monkeypatch):
    big_rows = 4096  # larger than any shape another test of this process sends through expert_group
    hidden, inter = 64, 32
    e = int4_expert(dev, 0x9002, hidden, inter)
    small = lcg_floats(0x6120, hidden).reshape(1, hidden)
    big = lcg_floats(0x6121, big_rows * hidden).reshape(big_rows, hidden)
    want_small = group(monkeypatch, False, [e], [1], small, hidden)
    before = cuda.graph_cache_stats()
    group(monkeypatch, True, [e], [1], small, hidden)
    got_big = group(monkeypatch, True, [e], [big_rows], big, hidden)
    got_small = group(monkeypatch, True, [e], [1], small, hidden)
    after = cuda.graph_cache_stats()
    want_big = group(monkeypatch, False, [e], [big_rows], big, hidden)
    assert np.array_equal(bits(want_big), bits(got_big))
    assert np.array_equal(bits(want_small), bits(got_small))
    assert after.invalidations > before.invalidations
    e.free()


def test_replay_uses_current_experts_and_w4a16_is_uncacheable(dev, monkeypatch):
    hidden, inter, n = 64, 32, 2
    a, b = int4_expert(dev, 0xA1, hidden, inter), int4_expert(dev, 0xB2, hidden, inter)
    x = lcg_floats(0xD1FF, n * hidden).reshape(n, hidden)
    want_a = group(monkeypatch, False, [a], [n], x, hidden)
    want_b = group(monkeypatch, False, [b], [n], x, hidden)
    assert not np.array_equal(want_a, want_b)
    assert np.array_equal(bits(group(monkeypatch, True, [a], [n], x, hidden)), bits(want_a))
    assert np.array_equal(bits(group(monkeypatch, True, [b], [n], x, hidden)), bits(want_b))
    # the arm the reference never caches: counted, not captured
    x24 = lcg_floats(0x16A1, 24 * hidden).reshape(24, hidden)
    monkeypatch.setenv("COLI_CUDA_TC_W4A16", "1")
    before = cuda.graph_cache_stats()
    group(monkeypatch, True, [a], [24], x24, hidden)
    after = cuda.graph_cache_stats()
    monkeypatch.delenv("COLI_CUDA_TC_W4A16")
    assert after.captures == before.captures
    assert after.uncacheable > before.uncacheable
    a.free()
    b.free()


def write_checkpoint(path, layer, hidden, inter, formats, seed):
    """Experts 0..len(formats)-1 of one layer in the container format: 'row' = per-row int4,
    'g128' = grouped int4 with group 128, 'i8' = per-row int8."""
    rng = np.random.default_rng(seed)
    tensors, mats = {}, {}
    for e, kind in enumerate(formats):
        for name, (o, i) in zip(expert_names(layer, e), ((inter, hidden), (inter, hidden), (hidden, inter))):
            w = (rng.standard_normal((o, i)) * 0.1).astype(np.float32)
            if kind == "row":
                q, s = po.quant_i4(w, o, i)
                gs = 0
            elif kind == "g128":
                q, s = po.quant_i4_grouped(w, o, i, 128)
                gs = 128
            else:
                amax = np.abs(w).max(axis=1)
                s = np.maximum(amax / 127.0, 1e-12).astype(np.float32)
                q = np.rint(w / s[:, None]).clip(-127, 127).astype(np.int8).view(np.uint8).reshape(-1)
                gs = -1
            tensors[name] = q.reshape(o, -1)
            tensors[name + ".qs"] = s
            mats[name] = (q, s, gs, o, i)
    write_safetensors(path, tensors)
    return mats


def test_tier_compute_returns_job_order_for_mixed_residency(dev, tmp_path):
    hidden, inter, layer = 256, 128, 3
    formats = ["row", "i8", "g128", "row", "i8"]
    f = str(tmp_path / "model.safetensors")
    mats = write_checkpoint(f, layer, hidden, inter, formats, seed=21)
    st = SafeTensors(str(tmp_path))
    tier = GpuTier(dev, hidden, inter)
    kept = [tier.upload_expert(st, layer, e) for e in range(len(formats))]
    assert kept == [True, False, True, True, False]  # grouped int4 stays packed; int8 goes to fp32
    rng = np.random.default_rng(5)
    jobs = [(4, rng.standard_normal(2 * hidden).astype(np.float32)),
            (0, rng.standard_normal(1 * hidden).astype(np.float32)),
            (2, rng.standard_normal(3 * hidden).astype(np.float32)),
            (1, rng.standard_normal(1 * hidden).astype(np.float32)),
            (3, rng.standard_normal(2 * hidden).astype(np.float32))]
    outs = tier.compute(layer, jobs, hidden)
    assert len(outs) == len(jobs)

    def weight(name):
        q, s, gs, o, i = mats[name]
        return po.Weight(q.reshape(-1), s, 4 if gs > 0 else 2, max(gs, 0), i, o)

    for (e, xg), y in zip(jobs, outs):
        nr = xg.size // hidden
        assert y.size == nr * hidden
        gn, un, dn = expert_names(layer, e)
        if formats[e] == "i8":
            def deq(name):
                q, s, _, o, i = mats[name]
                return q.view(np.int8).reshape(o, i).astype(np.float32) * s[:, None]
            x = xg.reshape(nr, hidden)
            gg, uu = x @ deq(gn).T, x @ deq(un).T
            ref = ((gg / (1 + np.exp(-gg))) * uu) @ deq(dn).T
            assert np.allclose(y.reshape(nr, hidden), ref, rtol=1e-3, atol=1e-3)
        else:
            want = po.swiglu(weight(gn), weight(un), weight(dn), xg.reshape(nr, hidden), nr)
            assert np.array_equal(bits(y.reshape(nr, hidden)), bits(want))  # int4 residency: bit-exact
    # the fused-reduce form: equals reducing compute()'s rows on the host, class by class
    dst = [0, 1, 2, 0, 1, 2, 0, 1, 2]
    wts = rng.random(9).astype(np.float32)
    got = tier.compute_reduced(layer, jobs, hidden, dst, wts, 3)
    again = tier.compute_reduced(layer, jobs, hidden, dst, wts, 3)
    assert np.array_equal(bits(got), bits(again))
    flat = np.concatenate([o.reshape(-1, hidden) for o in outs])
    want = np.zeros((3, hidden), np.float32)
    for r, (d, w) in enumerate(zip(dst, wts)):
        want[d] += w * flat[r]
    assert np.allclose(got, want, rtol=1e-4, atol=1e-4)
    with pytest.raises(cuda.CudaError):
        tier.compute(layer, [(9, jobs[0][1])], hidden)            # not resident
    with pytest.raises(cuda.CudaError):
        tier.compute(layer, [(0, jobs[0][1][:-1])], hidden)       # ragged rows
    tier.free()


class DevArray:
    def __init__(self, dev, host=None, nbytes=None):
        self.dev = dev
        self.nbytes = host.nbytes if host is not None else nbytes
        self.ptr = cuda.lib().coli_cuda_pipe_alloc(dev, self.nbytes)
        assert self.ptr
        if host is not None:
            host = np.ascontiguousarray(host)
            assert cuda.lib().coli_cuda_pipe_upload(dev, self.ptr, host.ctypes.data, host.nbytes) == 1

    def read(self, shape, dtype=np.float32):
        out = np.empty(shape, dtype)
        assert cuda.lib().coli_cuda_pipe_download(self.dev, self.ptr, out.ctypes.data, out.nbytes) == 1
        return out

    def free(self):
        cuda.lib().coli_cuda_pipe_free(self.dev, self.ptr)


@pytest.mark.parametrize("gs", [32, 0])
@pytest.mark.parametrize("rows", [1, 2, 7, 17])
def test_pipe_gemm_matches_oracle_weight_apply(dev, gs, rows):
    """y = x W^T through the device-pointer call, bit for bit against the CPU matmul
    (crates/peregrine-kernels/src/matmul.rs:75-124): dp4a kernel (1-2 rows), tensor-core kernel
    with one (7) and two (17) row passes."""
    lib = cuda.lib()
    rng = np.random.default_rng(1000 + gs + rows)
    i_n, o_n = 352, 200
    m = synth_matrix(rng, o_n, i_n, gs)
    t = (cuda.Tensor.upload_grouped(dev, m.q, m.scale, i_n, o_n, gs) if gs
         else cuda.Tensor.upload(dev, m.q, m.scale, 2, i_n, o_n))
    x = rng.standard_normal((rows, i_n)).astype(np.float32)
    xd, yd = DevArray(dev, x), DevArray(dev, nbytes=rows * o_n * 4)
    assert lib.coli_cuda_pipe_gemm(t.handle, C.c_void_p(yd.ptr), C.c_void_p(xd.ptr), rows) == 1
    want = po.Weight(m.q, m.scale, 4 if gs else 2, gs, i_n, o_n).apply(x, rows)
    assert np.array_equal(bits(yd.read((rows, o_n))), bits(want))
    assert cuda.last_device_error(dev) == 0
    xd.free()
    yd.free()
    t.free()


def test_pipe_gemm_inside_a_captured_graph(dev):
    """The reference treats the pipe calls as capturable (cuda/backend_cuda.cu:1532-1535): after one
    eager call has sized the scratch, the same call recorded between graph_begin / graph_end and
    replayed twice with x changed in place gives the eager result each time."""
    lib = cuda.lib()
    rng = np.random.default_rng(44)
    i_n, o_n, rows = 256, 96, 2
    m = synth_matrix(rng, o_n, i_n, 32)
    t = cuda.Tensor.upload_grouped(dev, m.q, m.scale, i_n, o_n, 32)
    xs = [rng.standard_normal((rows, i_n)).astype(np.float32) for _ in range(3)]
    xd, yd = DevArray(dev, xs[0]), DevArray(dev, nbytes=rows * o_n * 4)
    assert lib.coli_cuda_pipe_gemm(t.handle, C.c_void_p(yd.ptr), C.c_void_p(xd.ptr), rows) == 1  # sizes scratch
    assert lib.coli_cuda_pipe_sync(dev) == 1
    assert lib.coli_cuda_graph_begin(dev) == 1
    rc = lib.coli_cuda_pipe_gemm(t.handle, C.c_void_p(yd.ptr), C.c_void_p(xd.ptr), rows)
    g = C.c_void_p()
    assert lib.coli_cuda_graph_end(dev, C.byref(g)) == 1 and rc == 1 and g
    ow = po.Weight(m.q, m.scale, 4, 32, i_n, o_n)
    for x in xs[1:]:
        assert lib.coli_cuda_pipe_upload(dev, xd.ptr, x.ctypes.data, x.nbytes) == 1
        assert lib.coli_cuda_graph_launch(g) == 1
        assert np.array_equal(bits(yd.read((rows, o_n))), bits(ow.apply(x, rows)))
    lib.coli_cuda_graph_free(g)
    xd.free()
    yd.free()
    t.free()
