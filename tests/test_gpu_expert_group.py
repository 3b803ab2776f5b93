"""Parity of the reference ABI's expert-group calls with the CPU oracle.

Modelled on the reference's own GPU tests (crates/peregrine-cuda/src/lib.rs:823-1624)
with the tolerance tightened: the int4 paths here follow the CPU integer-dot
arithmetic, so they are compared bit for bit.
"""
import numpy as np
import pytest

import oracle as po
from peregrine_b200 import cuda
from peregrine_b200.resident import upload_expert
from peregrine_b200.synth import synth_expert
from tests.gpu_common import bits
from tests.refmodel import o_expert

pytestmark = pytest.mark.gpu


def oracle_group(experts, rows, x, hidden):
    out, r0 = [], 0
    for ex, n in zip(experts, rows):
        g, u, d = o_expert(ex)
        out.append(po.swiglu(g, u, d, x[r0:r0 + n], n))
        r0 += n
    return np.concatenate(out, 0)


@pytest.mark.parametrize("hidden,inter,gs,rows", [
    (64, 32, 0, [1]),
    (96, 40, 0, [2, 1, 3]),           # ragged: K not a multiple of 32 on the down side, O not of 16
    (70, 33, 0, [1, 5]),              # odd K: last byte half used
    (256, 128, 32, [1, 1, 1]),
    (288, 96, 32, [4, 2, 9, 1]),      # 9 rows: more than one pass at RMAX=8
    (384, 256, 128, [3, 1]),
    (512, 256, 256, [2]),
    (2048, 1024, 32, [1, 2]),         # configs[0] expert shape
])
def test_int4_group_is_bit_exact(dev, hidden, inter, gs, rows):
    rng = np.random.default_rng(hidden * 31 + inter + gs)
    exs = [synth_expert(rng, hidden, inter, gs) for _ in rows]
    gpu = [upload_expert(dev, e, hidden, inter) for e in exs]
    x = rng.standard_normal((sum(rows), hidden)).astype(np.float32)
    want = oracle_group(exs, rows, x, hidden)
    got = cuda.expert_group(gpu, rows, x, hidden)
    again = cuda.expert_group(gpu, rows, x, hidden)
    assert np.array_equal(bits(got), bits(want))
    assert np.array_equal(bits(got), bits(again))  # run-to-run identical
    assert cuda.last_device_error(dev) == 0
    for e in gpu:
        e.free()


def test_many_experts_one_row_each(dev):
    # crates/peregrine-cuda/src/lib.rs:1579-1623: more than 64 experts in one call
    hidden, inter, n = 64, 32, 70
    rng = np.random.default_rng(70)
    exs = [synth_expert(rng, hidden, inter, 32) for _ in range(n)]
    gpu = [upload_expert(dev, e, hidden, inter) for e in exs]
    x = rng.standard_normal((n, hidden)).astype(np.float32)
    got = cuda.expert_group(gpu, [1] * n, x, hidden)
    assert np.array_equal(bits(got), bits(oracle_group(exs, [1] * n, x, hidden)))


def test_int4_close_to_dequantised_f32(dev):
    # crates/peregrine-cuda/src/lib.rs:884-917: int4 result within 3e-2*max(|y|,1) of the f32
    # SwiGLU on the dequantised weights
    hidden, inter = 128, 64
    rng = np.random.default_rng(9)
    w = [rng.standard_normal((inter, hidden)).astype(np.float32) * 0.1,
         rng.standard_normal((inter, hidden)).astype(np.float32) * 0.1,
         rng.standard_normal((hidden, inter)).astype(np.float32) * 0.1]
    q = [po.quant_i4(w[0], inter, hidden), po.quant_i4(w[1], inter, hidden), po.quant_i4(w[2], hidden, inter)]
    ex = cuda.GpuExpert.upload_int4(dev, q[0], q[1], q[2], hidden, inter)

    def deq(qs, o, i):
        b = qs[0].reshape(o, -1)
        v = np.empty((o, i), np.float32)
        v[:, 0::2] = (b & 0x0F)[:, : (i + 1) // 2].astype(np.float32) - 8
        v[:, 1::2] = (b >> 4)[:, : i // 2].astype(np.float32) - 8
        return v * qs[1][:, None]

    g, u, d = deq(q[0], inter, hidden), deq(q[1], inter, hidden), deq(q[2], hidden, inter)
    x = rng.standard_normal((3, hidden)).astype(np.float32)
    gg, uu = x @ g.T, x @ u.T
    ref = ((gg / (1 + np.exp(-gg))) * uu) @ d.T
    got = cuda.expert_group([ex], [3], x, hidden)
    assert np.all(np.abs(got - ref) <= 3e-2 * np.maximum(np.abs(ref), 1.0))


def test_f32_and_mixed_groups(dev):
    # crates/peregrine-cuda/src/lib.rs:1553-1576: f32 group vs CPU within 1e-3
    hidden, inter = 96, 48
    rng = np.random.default_rng(3)
    mats = [rng.standard_normal((inter, hidden)).astype(np.float32) * 0.1,
            rng.standard_normal((inter, hidden)).astype(np.float32) * 0.1,
            rng.standard_normal((hidden, inter)).astype(np.float32) * 0.1]
    f32 = cuda.GpuExpert.upload(dev, mats[0], mats[1], mats[2], hidden, inter)
    i4s = synth_expert(rng, hidden, inter, 0)
    i4 = upload_expert(dev, i4s, hidden, inter)
    x = rng.standard_normal((5, hidden)).astype(np.float32)
    got = cuda.expert_group([f32, i4, f32], [2, 2, 1], x, hidden)

    def f32_ref(xr):
        gg, uu = xr @ mats[0].T, xr @ mats[1].T
        return ((gg / (1 + np.exp(-gg))) * uu) @ mats[2].T

    assert np.allclose(got[0:2], f32_ref(x[0:2]), rtol=1e-3, atol=1e-3)
    assert np.allclose(got[4:5], f32_ref(x[4:5]), rtol=1e-3, atol=1e-3)
    assert np.array_equal(bits(got[2:4]), bits(oracle_group([i4s], [2], x[2:4], hidden)))


def test_fused_reduce_matches_host_reduce_and_is_stable(dev):
    # crates/peregrine-cuda/src/lib.rs:1478-1550
    hidden, inter = 128, 64
    rng = np.random.default_rng(11)
    exs = [synth_expert(rng, hidden, inter, 32) for _ in range(3)]
    gpu = [upload_expert(dev, e, hidden, inter) for e in exs]
    rows = [2, 2, 1]
    dst = [0, 1, 0, 1, 0]
    rw = rng.random(5).astype(np.float32)
    x = rng.standard_normal((5, hidden)).astype(np.float32)
    lay = cuda.ReduceLayout.build(dst, 2)
    y = cuda.expert_group(gpu, rows, x, hidden)
    outs = [cuda.expert_group_reduce(gpu, rows, x, hidden, lay, rw, 2) for _ in range(3)]
    assert np.array_equal(bits(outs[0]), bits(outs[1])) and np.array_equal(bits(outs[0]), bits(outs[2]))
    want = np.zeros((2, hidden), np.float32)
    for s in range(2):
        for j in range(lay.row_ptr[s], lay.row_ptr[s + 1]):
            kx = lay.row_idx[j]
            want[s] = want[s] + (rw[kx] * y[kx]).astype(np.float32)
    assert np.array_equal(bits(outs[0]), bits(want))


def test_stats_arm_codes_and_validation(dev, monkeypatch):
    hidden, inter = 64, 32
    rng = np.random.default_rng(5)
    ex = upload_expert(dev, synth_expert(rng, hidden, inter, 32), hidden, inter)
    before = cuda.group_stats()
    x = rng.standard_normal((16, hidden)).astype(np.float32)
    y, arm = cuda.expert_group_tiled([ex], [16], x, hidden, None)
    assert arm == cuda.GroupArm.PackedW4
    monkeypatch.setenv("COLI_CUDA_TC_W4A16", "1")
    for tile in (None, (16, 16, 16), (32, 8, 16), (8, 32, 16)):
        y2, arm2 = cuda.expert_group_tiled([ex], [16], x, hidden, tile)
        assert arm2 == cuda.GroupArm.W4A16
        assert np.array_equal(bits(y2), bits(y))
    monkeypatch.delenv("COLI_CUDA_TC_W4A16")
    after = cuda.group_stats()
    assert after.calls == before.calls + 5 and after.experts == before.experts + 5
    assert after.rows == before.rows + 80
    # shape and argument validation: failure, not a fault
    with pytest.raises(cuda.CudaError):
        cuda.expert_group([ex], [0], x[:0], hidden)
    other = upload_expert(dev, synth_expert(rng, 32, 32, 32), 32, 32)
    with pytest.raises(cuda.CudaError):
        cuda.expert_group([ex, other], [1, 1], x[:2], hidden)
    with pytest.raises(cuda.CudaError):
        cuda.expert_group([ex] * 257, [1] * 257, np.zeros((257, hidden), np.float32), hidden)


def test_upload_is_idempotent_and_counts(dev):
    import ctypes as C
    lib = cuda.lib()
    rng = np.random.default_rng(1)
    q = rng.integers(0, 256, 32 * 16, dtype=np.uint8)
    sc = np.ones(32, np.float32)
    n0, b0 = C.c_size_t(0), C.c_size_t(0)
    lib.coli_cuda_stats(dev, C.byref(n0), C.byref(b0))
    t = cuda.Tensor.upload(dev, q, sc, 2, 32, 32)
    n1, b1 = C.c_size_t(0), C.c_size_t(0)
    lib.coli_cuda_stats(dev, C.byref(n1), C.byref(b1))
    assert n1.value == n0.value + 1 and b1.value == b0.value + t.bytes()
    # a second upload into a set handle reports the shape match and copies nothing
    assert lib.coli_cuda_tensor_upload(C.byref(t.handle), q.ctypes.data, sc.ctypes.data, 2, 32, 32, dev) == 1
    assert lib.coli_cuda_tensor_upload(C.byref(t.handle), q.ctypes.data, sc.ctypes.data, 2, 64, 32, dev) == 0
    assert lib.coli_cuda_tensor_device(t.handle) == dev
    t.free()
