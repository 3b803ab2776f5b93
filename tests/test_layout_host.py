"""CPU checks of the host logic: tile-stream layout, repacker and the per-lane
integer arithmetic of the GEMV walk, against the oracle (bit-exact)."""
import numpy as np
import pytest

import oracle as po
from tests import hostcheck as hc


def rand_matrix(rng, O, K, grouped, gs):
    q = rng.integers(0, 256, size=O * ((K + 1) // 2), dtype=np.uint8)
    if K % 2:  # the unused high nibble of each row's last byte is zero in the container
        q.reshape(O, -1)[:, -1] &= 0x0F
    ng = -(-K // gs) if grouped else 1
    sc = (np.abs(rng.standard_normal(O * ng)) * 0.02 + 1e-4).astype(np.float32)
    return q, sc


SHAPES = [
    (16, 32, True, 32), (33, 96, True, 32), (40, 100, True, 32), (7, 257, True, 32), (64, 256, True, 64),
    (20, 384, True, 128), (17, 300, True, 128), (9, 512, True, 256),
    (16, 32, False, 0), (33, 96, False, 0), (5, 70, False, 0), (48, 257, False, 0), (1, 1, False, 0),
]


@pytest.mark.parametrize("O,K,grouped,gs", SHAPES)
def test_repack_roundtrip(O, K, grouped, gs):
    rng = np.random.default_rng(O * 1000 + K)
    q, sc = rand_matrix(rng, O, K, grouped, gs)
    stream, rs, L = hc.repack(q, sc, O, K, grouped, gs)
    assert L["total_bytes"] == L["ntile"] * L["nchunk"] * L["chunk_bytes"]
    assert L["chunk_bytes"] <= 2560 and L["chunk_bytes"] % 16 == 0 and L["kp"] == L["nchunk"] * 256
    assert L["gpc"] * L["bpg"] == 8 and (not grouped or L["nchunk"] * L["gpc"] >= L["ng_src"])
    rb = (K + 1) // 2
    for o in rng.integers(0, O, size=min(O, 8)):
        for k in rng.integers(0, K, size=min(K, 40)):
            byte = q[o * rb + (k >> 1)]
            want = (byte >> 4) if (k & 1) else (byte & 0x0F)
            assert hc.nibble(stream, O, K, grouped, gs, int(o), int(k)) == want
    # padding elements decode to nibble 8 (value 0)
    if L["kp"] > K:
        assert hc.nibble(stream, O, K, grouped, gs, 0, K) == 8


def test_repack_threads_agree():
    rng = np.random.default_rng(5)
    O, K = 512, 4096
    q, sc = rand_matrix(rng, O, K, True, 32)
    a, _, _ = hc.repack(q, sc, O, K, True, 32, threads=1)
    b, _, _ = hc.repack(q, sc, O, K, True, 32, threads=4)
    assert np.array_equal(a, b)


@pytest.mark.parametrize("O,K,grouped,gs", SHAPES)
def test_walk_matches_oracle(O, K, grouped, gs):
    rng = np.random.default_rng(O * 7 + K)
    q, sc = rand_matrix(rng, O, K, grouped, gs)
    stream, rs, L = hc.repack(q, sc, O, K, grouped, gs)
    nrows = 3
    x = rng.standard_normal((nrows, K)).astype(np.float32)
    xq = np.zeros((nrows, L["kp"]), np.int8)
    cs = np.zeros((nrows, L["nblk"]), np.int32)
    sx = np.zeros(nrows, np.float32)
    for r in range(nrows):
        xq[r], sx[r], cs[r] = hc.qrow(x[r], L)
        oq, os_ = po.qrow_i8(x[r])
        assert np.array_equal(xq[r, :K], oq) and sx[r] == os_ and not xq[r, K:].any()
    y, tap = hc.walk(stream, rs, L, xq, cs, sx, nrows, want_tap=True)
    xq_nat = np.ascontiguousarray(xq[:, :K])
    if grouped:
        want, blocks = po.matmul_i4g_idot(xq_nat, sx, q, sc, nrows, K, O, gs, want_blocks=True)
        assert np.array_equal(tap, blocks)
    else:
        want, acc = po.matmul_i4_idot(xq_nat, sx, q, sc, nrows, K, O, want_acc=True)
        assert np.array_equal(tap[:, :, 0], acc)
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32))


def test_layout_rejects_bad_group_sizes():
    assert hc.layout(16, 64, True, 16) is None
    assert hc.layout(16, 64, True, 48) is None
    assert hc.layout(16, 64, True, 96) is None
    assert hc.layout(16, 1024, True, 512) is None
    L = hc.layout(2048, 6144, True, 32)  # the benchmark's gate matrix: no padding, container-sized
    assert L["total_bytes"] == 2048 * 6144 // 2 + 2048 * 6144 // 32 * 4 and L["nchunk"] == 24
