"""Host-side mirrors on CPU: the tier's partition / scatter helpers against the reference's own
vectors (crates/peregrine-model/src/gpu.rs:898-949) and container-format detection against the
reference's detection tests (crates/peregrine-core/src/qt.rs:183-290)."""
import numpy as np

from peregrine_b200.container import (QtFmt, QtInfo, QtWeight, SafeTensors, ContainerError, detect_group_size,
                                      write_safetensors)
from peregrine_b200.gpu_tier import partition_by_format, scatter_by_index


def test_homogeneous_group_makes_one_class():
    assert partition_by_format([True, True, True]) == [[0, 1, 2]]
    assert partition_by_format([False, False]) == [[0, 1]]
    assert partition_by_format([]) == []
    assert partition_by_format([True]) == [[0]]


def test_mixed_group_splits_preserving_relative_order():
    assert partition_by_format([True, False, True, False, True]) == [[0, 2, 4], [1, 3]]


def test_scatter_inverts_partition_exactly():
    for fmt in ([True, False, True, False, True], [True] * 4, [False] * 4, [False, True], [True]):
        classes = partition_by_format(fmt)
        per_class = [list(c) for c in classes]
        assert scatter_by_index(len(fmt), classes, per_class) == list(range(len(fmt)))


def test_scatter_rejects_malformed_input_instead_of_misaligning():
    classes = [[0, 2], [1]]
    assert scatter_by_index(3, classes, [[0, 2]]) is None            # wrong number of result groups
    assert scatter_by_index(3, classes, [[0], [1]]) is None          # group length mismatch
    assert scatter_by_index(2, classes, [[0, 2], [1]]) is None       # index out of range
    assert scatter_by_index(3, [[0, 0], [1]], [[0, 0], [1]]) is None  # duplicate index leaves a hole


def test_group_size_probe():
    assert detect_group_size(2, 32, 4) == 16
    assert detect_group_size(2, 32, 2) == 0
    assert detect_group_size(2, 64, 4) == 32
    assert detect_group_size(4, 8, 100) == 0


def test_detect_formats(tmp_path):
    o, i = 2, 32
    f = str(tmp_path / "model.safetensors")
    write_safetensors(f, {
        "w4": np.zeros((o, i // 2), np.uint8), "w4.qs": np.zeros(o, np.float32),
        "wg": np.zeros((o, i // 2), np.uint8), "wg.qs": np.zeros(o * 2, np.float32),
        "w8": np.zeros((o, i), np.uint8), "w8.qs": np.zeros(o, np.float32),
        "wf": np.zeros((o, i), np.float32),
    })
    st = SafeTensors(str(tmp_path))
    assert QtInfo.detect(st, "w4", o, i).fmt == QtFmt.Int4
    g = QtInfo.detect(st, "wg", o, i)
    assert (g.fmt, g.gs, g.scale_count) == (QtFmt.Int4Grouped, 16, 4)
    assert QtInfo.detect(st, "w8", o, i).fmt == QtFmt.Int8
    assert QtInfo.detect(st, "wf", o, i).fmt == QtFmt.F32
    assert QtInfo.detect(st, "absent", o, i).fmt == QtFmt.F32


def test_int2_and_int2_g64_are_told_apart_by_scales(tmp_path):
    o, i = 4, 128
    ng = (i + 63) // 64
    f = str(tmp_path / "model.safetensors")
    write_safetensors(f, {
        "wr": np.zeros((o, i // 4), np.uint8), "wr.qs": np.zeros(o, np.float32),
        "wg": np.zeros((o, i // 4), np.uint8), "wg.qs": np.zeros(o * ng * 2, np.float32),
    })
    st = SafeTensors(f)
    assert QtInfo.detect(st, "wr", o, i).fmt == QtFmt.Int2
    g = QtInfo.detect(st, "wg", o, i)
    assert (g.fmt, g.gs, g.scale_count) == (QtFmt.Int2G64, 64, o * ng * 2)


def test_ragged_int2_g64_and_unknown(tmp_path):
    o, i = 3, 100
    ng = 2
    f = str(tmp_path / "model.safetensors")
    write_safetensors(f, {"w": np.zeros((o, ng * 16), np.uint8), "w.qs": np.zeros(o * ng * 2, np.float32),
                          "bad": np.zeros(7, np.uint8), "bad.qs": np.zeros(o, np.float32)})
    st = SafeTensors(f)
    d = QtInfo.detect(st, "w", o, i)
    assert (d.fmt, d.scale_count) == (QtFmt.Int2G64, o * ng * 2)
    assert QtInfo.detect(st, "bad", o, i).fmt == QtFmt.Unknown
    try:
        QtWeight.load(st, "bad", o, i)
        raise AssertionError("an unknown container must not load")
    except ContainerError as e:
        assert "match no quantized container" in str(e)


def test_load_and_dequant_round_trip(tmp_path):
    """quant_i4 / quant_i4_grouped (oracle, crates/peregrine-core/src/pack.rs:492-542) written to a
    checkpoint and read back: bytes and scales identical, dequantised values = nibble x scale."""
    import oracle as po

    rng = np.random.default_rng(3)
    o, i, gs = 6, 96, 32
    w = rng.standard_normal((o, i)).astype(np.float32)
    q, s = po.quant_i4(w, o, i)
    qg, sg = po.quant_i4_grouped(w, o, i, gs)
    f = str(tmp_path / "model.safetensors")
    write_safetensors(f, {"a": q.reshape(o, -1), "a.qs": s, "g": qg.reshape(o, -1), "g.qs": sg})
    st = SafeTensors(f)
    a = QtWeight.load(st, "a", o, i)
    g = QtWeight.load(st, "g", o, i)
    assert a.fmt == QtFmt.Int4 and g.fmt == QtFmt.Int4Grouped and g.gs == gs
    assert np.array_equal(a.raw()[0], q.reshape(-1)) and np.array_equal(a.raw()[1], s)
    assert np.array_equal(g.raw()[1], sg)
    da, dg = a.dequant(), g.dequant()
    assert np.max(np.abs(da - w)) <= np.max(s) * 0.5 + 1e-6
    assert np.max(np.abs(dg - w)) <= np.max(sg) * 0.5 + 1e-6
    # grouped scales are finer, so its worst error cannot exceed the per-row one by construction
    assert np.max(np.abs(dg - w)) <= np.max(np.abs(da - w)) + 1e-6
