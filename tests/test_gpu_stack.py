"""Greedy token ids of the synthetic FFN-only decode stack over 256 steps: the device loop must
pick exactly the ids the CPU oracle picks (the full-stack parity rule), on a scaled-down
stack (1 dense + 3 MoE layers) that the oracle finishes in seconds."""
import numpy as np
import pytest

from peregrine_b200.stack import DeviceStack, synth_stack
from peregrine_b200 import cuda
from tests.refmodel import oracle_stack_decode

pytestmark = pytest.mark.gpu


def test_greedy_ids_identical_over_256_steps(dev):
    st = synth_stack(seed=3, hidden=256, inter=96, dense_inter=384, n_experts=16, k=4, n_layers=4, first_dense=1,
                     vocab=4096)
    batch, steps = 4, 256
    ids0 = np.array([1, 17, 300, 4011], np.int32)
    ds = DeviceStack(dev, st, batch, steps)
    got = ds.decode(ids0, steps)
    want = oracle_stack_decode(st, ids0, steps)
    assert got.shape == (steps, batch)
    assert np.array_equal(got, want)
    assert len(np.unique(got)) > 8  # the sequence is not stuck on one token
    again = ds.decode(ids0, 32)
    assert np.array_equal(again, want[:32])
    assert cuda.last_device_error(dev) == 0
    ds.free()


def test_greedy_ids_at_the_benchmark_layer_shape(dev):
    """The stack at the real layer shapes of the full-stack benchmark config: hidden 6144, one dense layer
    of width 12288, two MoE layers with 256 experts (top-8 + shared, width 2048), batch 4, 16 greedy
    steps; ids identical to the oracle's.  The experts reuse four host blobs (the oracle's memory and
    the upload time stay small); every expert id is attached and routable."""
    st = synth_stack(seed=5, hidden=6144, inter=2048, dense_inter=12288, n_experts=256, k=8, n_layers=3,
                     first_dense=1, vocab=4096, distinct_experts=4, scale_std=0.02 / 64)
    batch, steps = 4, 16
    ids0 = np.array([3, 1000, 2222, 4000], np.int32)
    ds = DeviceStack(dev, st, batch, steps, repeats="share")
    got = ds.decode(ids0, steps)
    want = oracle_stack_decode(st, ids0, steps, threads=8)
    assert np.array_equal(got, want)
    assert len(np.unique(got)) > 4
    assert cuda.last_device_error(dev) == 0
    ds.free()


def test_argmax_rules_on_device(dev):
    import ctypes as C

    from peregrine_b200.stack import _DevBuf

    rows = np.array([[1.0, 3.0, 3.0, 2.0], [np.nan, 1.0, np.nan, 2.0], [np.nan] * 4, [-np.inf, -np.inf, -1.0, -1.0]],
                    np.float32)
    lo = _DevBuf(dev, rows)
    ids = _DevBuf(dev, nbytes=16)
    assert cuda.lib().coli_cuda_pipe_argmax(dev, C.c_void_p(ids.ptr), C.c_void_p(lo.ptr), 4, 4) == 1
    assert ids.download((4,), np.int32).tolist() == [1, 3, 0, 2]
    lo.free()
    ids.free()
