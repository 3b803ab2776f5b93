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


def test_speculative_rows_emit_exactly_what_greedy_would(dev):
    """Three sequences speculating three tokens deep are twelve rows of one forward; with right and
    deliberately wrong drafts mixed the emitted streams equal token-by-token greedy decoding
    (the rule of crates/peregrine-model/src/model.rs:383-406, 4028-4116)."""
    from peregrine_b200.speculative import stack_forward_rows, verify_drafts

    st = synth_stack(5, hidden=256, inter=64, dense_inter=128, n_experts=8, k=2, n_layers=3, first_dense=1, vocab=64)
    ds = DeviceStack(dev, st, batch=12, max_steps=40)
    start = [3, 17, 40]
    steps = 24
    greedy = ds.decode(np.asarray(start + [0] * 9, np.int32), steps)[:, :3].T  # [3, steps]: tokens after `start`
    forward_rows = stack_forward_rows(ds)
    rng = np.random.default_rng(0)
    emitted = [[] for _ in start]
    nxt = [None] * 3
    # round 0: plain greedy for the first token (nothing confirmed yet to speculate from)
    first = forward_rows(np.asarray(start, np.int32))
    for s in range(3):
        nxt[s] = int(first[s])
    rounds = 0
    while min(len(e) for e in emitted) < steps - 4:
        drafts = []
        for s in range(3):
            pos = len(emitted[s]) + 1            # index in `greedy` of the token after nxt[s]
            true = [int(t) for t in greedy[s, pos:pos + 3]]
            if rng.random() < 0.5 and true:      # corrupt one draft: everything from it on must be rejected
                j = int(rng.integers(len(true)))
                true[j] = (true[j] + 1) % 64
            drafts.append(true)
        out = verify_drafts(forward_rows, nxt, drafts, [len(e) for e in emitted])
        for s, v in enumerate(out):
            emitted[s].extend(v.tokens)
            nxt[s] = v.next
        rounds += 1
    for s in range(3):
        n = min(len(emitted[s]), steps)  # (the last round may run past the reference's length)
        assert n >= steps - 4 and emitted[s][:n] == [int(t) for t in greedy[s, :n]], f"sequence {s}"
    assert rounds < steps  # speculation did accept drafts: fewer forwards than tokens
    assert cuda.last_device_error(dev) == 0
    ds.free()
