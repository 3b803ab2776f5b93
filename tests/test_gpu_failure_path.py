"""The failure path shared by every kernel: a bounded wait that runs out must give up, report
through the device error word and leave the context usable.  The wait is made to run out on
purpose by waiting (with a short limit) on a barrier nothing completes; no fault is raised."""
import numpy as np
import pytest

from peregrine_b200 import cuda
from peregrine_b200.resident import upload_layer
from peregrine_b200.synth import synth_layer, synth_tokens
from tests.gpu_common import bits
from tests.refmodel import oracle_layer_forward

pytestmark = pytest.mark.gpu


def test_expired_wait_reports_and_context_survives(dev):
    assert cuda.last_device_error(dev) == 0
    assert cuda.selftest_bounded_wait(dev, 200_000)
    assert cuda.last_device_error(dev) == 1      # the expired wait, reported once
    assert cuda.last_device_error(dev) == 0      # reading clears it
    # the same context still computes, bit for bit
    layer = synth_layer(21, hidden=256, inter=96, n_experts=8, k=2, gs=32)
    x = synth_tokens(4, 1, 256)
    ml = upload_layer(dev, layer)
    assert np.array_equal(bits(ml.forward(x)), bits(oracle_layer_forward(layer, x)))
    assert cuda.last_device_error(dev) == 0
    ml.free()


def test_host_forward_refuses_a_result_when_the_error_word_is_set(dev):
    layer = synth_layer(22, hidden=256, inter=96, n_experts=8, k=2, gs=32)
    x = synth_tokens(5, 1, 256)
    ml = upload_layer(dev, layer)
    assert cuda.selftest_bounded_wait(dev, 100_000)
    with pytest.raises(cuda.CudaError):
        ml.forward(x)                             # sees the pending error, returns failure, clears it
    assert np.array_equal(bits(ml.forward(x)), bits(oracle_layer_forward(layer, x)))
    ml.free()
