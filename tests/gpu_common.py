"""Shared set-up for the GPU parity tests: one backend context on device 0."""
import pytest

from peregrine_b200 import cuda


@pytest.fixture(scope="session")
def dev():
    n = cuda.init([0])
    if n < 1:
        pytest.fail("a CUDA device is visible to torch but the backend could not initialise it")
    yield 0
    cuda.shutdown()


def bits(a):
    import numpy as np

    return np.ascontiguousarray(a, np.float32).view(np.uint32)
