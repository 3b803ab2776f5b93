"""Helpers shared by the GPU parity tests (the `dev` fixture lives in conftest.py)."""
import numpy as np


def bits(a):
    return np.ascontiguousarray(a, np.float32).view(np.uint32)
