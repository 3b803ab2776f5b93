"""peregrine_b200 — B200 (sm_100a) backend for peregrine's MoE expert-FFN path.

The product is ``libcoli_cuda_backend.so`` (CUDA kernels + the C ABI of
``include/peregrine_b200.h``).  ``peregrine_b200.cuda`` is the host-side mirror
of the reference's FFI crate (``crates/peregrine-cuda/src/lib.rs``): same entry
points, same argument meaning, same error behaviour, over ctypes.
"""
from . import cuda  # noqa: F401
from .build import build  # noqa: F401

__all__ = ["cuda", "build"]
