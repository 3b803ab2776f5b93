"""coli_cuda_pipe_gemm_noalloc against coli_cuda_pipe_gemm, through the C ABI.

The allocation-free entry point serves callers that cannot call cudaMalloc: a
decode lane running with VRAM already committed to resident experts, or code
that may not trigger the device-wide synchronisation an allocation implies.  Its
scratch is one fixed array inside the library, shared by every call, so the test
makes two calls in a row with different inputs and row counts (the second must
not see anything the first left behind) and compares each, bit for bit, with
the allocating entry point.  This file sorts last on purpose: a run that stops
at the first failure has then already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

from peregrine_b200 import cuda
from peregrine_b200.synth import synth_matrix

pytestmark = pytest.mark.gpu


class DevArray:
    """A caller-owned device buffer (inputs and outputs stay the caller's to allocate)."""

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
def test_noalloc_gemm_matches_allocating_gemm_twice(dev, gs):
    lib = cuda.lib()
    rng = np.random.default_rng(77 + gs)
    i_n, o_n = 320, 200  # K padded inside the kernel, O not a multiple of 16
    m = synth_matrix(rng, o_n, i_n, gs)
    t = (cuda.Tensor.upload_grouped(dev, m.q, m.scale, i_n, o_n, gs) if gs
         else cuda.Tensor.upload(dev, m.q, m.scale, 2, i_n, o_n))
    # calls in a row on the one shared array, each with other data and another row count: 7 and 3
    # rows (tensor-core kernel, one pass), 1 and 2 (dp4a kernel, row-major scratch), 17 (two passes)
    for rows in (7, 3, 1, 17, 2):
        x = rng.standard_normal((rows, i_n)).astype(np.float32)
        xd = DevArray(dev, x)
        y_ref = DevArray(dev, nbytes=rows * o_n * 4)
        y_new = DevArray(dev, nbytes=rows * o_n * 4)
        assert lib.coli_cuda_pipe_gemm(t.handle, C.c_void_p(y_ref.ptr), C.c_void_p(xd.ptr), rows) == 1
        assert lib.coli_cuda_pipe_gemm_noalloc(t.handle, C.c_void_p(y_new.ptr), C.c_void_p(xd.ptr), rows) == 1
        want = y_ref.read((rows, o_n))
        got = y_new.read((rows, o_n))
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # the repo's int4 tolerance: bit-exact
        assert np.abs(want).max() > 0
        for b in (xd, y_ref, y_new):
            b.free()
    assert cuda.last_device_error(dev) == 0
    t.free()


def test_noalloc_gemm_limit_is_143_rows_at_width_6144(dev):
    """The largest request the 1 MiB array holds at I = 6144 is 143 rows: it is accepted and matches
    the allocating entry point bit for bit; 144 rows are refused (0, nothing launched)."""
    lib = cuda.lib()
    rng = np.random.default_rng(5)
    i_n, o_n = 6144, 48
    m = synth_matrix(rng, o_n, i_n, 32)
    t = cuda.Tensor.upload_grouped(dev, m.q, m.scale, i_n, o_n, 32)
    rows = 143
    x = rng.standard_normal((rows + 1, i_n)).astype(np.float32)
    xd = DevArray(dev, x)
    y_ref = DevArray(dev, nbytes=(rows + 1) * o_n * 4)
    y_new = DevArray(dev, nbytes=(rows + 1) * o_n * 4)
    assert lib.coli_cuda_pipe_gemm(t.handle, C.c_void_p(y_ref.ptr), C.c_void_p(xd.ptr), rows) == 1
    assert lib.coli_cuda_pipe_gemm_noalloc(t.handle, C.c_void_p(y_new.ptr), C.c_void_p(xd.ptr), rows) == 1
    want, got = y_ref.read((rows, o_n)), y_new.read((rows, o_n))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)) and np.abs(want).max() > 0
    assert lib.coli_cuda_pipe_gemm_noalloc(t.handle, C.c_void_p(y_new.ptr), C.c_void_p(xd.ptr), rows + 1) == 0
    assert cuda.last_device_error(dev) == 0
    f = cuda.Tensor.upload(dev, rng.standard_normal((8, 16)).astype(np.float32), None, 0, 16, 8)
    assert lib.coli_cuda_pipe_gemm_noalloc(f.handle, C.c_void_p(y_new.ptr), C.c_void_p(xd.ptr), 1) == 0  # not int4
    for b in (xd, y_ref, y_new):
        b.free()
    t.free()
    f.free()
