"""Two devices in one process: kernel attributes (the dynamic shared-memory opt-in) are per device,
so a layer and a single-matrix call on the second device must configure their kernels there too.
Skipped when fewer than two devices are visible.  Plain kernels only, no peer operands."""
import ctypes as C

import numpy as np
import pytest

import oracle as po
from peregrine_b200 import cuda
from peregrine_b200.resident import upload_layer
from peregrine_b200.synth import synth_layer, synth_matrix, synth_tokens
from tests.gpu_common import bits
from tests.refmodel import oracle_layer_forward

pytestmark = pytest.mark.gpu


def test_layer_and_gemm_on_a_second_device(dev):
    if cuda.probe_device_count() < 2:
        pytest.skip("needs two visible devices")
    # the session fixture holds device 0; re-initialise with both for this test and restore after
    assert cuda.init([0, 1]) == 2
    try:
        layer = synth_layer(31, hidden=256, inter=96, n_experts=12, k=3, gs=32)
        x = synth_tokens(31, 1, 256)
        want = oracle_layer_forward(layer, x, threads=2)
        for d in (0, 1):
            ml = upload_layer(d, layer)
            assert np.array_equal(bits(ml.forward(x)), bits(want))
            assert cuda.last_device_error(d) == 0
            ml.free()
        rng = np.random.default_rng(2)
        m = synth_matrix(rng, 64, 256, 32)
        xr = rng.standard_normal((2, 256)).astype(np.float32)
        t = cuda.Tensor.upload_grouped(1, m.q, m.scale, 256, 64, 32)
        lib = cuda.lib()
        xp = lib.coli_cuda_pipe_alloc(1, xr.nbytes)
        yp = lib.coli_cuda_pipe_alloc(1, 2 * 64 * 4)
        assert lib.coli_cuda_pipe_upload(1, xp, xr.ctypes.data, xr.nbytes) == 1
        assert lib.coli_cuda_pipe_gemm(t.handle, C.c_void_p(yp), C.c_void_p(xp), 2) == 1
        got = np.empty((2, 64), np.float32)
        assert lib.coli_cuda_pipe_download(1, yp, got.ctypes.data, got.nbytes) == 1
        assert np.array_equal(bits(got), bits(po.Weight(m.q, m.scale, 4, 32, 256, 64).apply(xr, 2)))
        lib.coli_cuda_pipe_free(1, xp)
        lib.coli_cuda_pipe_free(1, yp)
        t.free()
    finally:
        assert cuda.init([0]) == 1
