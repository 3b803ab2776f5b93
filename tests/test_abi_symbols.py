"""The C-ABI library loads and exports every symbol the header declares."""
import ctypes as C
import os
import re

from peregrine_b200 import cuda
from peregrine_b200.build import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_builds_and_exports_header_symbols():
    path = build()
    lib = C.CDLL(path)
    header = open(os.path.join(ROOT, "include", "peregrine_b200.h")).read()
    declared = set(re.findall(r"\b(coli_cuda_\w+)\s*\(", header))
    assert len(declared) >= 47 + 10
    for name in sorted(declared):
        assert hasattr(lib, name), name
    assert declared == set(cuda.SYMBOLS)


def test_reference_surface_is_complete():
    # the 47 entry points of the reference header (cuda/backend_cuda.h:30-192)
    ref = """init shutdown device_count probe_device_count device_at mem_info stats group_stats tensor_upload
    matmul expert_mlp shared_mlp_w4a16 expert_group expert_group_tiled expert_group_reduce attention_absorb
    attention_absorb_batch attention_project_batch tensor_free tensor_bytes tensor_device tensor_update
    pipe_scratch pipe_alloc pipe_free pipe_upload pipe_download pipe_rmsnorm pipe_rope pipe_silu_mul pipe_add
    pipe_rows_add pipe_gemm pipe_rmsnorm_s pipe_rope_base pipe_copy2d attention_project_batch_dev
    attention_absorb_batch_dev attention_absorb_kvdev pipe_peer_copy attention_project_batch_dev_out pipe_sync
    graph_begin graph_end graph_launch graph_free graph_cache_stats""".split()
    assert len(ref) == 47
    for n in ref:
        assert "coli_cuda_" + n in cuda.SYMBOLS


def test_calls_fail_cleanly_without_init():
    # no context: every call reports failure instead of touching a device
    lib = cuda.lib()
    assert lib.coli_cuda_device_count() == 0
    assert lib.coli_cuda_device_at(0) == -1
    assert lib.coli_cuda_pipe_sync(0) == 0
    free, total = C.c_size_t(0), C.c_size_t(0)
    assert lib.coli_cuda_mem_info(0, C.byref(free), C.byref(total)) == 0
    h = C.c_void_p(None)
    w = (C.c_float * 4)()
    assert lib.coli_cuda_tensor_upload(C.byref(h), w, None, 0, 2, 2, 0) == 0
    assert lib.coli_cuda_tensor_bytes(None) == 0
    lib.coli_cuda_tensor_free(None)  # NULL-safe
    lib.coli_cuda_graph_free(None)


def test_reduce_layout_matches_reference_vector():
    # crates/peregrine-cuda/src/lib.rs:1652-1697
    lay = cuda.ReduceLayout.build([0, 1, 0, 1, 0], 2)
    assert list(lay.row_ptr) == [0, 3, 5] and list(lay.row_idx) == [0, 2, 4, 1, 3]
    assert cuda.ReduceLayout.build([0, 2], 2) is None
    empty = cuda.ReduceLayout.build([], 3)
    assert list(empty.row_ptr) == [0, 0, 0, 0] and empty.row_idx.size == 0
