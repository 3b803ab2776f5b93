"""Builds libcoli_cuda_backend.so (sm_100a only) in-tree with nvcc."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libcoli_cuda_backend.so")

SOURCES = ["backend.cu", "w4_host.cpp"]
DEPS = ["kernels.cuh", "kernels_mma.cuh", "kernels_tile.cuh", "kernels_umma.cuh", "kernels_decode.cuh", "kernels_block.cuh", "kernels_ep.cuh", "backend_ep.inc", "w4_layout.h", "w4_host.h", "backend_layer.inc", "backend_pipe.inc", "backend_noalloc.inc",
        os.path.join("..", "..", "include", "peregrine_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    # the CPU reference never contracts a*b+c; neither may the device code
    "-fmad=false", "-prec-div=true", "-prec-sqrt=true",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-O2",
    "-shared", "-cudart", "static",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA backend cannot be built")


def _stale(target: str, inputs) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(p) > t for p in inputs)


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, d) for d in DEPS]
    if force or _stale(LIB, deps):
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + srcs
        subprocess.check_call(cmd, cwd=CSRC)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
