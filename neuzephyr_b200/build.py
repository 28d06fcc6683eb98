"""Builds libnzb.so (the sm_100a kernel library) in-tree with nvcc.

    python -m neuzephyr_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The shared object is written next to this file so it
travels with a snapshot of the repository.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libnzb.so")
SOURCES = ["nzb_api.cu", "nzb_cast.cu", "nzb_gemm.cu", "nzb_static.cu", "nzb_ops.cu", "nzb_conv.cu", "nzb_linear.cu"]
HEADERS = ["nzb_internal.h", "nzb_ptx.cuh", os.path.join("..", "..", "include", "nzb.h")]
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC,-fvisibility=hidden", "-shared"]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(CSRC, f)) > t for f in SOURCES + HEADERS)


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB
    cmd = [NVCC] + FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + SOURCES
    subprocess.check_call(cmd, cwd=CSRC)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
