"""Compile the native library in-tree for sm_100a with nvcc.

    python -m svox_b200.csrc.build [--force] [--verbose]

Produces ``svox_b200/csrc/libsvox_b200.so``.  Default nvcc floating-point
behaviour is kept on purpose (no --use_fast_math, IEEE division and square
root): the kernels must reproduce the reference's arithmetic.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "svox_b200.cu")
LIB = os.path.join(HERE, "libsvox_b200.so")
DEPS = ["svox_b200.cu", "common.cuh", "arith.cuh", "host.cuh", "query.cuh", "render.cuh", "render_queue.cuh", "render_replay.cuh", "noalloc.cuh", "collective.cuh",
        os.path.join("..", "..", "include", "svox_b200.h")]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    return any(os.path.getmtime(os.path.join(HERE, d)) > t for d in DEPS)


def build(force=False, verbose=False):
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
           "-std=c++17", "-shared", "-Xcompiler", "-fPIC", "-o", LIB, SRC]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
