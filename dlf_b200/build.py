"""Builds the in-tree shared library ``dlf_b200/libdlf_b200.so`` with nvcc for sm_100a.

Run as ``python -m dlf_b200.build`` (add ``--force`` to rebuild, ``--verbose`` to see the
ptxas resource report). The library is the product: nothing in the package works without it.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libdlf_b200.so")
SOURCES = ["api.cu"]
HEADERS = ["channels_last.cuh", "conv_halo.cuh", "conv_small.cuh", "contraction.cuh", "contraction_ts.cuh", "epilogue.cuh", "level3.cuh", "pooling.cuh", "ptx.cuh", os.path.join("..", "..", "include", "dlf_b200.h")]


def _stale():
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def build(force=False, verbose=False):
    """Compile the CUDA sources into libdlf_b200.so; returns the library path."""
    if not force and not _stale():
        return LIB
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    cmd = [
        nvcc, "-std=c++17", "-O3", "-lineinfo",
        "-gencode", "arch=compute_100a,code=sm_100a",
        "-shared", "-Xcompiler", "-fPIC",
        "-o", LIB,
    ] + [os.path.join(CSRC, f) for f in SOURCES]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
    if verbose:
        sys.stderr.write(res.stdout + res.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
