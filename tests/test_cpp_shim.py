"""Builds and runs tests/cpp/test_shim.cpp: the C++ templates of include/dlf_b200_gpgpu.hpp
(reference signatures over the C ABI) on the reference's golden vectors."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "cpp", "test_shim.cpp")
EXE = os.path.join(ROOT, "tests", "cpp", "test_shim")


def build_shim_test():
    from dlf_b200 import build
    build.build()
    deps = [SRC, os.path.join(ROOT, "include", "dlf_b200_gpgpu.hpp"), os.path.join(ROOT, "include", "dlf_b200.h")]
    if os.path.exists(EXE) and all(os.path.getmtime(EXE) >= os.path.getmtime(d) for d in deps):
        return EXE
    libdir = os.path.join(ROOT, "dlf_b200")
    cmd = ["/usr/local/cuda/bin/nvcc", "-std=c++17", "-O1", "-x", "cu", "-o", EXE, SRC,
           "-I" + os.path.join(ROOT, "include"), "-L" + libdir, "-ldlf_b200",
           "-Xlinker", "-rpath=" + libdir]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    return EXE


def test_cpp_shim_compiles():
    """Host-only check: the header compiles and links against the library (no GPU needed)."""
    build_shim_test()


@pytest.mark.gpu
def test_cpp_shim_goldens_and_errors():
    exe = build_shim_test()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and res.stdout.strip().endswith("ok"), res.stdout + res.stderr
