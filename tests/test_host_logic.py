"""CPU suite, part 2: the boundary and the host-side logic, without a GPU: the C-ABI library
builds, loads and exports every declared symbol; argument errors come back as the reference's
StatusCode values before any device work; Filter2D geometry; missing library fails loudly."""
import ctypes
import os
import re

import pytest
import torch

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol(built_lib):
    header = open(os.path.join(ROOT, "include", "dlf_b200.h")).read()
    declared = set(re.findall(r"\b(dlf_b200_\w+)\s*\(", header))
    import dlf_b200
    assert declared == set(dlf_b200.EXPORTED_SYMBOLS)
    for name in declared:
        assert hasattr(built_lib, name), name


def test_status_strings(built_lib):
    import dlf_b200
    assert dlf_b200.status_string(0) == "kSuccess"
    assert dlf_b200.status_string(-1017) == "kInvalidDimension"
    assert dlf_b200.status_string(-2049) == "kInvalidBatchCount"


def _gemm_rc(L, dtype=32, layout=101, ta=111, tb=111, m=4, n=4, k=4, lda=4, ldb=4, ldc=4,
             a=0x1000, b=0x1000, c=0x1000):
    one = ctypes.c_float(1.0)
    return L.dlf_b200_gemm(dtype, layout, ta, tb, m, n, k, ctypes.byref(one), ctypes.c_void_p(a),
                           lda, ctypes.c_void_p(b), ldb, ctypes.byref(one), ctypes.c_void_p(c),
                           ldc, None)


def test_c_abi_argument_errors_without_a_device(built_lib):
    """Validation follows Xgemm::ProcessArguments and TestMatrixA/B/C and happens before any
    CUDA call, so the codes can be checked on a machine without a GPU."""
    L = built_lib
    assert _gemm_rc(L, m=0) == -1017                     # kInvalidDimension
    assert _gemm_rc(L, k=0) == -1017
    assert _gemm_rc(L, dtype=64) == -1024                # kNotImplemented (double)
    assert _gemm_rc(L, layout=7) == -30                  # kInvalidValue
    assert _gemm_rc(L, m=8, k=4, lda=3) == -1016         # row-major NoTrans A: ld >= k
    assert _gemm_rc(L, m=8, k=4, ta=112, lda=7) == -1016  # row-major Trans A: ld >= m
    assert _gemm_rc(L, n=8, ldb=7) == -1015              # row-major NoTrans B: ld >= n
    assert _gemm_rc(L, n=8, ldc=7, ldb=8) == -1014
    assert _gemm_rc(L, layout=102, m=8, lda=7) == -1016  # col-major NoTrans A: ld >= m
    assert _gemm_rc(L, a=0) == -1022                     # kInvalidMatrixA
    assert _gemm_rc(L, c=0) == -1020
    one = ctypes.c_float(1.0)
    p = ctypes.c_void_p(0x1000)
    rc = L.dlf_b200_gemm_strided_batched(32, 101, 111, 111, 4, 4, 4, ctypes.byref(one), p, 4, 16, p,
                                         4, 16, ctypes.byref(one), p, 4, 16, 0, None)
    assert rc == -2049                                   # kInvalidBatchCount
    offs = (ctypes.c_size_t * 2)(0, 16)
    al = (ctypes.c_float * 2)(1.0, 1.0)
    rc = L.dlf_b200_gemm_batched(32, 101, 111, 111, 4, 4, 4, al, p, offs, 4, p, offs, 4, al, p, offs,
                                 4, 2, None, 0, None)
    assert rc == -2050                                   # kInsufficientMemoryTemp
    assert L.dlf_b200_gemm_batched_workspace_bytes(10) == 10 * 44    # 3 offset, 2 scalar and 3 index tables
    rc = L.dlf_b200_conv2d(32, 1, 3, 5, 5, 5, 5, 4, 2, 3, 3, 1, 1, 1, 1, 1, 1, 1, 1, p, p, None, p,
                           None, 0, None)
    assert rc == -1017                                   # channels not divisible by group


def test_level3_argument_errors_without_a_device(built_lib):
    """symm / syrk / trmm / trsm check their arguments before any CUDA call, with the StatusCode
    values of the reference's routines."""
    L = built_lib
    one = ctypes.c_float(1.0)
    al = ctypes.byref(one)
    p = ctypes.c_void_p(0x1000)
    assert L.dlf_b200_symm(32, 101, 141, 121, 0, 4, al, p, 4, p, 4, al, p, 4, p, 1 << 20, None) == -1017
    assert L.dlf_b200_symm(32, 101, 141, 121, 4, 6, al, p, 3, p, 6, al, p, 6, p, 1 << 20, None) == -1016   # A is m x m
    assert L.dlf_b200_symm(32, 101, 142, 121, 4, 6, al, p, 5, p, 6, al, p, 6, p, 1 << 20, None) == -1016   # A is n x n
    assert L.dlf_b200_symm(32, 101, 141, 121, 4, 6, al, p, 4, p, 5, al, p, 6, p, 1 << 20, None) == -1015
    assert L.dlf_b200_symm(32, 102, 141, 121, 4, 6, al, p, 4, p, 4, al, p, 3, p, 1 << 20, None) == -1014   # col-major: ld >= m
    assert L.dlf_b200_symm(32, 101, 141, 121, 4, 6, al, p, 4, p, 6, al, p, 6, None, 0, None) == -2050
    assert L.dlf_b200_symm(32, 101, 140, 121, 4, 6, al, p, 4, p, 6, al, p, 6, p, 1 << 20, None) == -30
    assert L.dlf_b200_syrk(32, 101, 121, 111, 4, 0, al, p, 4, al, p, 4, p, 1 << 20, None) == -1017
    assert L.dlf_b200_syrk(32, 101, 121, 111, 4, 8, al, p, 7, al, p, 4, p, 1 << 20, None) == -1016         # row-major NoTrans: ld >= k
    assert L.dlf_b200_syrk(32, 101, 121, 112, 4, 8, al, p, 3, al, p, 4, p, 1 << 20, None) == -1016         # row-major Trans: ld >= n
    assert L.dlf_b200_syrk(32, 101, 121, 111, 4, 8, al, p, 8, al, p, 3, p, 1 << 20, None) == -1014
    for fn in (L.dlf_b200_trmm, L.dlf_b200_trsm):
        assert fn(32, 101, 141, 121, 111, 131, 4, 0, al, p, 4, p, 4, p, 1 << 20, None) == -1017
        assert fn(32, 101, 141, 121, 111, 131, 4, 6, al, p, 3, p, 6, p, 1 << 20, None) == -1016
        assert fn(32, 101, 142, 121, 111, 131, 4, 6, al, p, 6, p, 5, p, 1 << 20, None) == -1015
        assert fn(32, 101, 141, 121, 111, 130, 4, 6, al, p, 4, p, 6, p, 1 << 20, None) == -30
        assert fn(64, 101, 141, 121, 111, 131, 4, 6, al, p, 4, p, 6, p, 1 << 20, None) == -1024           # double: not implemented
    assert L.dlf_b200_trmm(32, 101, 141, 121, 111, 131, 4, 6, al, p, 4, p, 6, None, 0, None) == -2050
    assert L.dlf_b200_level3_workspace_bytes(4, 32, 100, 100) == 0
    assert L.dlf_b200_level3_workspace_bytes(1, 32, 100, 50) >= 100 * 100 * 4


def test_python_mirror_validates_buffer_sizes():
    from dlf_b200 import gblas
    a = torch.zeros(16)
    c = torch.zeros(15)
    with pytest.raises(gblas.BLASError) as e:
        gblas._validate(gblas.Layout.RowMajor, gblas.Transpose.NoTrans, gblas.Transpose.NoTrans,
                        4, 4, 4, a, [0], 4, a, [0], 4, c, [0], 4)
    assert e.value.status == gblas.StatusCode.kInsufficientMemoryC
    with pytest.raises(gblas.BLASError) as e:
        gblas._validate(gblas.Layout.RowMajor, gblas.Transpose.NoTrans, gblas.Transpose.NoTrans,
                        4, 4, 4, a, [1], 4, a, [0], 4, a, [0], 4)
    assert e.value.status == gblas.StatusCode.kInsufficientMemoryA


@pytest.mark.parametrize("h,pt,pb,k,s,d", [(5, 1, 1, 3, 1, 1), (7, 1, 1, 3, 2, 1), (7, 1, 0, 3, 2, 1),
                                           (10, 1, 2, 3, 1, 1), (224, 3, 3, 7, 2, 1), (2, 0, 0, 5, 1, 1),
                                           (9, 0, 0, 3, 1, 2)])
def test_filter2d_geometry_matches_oracle(h, pt, pb, k, s, d):
    from dlf_b200 import gdnn
    f = gdnn.Filter2D((1, 1, h, h), (1, 1, k, k)).pads(pt, pt, pb, pb).strides(s, s).dilations(d, d)
    assert f.output_h == oracle.output_dim(h, pt, pb, k, s, d)
    assert f.output_w == f.output_h


def test_missing_library_fails_loudly(monkeypatch):
    import dlf_b200
    monkeypatch.setattr(dlf_b200, "_lib", None)
    monkeypatch.setattr(dlf_b200, "LIB_PATH", "/nonexistent/libdlf_b200.so")
    with pytest.raises(dlf_b200.LibraryMissing):
        dlf_b200.lib()


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "dlf_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(dirpath, fn)).read()
                assert "import oracle" not in text and "dlf_oracle" not in text, fn
