"""numpy front for the CPU oracle (oracle/dlf_oracle.c).

TEST INFRASTRUCTURE ONLY: the checker for the CUDA path. Nothing in the product package
imports this module; only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` do.

``build()`` compiles ``oracle/_ref/libdlf_oracle.so`` with the Makefile beside this file. The
reference's own CPU code cannot be compiled here (Intel TBB and MKL are absent), so the library
is the restatement, pinned on the reference's golden vectors under ``tests/golden/``.
"""
import ctypes
import glob
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libdlf_oracle.so")

ROW_MAJOR, COL_MAJOR = 101, 102
NO_TRANS, TRANS, CONJ_TRANS = 111, 112, 113

_lib = None
_SGEMM_NN_FN = ctypes.CFUNCTYPE(None, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p,
                                ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                ctypes.c_int)


def build(force=False):
    src = os.path.join(_HERE, "dlf_oracle.c")
    if (force or not os.path.exists(LIB_PATH)
            or os.path.getmtime(LIB_PATH) < os.path.getmtime(src)):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        _lib = ctypes.CDLL(LIB_PATH)
        _lib.dlf_oracle_output_dim.restype = ctypes.c_size_t
        _lib.dlf_oracle_output_dim.argtypes = [ctypes.c_size_t] * 6
    return _lib


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


_SUFFIX = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64",
           np.dtype(np.int32): "i32", np.dtype(np.int64): "i64"}
_CT = {"f32": ctypes.c_float, "f64": ctypes.c_double, "i32": ctypes.c_int32, "i64": ctypes.c_int64}


def gemm_generic(trans_a, trans_b, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc):
    """detail::gemm for non-BLAS element types (exact evaluation order); C is updated in place.
    A, B, C are flat row-major numpy buffers of one of float32/float64/int32/int64."""
    sfx = _SUFFIX[C.dtype]
    ct = _CT[sfx]
    fn = getattr(lib(), "dlf_oracle_gemm_generic_" + sfx)
    fn.restype = None
    fn.argtypes = [ctypes.c_int] * 5 + [ct, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                        ctypes.c_int, ct, ctypes.c_void_p, ctypes.c_int]
    fn(trans_a, trans_b, m, n, k, alpha, _p(A), lda, _p(B), ldb, beta, _p(C), ldc)
    return C


def gblas_sgemm(layout, trans_a, trans_b, m, n, k, alpha, A, a_offset, a_ld, B, b_offset, b_ld,
                beta, C, c_offset, c_ld, wide=False):
    """gpgpu::blas::gemm<float> semantics on flat float32 buffers; C updated in place."""
    fn = lib().dlf_oracle_gblas_sgemm
    fn.restype = None
    fn.argtypes = [ctypes.c_int] * 3 + [ctypes.c_size_t] * 3 + [
        ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p,
        ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t,
        ctypes.c_size_t, ctypes.c_int]
    fn(layout, trans_a, trans_b, m, n, k, alpha, _p(A), a_offset, a_ld, _p(B), b_offset, b_ld,
       beta, _p(C), c_offset, c_ld, 1 if wide else 0)
    return C


def gblas_sgemm_strided_batched(layout, trans_a, trans_b, m, n, k, alpha, A, a_offset, a_ld,
                                a_stride, B, b_offset, b_ld, b_stride, beta, C, c_offset, c_ld,
                                c_stride, batch, wide=False):
    fn = lib().dlf_oracle_gblas_sgemm_strided_batched
    fn.restype = None
    fn.argtypes = [ctypes.c_int] * 3 + [ctypes.c_size_t] * 3 + [
        ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t,
        ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float,
        ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t,
        ctypes.c_int]
    fn(layout, trans_a, trans_b, m, n, k, alpha, _p(A), a_offset, a_ld, a_stride, _p(B), b_offset,
       b_ld, b_stride, beta, _p(C), c_offset, c_ld, c_stride, batch, 1 if wide else 0)
    return C


def gblas_sgemm_batched(layout, trans_a, trans_b, m, n, k, alphas, A, a_offsets, a_ld, B,
                        b_offsets, b_ld, betas, C, c_offsets, c_ld, batch, wide=False):
    fn = lib().dlf_oracle_gblas_sgemm_batched
    fn.restype = None
    fn.argtypes = [ctypes.c_int] * 3 + [ctypes.c_size_t] * 3 + [
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
        ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
        ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int]
    al = np.ascontiguousarray(alphas, dtype=np.float32)
    be = np.ascontiguousarray(betas, dtype=np.float32)
    ao = np.ascontiguousarray(a_offsets, dtype=np.uint64)
    bo = np.ascontiguousarray(b_offsets, dtype=np.uint64)
    co = np.ascontiguousarray(c_offsets, dtype=np.uint64)
    fn(layout, trans_a, trans_b, m, n, k, _p(al), _p(A), _p(ao), a_ld, _p(B), _p(bo), b_ld,
       _p(be), _p(C), _p(co), c_ld, batch, 1 if wide else 0)
    return C


def output_dim(size, pad_lo, pad_hi, kernel, stride, dilation):
    return int(lib().dlf_oracle_output_dim(size, pad_lo, pad_hi, kernel, stride, dilation))


def conv2d(X, W, group=1, pads=(0, 0, 0, 0), strides=(1, 1), dilations=(1, 1), bias=None,
           wide=False, sgemm_nn=None):
    """dlf::dnn::conv2d on the CPU (per image, per group: im2col then sgemm) followed, when bias
    is given, by the separate bias pass of ConvOp. X: NCHW float32, W: OIHW float32.
    pads = (top, left, bottom, right). Returns Y (NCHW float32)."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    W = np.ascontiguousarray(W, dtype=np.float32)
    n, c, h, w = X.shape
    co, cg, kh, kw = W.shape
    assert cg * group == c and co % group == 0
    pt, pl, pb, pr = pads
    oh = output_dim(h, pt, pb, kh, strides[0], dilations[0])
    ow = output_dim(w, pl, pr, kw, strides[1], dilations[1])
    Y = np.empty((n, co, oh, ow), dtype=np.float32)
    fn = lib().dlf_oracle_conv2d_f32
    fn.restype = None
    fn.argtypes = [ctypes.c_void_p] * 3 + [ctypes.c_size_t] * 16 + [ctypes.c_int, ctypes.c_void_p]
    cb = ctypes.cast(sgemm_nn, ctypes.c_void_p) if sgemm_nn is not None else None
    fn(_p(X), _p(W), _p(Y), n, c, h, w, co, group, kh, kw, pt, pl, pb, pr, strides[0], strides[1],
       dilations[0], dilations[1], 1 if wide else 0, cb)
    if bias is not None:
        b = np.ascontiguousarray(bias, dtype=np.float32)
        fb = lib().dlf_oracle_bias_f32
        fb.restype = None
        fb.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_size_t] * 3
        fb(_p(Y), _p(b), n, co, oh * ow)
    return Y


def pool2d(X, kernel, mode="max", pads=(0, 0, 0, 0), strides=(1, 1), dilations=(1, 1),
           count_include_pad=False):
    """dlf::dnn::max_pooling / average_pooling on the CPU (dnn.h:207-247 over
    dnn_detail.h:172-227). X: NCHW float32; kernel = (kh, kw); pads = (top, left, bottom, right)."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    n, c, h, w = X.shape
    kh, kw = kernel
    pt, pl, pb, pr = pads
    oh = output_dim(h, pt, pb, kh, strides[0], dilations[0])
    ow = output_dim(w, pl, pr, kw, strides[1], dilations[1])
    Y = np.empty((n, c, oh, ow), dtype=np.float32)
    fn = lib().dlf_oracle_pool2d_f32
    fn.restype = None
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int] + [ctypes.c_size_t] * 14
    fn(_p(X), _p(Y), 0 if mode == "max" else 1, 1 if count_include_pad else 0, n, c, h, w, oh, ow, kh, kw,
       pt, pl, strides[0], strides[1], dilations[0], dilations[1])
    return Y


def global_pool(X, mode="avg", wide=False):
    """dlf::dnn::global_max_pooling / global_average_pooling (dnn.h:337-375 over
    dnn_detail.h:229-260): {N, C, ...} -> {N, C, 1, 1}."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    planes = X.shape[0] * X.shape[1]
    Y = np.empty((X.shape[0], X.shape[1]) + (1,) * (X.ndim - 2), dtype=np.float32)
    fn = lib().dlf_oracle_global_pool_f32
    fn.restype = None
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int]
    fn(_p(X), _p(Y), 0 if mode == "max" else 1, planes, X.size // planes, 1 if wide else 0)
    return Y


def conv2d_fused(X, W, residual=None, relu=False, **kw):
    """The operator chain dlf's graph runtime evaluates around a convolution, as separate passes:
    ConvOp (conv + bias, dlf/include/predict.h:1258-1286), then Add of a residual tensor
    (BinaryOp<xfn::plus>, predict.h:928-960), then Relu (ReluOp, predict.h:776-784;
    xfn::relu = max(0, x), dlf/include/tensor/xfn.h:588-591). Every pass rounds to float32."""
    Y = conv2d(X, W, **kw)
    if residual is not None:
        Y = (Y + np.asarray(residual, dtype=np.float32)).astype(np.float32)
    if relu:
        Y = np.maximum(np.float32(0), Y)
    return Y


# ---------------------------------------------------------------------------------------------
# Tuned host BLAS for the timed CPU baseline: the reference calls cblas_sgemm of whatever BLAS it
# was linked with (MKL in its Dockerfile). On this box the closest stand-in is the OpenBLAS that
# ships inside the scipy / numpy wheels.
# ---------------------------------------------------------------------------------------------
def find_host_cblas():
    """Returns (ctypes function for row-major cblas_sgemm, description) or (None, reason)."""
    import importlib.util
    cands = []
    for pkg, sym in (("scipy", "scipy_cblas_sgemm"), ("numpy", "scipy_cblas_sgemm64_")):
        spec = importlib.util.find_spec(pkg)
        if spec is None or not spec.submodule_search_locations:
            continue
        root = os.path.dirname(list(spec.submodule_search_locations)[0])
        for so in sorted(glob.glob(os.path.join(root, pkg + ".libs", "libscipy_openblas*.so"))):
            cands.append((so, sym))
    for so, sym in cands:
        try:
            L = ctypes.CDLL(so)
            fn = getattr(L, sym)
        except (OSError, AttributeError):
            continue
        ilp64 = sym.endswith("64_")
        it = ctypes.c_int64 if ilp64 else ctypes.c_int
        fn.restype = None
        fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, it, it, it, ctypes.c_float,
                       ctypes.c_void_p, it, ctypes.c_void_p, it, ctypes.c_float, ctypes.c_void_p, it]
        return fn, "OpenBLAS %s (%s)" % (os.path.basename(so), "ILP64" if ilp64 else "LP64")
    return None, "no host cblas found"


def host_sgemm(fn, layout, trans_a, trans_b, m, n, k, alpha, A, lda, B, ldb, beta, C, ldc):
    fn(layout, trans_a, trans_b, m, n, k, alpha, _p(A), lda, _p(B), ldb, beta, _p(C), ldc)


def host_sgemm_nn_callback(fn):
    """Wraps a cblas_sgemm as the row-major NoTrans/NoTrans callback dlf_oracle_conv2d_f32 takes."""
    def cb(m, n, k, a, lda, b, ldb, c, ldc):
        fn(ROW_MAJOR, NO_TRANS, NO_TRANS, m, n, k, 1.0, a, lda, b, ldb, 0.0, c, ldc)
    return _SGEMM_NN_FN(cb)


# ---------------------------------------------------------------------------------------------
# level-3 routines built on GEMM (row-major float32; flat or 2-D C-contiguous numpy buffers)
# ---------------------------------------------------------------------------------------------
UPPER, LOWER = 121, 122
NON_UNIT, UNIT = 131, 132
LEFT, RIGHT = 141, 142


def symm(side, uplo, m, n, alpha, A, lda, B, ldb, beta, C, ldc, wide=False):
    """gblas::symm / cblas_ssymm, row-major: C = alpha*S*B + beta*C (Left) or alpha*B*S + beta*C
    (Right), S symmetric with only its `uplo` triangle stored in A. C is updated in place."""
    fn = lib().dlf_oracle_symm_f32
    fn.restype = None
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float, ctypes.c_void_p,
                   ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_void_p,
                   ctypes.c_size_t, ctypes.c_int]
    fn(side, uplo, m, n, alpha, _p(A), lda, _p(B), ldb, beta, _p(C), ldc, 1 if wide else 0)
    return C


def syrk(uplo, trans, n, k, alpha, A, lda, beta, C, ldc, wide=False):
    """gblas::syrk / cblas_ssyrk, row-major: the `uplo` triangle of C = alpha*op(A)*op(A)^T + beta*C."""
    fn = lib().dlf_oracle_syrk_f32
    fn.restype = None
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float, ctypes.c_void_p,
                   ctypes.c_size_t, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    fn(uplo, trans, n, k, alpha, _p(A), lda, beta, _p(C), ldc, 1 if wide else 0)
    return C


def _tri(name, side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, wide):
    fn = getattr(lib(), name)
    fn.restype = None
    fn.argtypes = [ctypes.c_int] * 4 + [ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float, ctypes.c_void_p,
                                        ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    fn(side, uplo, trans, diag, m, n, alpha, _p(A), lda, _p(B), ldb, 1 if wide else 0)
    return B


def trmm(side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, wide=False):
    """gblas::trmm / cblas_strmm, row-major: B = alpha*op(T)*B (Left) or alpha*B*op(T) (Right), in place."""
    return _tri("dlf_oracle_trmm_f32", side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, wide)


def trsm(side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, wide=False):
    """gblas::trsm / cblas_strsm, row-major: solves op(T)*X = alpha*B (Left) or X*op(T) = alpha*B
    (Right); X overwrites B."""
    return _tri("dlf_oracle_trsm_f32", side, uplo, trans, diag, m, n, alpha, A, lda, B, ldb, wide)
