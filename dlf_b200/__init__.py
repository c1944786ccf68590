"""dlf_b200 - B200 (sm_100a) backend for dlf's dense-contraction path.

The product is the C-ABI shared library ``libdlf_b200.so`` (sources in ``csrc/``, interface in
``include/dlf_b200.h``). This package loads it with ctypes and mirrors, name for name, the
reference's ``gpgpu::blas`` / ``gpgpu::dnn`` operator interface for this path
(``gblas.gemm``, ``gblas.gemmBatched``, ``gblas.gemmStridedBatched``, ``gdnn.conv2d``) over
device buffers held as torch CUDA tensors. There is no CPU path: importing the operators
without the built library raises.
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdlf_b200.so")

_lib = None


class LibraryMissing(RuntimeError):
    pass


def lib():
    """Returns the loaded C-ABI library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                "libdlf_b200.so is not built: run `python -m dlf_b200.build` "
                "(there is no fallback path)")
        L = ctypes.CDLL(LIB_PATH)
        _declare(L)
        _lib = L
    return _lib


def _declare(L):
    c_int, c_size, c_void = ctypes.c_int, ctypes.c_size_t, ctypes.c_void_p
    psize = ctypes.POINTER(ctypes.c_size_t)
    L.dlf_b200_gemm.restype = c_int
    L.dlf_b200_gemm.argtypes = [c_int] * 4 + [c_size] * 3 + [
        c_void, c_void, c_size, c_void, c_size, c_void, c_void, c_size, c_void]
    L.dlf_b200_gemm_ex.restype = c_int
    L.dlf_b200_gemm_ex.argtypes = L.dlf_b200_gemm.argtypes[:-1] + [c_void, c_size, c_void]
    L.dlf_b200_gemm_workspace_bytes.restype = c_size
    L.dlf_b200_gemm_workspace_bytes.argtypes = [c_int, c_size, c_size, c_size]
    L.dlf_b200_gemm_strided_batched.restype = c_int
    L.dlf_b200_gemm_strided_batched.argtypes = [c_int] * 4 + [c_size] * 3 + [
        c_void, c_void, c_size, c_size, c_void, c_size, c_size, c_void, c_void, c_size, c_size,
        c_size, c_void]
    L.dlf_b200_gemm_batched.restype = c_int
    L.dlf_b200_gemm_batched.argtypes = [c_int] * 4 + [c_size] * 3 + [
        c_void, c_void, psize, c_size, c_void, psize, c_size, c_void, c_void, psize, c_size,
        c_size, c_void, c_size, c_void]
    L.dlf_b200_gemm_batched_noalloc.restype = c_int
    L.dlf_b200_gemm_batched_noalloc.argtypes = [c_int] * 4 + [c_size] * 3 + [
        c_void, c_void, psize, c_size, c_void, psize, c_size, c_void, c_void, psize, c_size,
        c_size, c_void]
    L.dlf_b200_gemm_batched_workspace_bytes.restype = c_size
    L.dlf_b200_gemm_batched_workspace_bytes.argtypes = [c_size]
    L.dlf_b200_conv2d.restype = c_int
    L.dlf_b200_conv2d.argtypes = [c_int] + [c_size] * 18 + [
        c_void, c_void, c_void, c_void, c_void, c_size, c_void]
    L.dlf_b200_conv2d_fused.restype = c_int
    L.dlf_b200_conv2d_fused.argtypes = [c_int] + [c_size] * 18 + [
        c_void, c_void, c_void, c_void, c_int, c_void, c_void, c_size, c_void]
    L.dlf_b200_maxpool.restype = c_int
    L.dlf_b200_maxpool.argtypes = [c_int] + [c_size] * 16 + [c_void, c_void, c_void]
    L.dlf_b200_avgpool.restype = c_int
    L.dlf_b200_avgpool.argtypes = [c_int] + [c_size] * 16 + [c_int, c_void, c_void, c_void]
    L.dlf_b200_nhwc_filter_elems.restype = c_size
    L.dlf_b200_nhwc_filter_elems.argtypes = [c_size] * 4
    L.dlf_b200_pack_filters_nhwc.restype = c_int
    L.dlf_b200_pack_filters_nhwc.argtypes = [c_int] + [c_size] * 4 + [c_void, c_void, c_void]
    L.dlf_b200_nchw_to_nhwc.restype = c_int
    L.dlf_b200_nchw_to_nhwc.argtypes = [c_int] + [c_size] * 4 + [c_void, c_void, c_void]
    L.dlf_b200_conv2d_nhwc.restype = c_int
    L.dlf_b200_conv2d_nhwc.argtypes = [c_int] + [c_size] * 17 + [c_void, c_void, c_void, c_void, c_int, c_void, c_int,
                                                               c_void]
    L.dlf_b200_pool_nhwc.restype = c_int
    L.dlf_b200_pool_nhwc.argtypes = [c_int, c_int, c_int] + [c_size] * 12 + [c_void, c_void, c_void]
    L.dlf_b200_conv2d_workspace_bytes.restype = c_size
    L.dlf_b200_conv2d_workspace_bytes.argtypes = [c_int] + [c_size] * 10
    L.dlf_b200_level3_workspace_bytes.restype = c_size
    L.dlf_b200_level3_workspace_bytes.argtypes = [c_int, c_int, c_size, c_size]
    L.dlf_b200_symm.restype = c_int
    L.dlf_b200_symm.argtypes = [c_int] * 4 + [c_size, c_size, c_void, c_void, c_size, c_void, c_size, c_void, c_void,
                                              c_size, c_void, c_size, c_void]
    L.dlf_b200_syrk.restype = c_int
    L.dlf_b200_syrk.argtypes = [c_int] * 4 + [c_size, c_size, c_void, c_void, c_size, c_void, c_void, c_size, c_void,
                                              c_size, c_void]
    for fn in (L.dlf_b200_trmm, L.dlf_b200_trsm):
        fn.restype = c_int
        fn.argtypes = [c_int] * 6 + [c_size, c_size, c_void, c_void, c_size, c_void, c_size, c_void, c_size, c_void]
    L.dlf_b200_status_string.restype = ctypes.c_char_p
    L.dlf_b200_status_string.argtypes = [c_int]
    L.dlf_b200_device_status.restype = c_int
    L.dlf_b200_device_status.argtypes = [ctypes.POINTER(c_int)]
    L.dlf_b200_set_tuning.restype = None
    L.dlf_b200_set_tuning.argtypes = [c_int, c_int]
    L.dlf_b200_launch_count.restype = ctypes.c_ulonglong
    L.dlf_b200_launch_count.argtypes = []


EXPORTED_SYMBOLS = (
    "dlf_b200_gemm",
    "dlf_b200_gemm_ex",
    "dlf_b200_gemm_workspace_bytes",
    "dlf_b200_gemm_strided_batched",
    "dlf_b200_gemm_batched",
    "dlf_b200_gemm_batched_workspace_bytes",
    "dlf_b200_gemm_batched_noalloc",
    "dlf_b200_conv2d",
    "dlf_b200_conv2d_fused",
    "dlf_b200_conv2d_workspace_bytes",
    "dlf_b200_nhwc_filter_elems",
    "dlf_b200_pack_filters_nhwc",
    "dlf_b200_nchw_to_nhwc",
    "dlf_b200_conv2d_nhwc",
    "dlf_b200_pool_nhwc",
    "dlf_b200_level3_workspace_bytes",
    "dlf_b200_symm",
    "dlf_b200_syrk",
    "dlf_b200_trmm",
    "dlf_b200_trsm",
    "dlf_b200_maxpool",
    "dlf_b200_avgpool",
    "dlf_b200_status_string",
    "dlf_b200_device_status",
    "dlf_b200_set_tuning",
    "dlf_b200_launch_count",
)


def status_string(code):
    return lib().dlf_b200_status_string(int(code)).decode()


def device_status():
    """Synchronises the current device and returns (and clears) its kernel status word."""
    v = ctypes.c_int(0)
    rc = lib().dlf_b200_device_status(ctypes.byref(v))
    if rc != 0:
        raise RuntimeError("dlf_b200_device_status failed: " + status_string(rc))
    return v.value


def launch_count():
    return int(lib().dlf_b200_launch_count())


def set_tuning(force_bn=0, force_generic_loader=False):
    lib().dlf_b200_set_tuning(int(force_bn), int(force_generic_loader))
