"""Host-side mirror of the reference's ``gpgpu::blas`` GEMM family (gpgpu/include/gblas.h).

Same names, argument order and meaning as ``gpgpu::blas::gemm`` (gblas.h:496-504),
``gemmBatched`` (:661-671) and ``gemmStridedBatched`` (:673-683). A ``Buffer<T>`` is a torch
CUDA tensor of dtype float16 / bfloat16 / float32 viewed flat; offsets, leading dimensions and
strides are in elements; ``queue`` is a ``torch.cuda.Stream`` (default: the current stream);
``event`` is an optional :class:`Event` that brackets the launch like the reference's
``Event*`` (gpgpu/src/gpgpu_cu.cpp:389-398). Errors raise :class:`BLASError` carrying the
reference's ``StatusCode`` value. Every call goes through the C-ABI of libdlf_b200.so.
"""
import ctypes
import enum
import threading

import torch

from . import lib, status_string


class Layout(enum.IntEnum):
    RowMajor = 101
    ColMajor = 102


class Transpose(enum.IntEnum):
    NoTrans = 111
    Trans = 112
    ConjTrans = 113


class Precision(enum.IntEnum):
    Half = 16
    Single = 32
    BFloat16 = 1600  # addition: the reference has no bf16 storage type


class StatusCode(enum.IntEnum):
    kSuccess = 0
    kInvalidValue = -30
    kNotImplemented = -1024
    kInvalidMatrixA = -1022
    kInvalidMatrixB = -1021
    kInvalidMatrixC = -1020
    kInvalidDimension = -1017
    kInvalidLeadDimA = -1016
    kInvalidLeadDimB = -1015
    kInvalidLeadDimC = -1014
    kInsufficientMemoryA = -1011
    kInsufficientMemoryB = -1010
    kInsufficientMemoryC = -1009
    kInsufficientMemoryTemp = -2050
    kInvalidBatchCount = -2049
    kUnexpectedError = -2039


class BLASError(RuntimeError):
    """Counterpart of gpgpu::blas::BLASError (gpgpu/src/utilities/exceptions.hpp:24-35)."""

    def __init__(self, status):
        self.status = int(status)
        super().__init__("BLAS error %d: %s" % (self.status, status_string(self.status)))


class Event:
    """Pair of CUDA events recorded before and after the launch."""

    def __init__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.end = torch.cuda.Event(enable_timing=True)

    def elapsed_ms(self):
        self.end.synchronize()
        return self.start.elapsed_time(self.end)


_PRECISION = {torch.float16: Precision.Half, torch.bfloat16: Precision.BFloat16,
              torch.float32: Precision.Single}
_NP_SCALAR = {torch.float16: ctypes.c_uint16, torch.bfloat16: ctypes.c_uint16,
              torch.float32: ctypes.c_float}


def precision_of(buf):
    try:
        return _PRECISION[buf.dtype]
    except KeyError:
        raise BLASError(StatusCode.kNotImplemented)


def _scalar(value, dtype):
    """Packs a host scalar in the storage type T, as the reference passes `const T alpha`."""
    t = torch.tensor([value], dtype=dtype)
    if dtype == torch.float32:
        return ctypes.c_float(float(t.item()))
    return ctypes.c_uint16(int(t.view(torch.int16).item()) & 0xFFFF)


def _scalars(values, dtype):
    t = torch.as_tensor(values, dtype=torch.float64).to(dtype).contiguous()
    raw = t.view(torch.int16 if dtype != torch.float32 else torch.int32).numpy()
    return raw, raw.ctypes.data_as(ctypes.c_void_p)


def _ptr(buf, offset=0):
    if not buf.is_cuda:
        raise BLASError(StatusCode.kInvalidMatrixA)
    return ctypes.c_void_p(buf.data_ptr() + int(offset) * buf.element_size())


def _stream(queue):
    s = queue if queue is not None else torch.cuda.current_stream()
    return s, ctypes.c_void_p(s.cuda_stream)


_GEMM_WORKSPACES = {}
_SCRATCH = threading.local()


class scratch:
    """``with scratch(buffer):`` makes the calls of this thread take their device scratch (K-split
    partial sums, packed filter banks, channels-last copies) from ``buffer`` (a uint8 device tensor
    the caller owns) instead of the per-stream buffers that grow on demand: nothing is allocated
    inside, which a CUDA-graph capture of a sequence of calls needs. A call that needs more than
    the buffer holds raises."""

    def __init__(self, buffer):
        self.buffer = buffer

    def __enter__(self):
        self.previous = getattr(_SCRATCH, "buffer", None)
        _SCRATCH.buffer = self.buffer
        return self

    def __exit__(self, *exc):
        _SCRATCH.buffer = self.previous
        return False


def _caller_scratch(device, nbytes):
    buf = getattr(_SCRATCH, "buffer", None)
    if buf is None:
        return None
    if buf.device != device or buf.numel() < nbytes:
        raise BLASError(StatusCode.kInsufficientMemoryTemp)
    return buf


def _gemm_workspace(device, stream, nbytes):
    """One scratch buffer per (device, stream), grown on demand; calls on a stream are ordered, so
    they can share it."""
    own = _caller_scratch(device, nbytes)
    if own is not None:
        return own
    key = (device.index, stream.cuda_stream)
    buf = _GEMM_WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            buf.record_stream(stream)
        buf = torch.empty(int(nbytes), dtype=torch.uint8, device=device)
        buf.record_stream(stream)
        _GEMM_WORKSPACES[key] = buf
    return buf


def _check(rc):
    if rc != 0:
        raise BLASError(rc)


def _dims(layout, ta, tb, m, n, k):
    """a_one/a_two/... of Xgemm::ProcessArguments (routines/level3/xgemm.hpp:54-91)."""
    row = int(layout) == Layout.RowMajor
    a_rot = (not row and int(ta) != Transpose.NoTrans) or (row and int(ta) == Transpose.NoTrans)
    b_rot = (not row and int(tb) != Transpose.NoTrans) or (row and int(tb) == Transpose.NoTrans)
    a_one, a_two = (k, m) if a_rot else (m, k)
    b_one, b_two = (n, k) if b_rot else (k, n)
    c_one, c_two = (n, m) if row else (m, n)
    return a_one, a_two, b_one, b_two, c_one, c_two


def _test_matrix(one, two, buf, offset, ld, lead_err, mem_err):
    """TestMatrixA/B/C (gpgpu/src/utilities/buffer_test.hpp:24-55)."""
    if ld < one:
        raise BLASError(lead_err)
    if buf.numel() < ld * (two - 1) + one + offset:
        raise BLASError(mem_err)


def _validate(layout, ta, tb, m, n, k, a, a_off, a_ld, b, b_off, b_ld, c, c_off, c_ld):
    if m == 0 or n == 0 or k == 0:
        raise BLASError(StatusCode.kInvalidDimension)
    a_one, a_two, b_one, b_two, c_one, c_two = _dims(layout, ta, tb, m, n, k)
    for off in a_off:
        _test_matrix(a_one, a_two, a, off, a_ld, StatusCode.kInvalidLeadDimA,
                     StatusCode.kInsufficientMemoryA)
    for off in b_off:
        _test_matrix(b_one, b_two, b, off, b_ld, StatusCode.kInvalidLeadDimB,
                     StatusCode.kInsufficientMemoryB)
    for off in c_off:
        _test_matrix(c_one, c_two, c, off, c_ld, StatusCode.kInvalidLeadDimC,
                     StatusCode.kInsufficientMemoryC)


def gemm(layout, a_transpose, b_transpose, m, n, k, alpha, a_buffer, a_offset, a_ld, b_buffer,
         b_offset, b_ld, beta, c_buffer, c_offset, c_ld, queue=None, event=None):
    """C = alpha*op(A)*op(B) + beta*C  (gpgpu::blas::gemm, gblas.h:496-504)."""
    prec = precision_of(c_buffer)
    if a_buffer.dtype != c_buffer.dtype or b_buffer.dtype != c_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    _validate(layout, a_transpose, b_transpose, m, n, k, a_buffer, [a_offset], a_ld, b_buffer,
              [b_offset], b_ld, c_buffer, [c_offset], c_ld)
    al, be = _scalar(alpha, c_buffer.dtype), _scalar(beta, c_buffer.dtype)
    s, sp = _stream(queue)
    # scratch for a K-split of products with few output tiles (the reference's Xgemm takes its
    # temporaries from the context's pool, routines/level3/xgemm.cpp:107-223); 0 bytes = not useful
    need = lib().dlf_b200_gemm_workspace_bytes(int(prec), m, n, k)
    ws = _gemm_workspace(c_buffer.device, s, need) if need else None
    if event is not None:
        event.start.record(s)
    rc = lib().dlf_b200_gemm_ex(int(prec), int(layout), int(a_transpose), int(b_transpose), m, n, k,
                                ctypes.byref(al), _ptr(a_buffer, a_offset), a_ld,
                                _ptr(b_buffer, b_offset), b_ld, ctypes.byref(be),
                                _ptr(c_buffer, c_offset), c_ld,
                                ctypes.c_void_p(ws.data_ptr()) if ws is not None else None,
                                ws.numel() if ws is not None else 0, sp)
    if event is not None:
        event.end.record(s)
    _check(rc)


def gemmStridedBatched(layout, a_transpose, b_transpose, m, n, k, alpha, a_buffer, a_offset, a_ld,
                       a_stride, b_buffer, b_offset, b_ld, b_stride, beta, c_buffer, c_offset,
                       c_ld, c_stride, batch_count, queue=None, event=None):
    """gpgpu::blas::gemmStridedBatched (gblas.h:673-683); a stride of 0 shares an operand."""
    prec = precision_of(c_buffer)
    if a_buffer.dtype != c_buffer.dtype or b_buffer.dtype != c_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if batch_count < 1:
        raise BLASError(StatusCode.kInvalidBatchCount)
    last = batch_count - 1
    _validate(layout, a_transpose, b_transpose, m, n, k, a_buffer, [a_offset + last * a_stride],
              a_ld, b_buffer, [b_offset + last * b_stride], b_ld, c_buffer,
              [c_offset + last * c_stride], c_ld)
    al, be = _scalar(alpha, c_buffer.dtype), _scalar(beta, c_buffer.dtype)
    s, sp = _stream(queue)
    if event is not None:
        event.start.record(s)
    rc = lib().dlf_b200_gemm_strided_batched(
        int(prec), int(layout), int(a_transpose), int(b_transpose), m, n, k, ctypes.byref(al),
        _ptr(a_buffer, a_offset), a_ld, a_stride, _ptr(b_buffer, b_offset), b_ld, b_stride,
        ctypes.byref(be), _ptr(c_buffer, c_offset), c_ld, c_stride, batch_count, sp)
    if event is not None:
        event.end.record(s)
    _check(rc)


def gemmBatched(layout, a_transpose, b_transpose, m, n, k, alphas, a_buffer, a_offsets, a_ld,
                b_buffer, b_offsets, b_ld, betas, c_buffer, c_offsets, c_ld, batch_count,
                queue=None, event=None, workspace=None):
    """gpgpu::blas::gemmBatched (gblas.h:661-671): host arrays of per-batch scalars / offsets.

    ``workspace`` is a device byte buffer for the tables (the reference takes it from its
    TemporaryBuffer pool, gblas.cpp:2972-2988); allocated here when not given.
    """
    prec = precision_of(c_buffer)
    if a_buffer.dtype != c_buffer.dtype or b_buffer.dtype != c_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if (batch_count < 1 or len(alphas) != batch_count or len(betas) != batch_count or
            len(a_offsets) != batch_count or len(b_offsets) != batch_count or
            len(c_offsets) != batch_count):
        raise BLASError(StatusCode.kInvalidBatchCount)
    _validate(layout, a_transpose, b_transpose, m, n, k, a_buffer, list(a_offsets), a_ld,
              b_buffer, list(b_offsets), b_ld, c_buffer, list(c_offsets), c_ld)
    need = lib().dlf_b200_gemm_batched_workspace_bytes(batch_count)
    s, sp = _stream(queue)
    if workspace is None:
        workspace = torch.empty(max(need, 8), dtype=torch.uint8, device=c_buffer.device)
        # the tables are read by work queued on `s`, which may not be the allocator's current
        # stream: the block must not be handed out again before that work has passed
        workspace.record_stream(s)
    arr = ctypes.c_size_t * batch_count
    ao, bo, co = arr(*map(int, a_offsets)), arr(*map(int, b_offsets)), arr(*map(int, c_offsets))
    al_keep, al = _scalars(alphas, c_buffer.dtype)
    be_keep, be = _scalars(betas, c_buffer.dtype)
    if event is not None:
        event.start.record(s)
    rc = lib().dlf_b200_gemm_batched(
        int(prec), int(layout), int(a_transpose), int(b_transpose), m, n, k, al,
        _ptr(a_buffer), ao, a_ld, _ptr(b_buffer), bo, b_ld, be, _ptr(c_buffer), co, c_ld,
        batch_count, ctypes.c_void_p(workspace.data_ptr()), workspace.numel(), sp)
    if event is not None:
        event.end.record(s)
    del al_keep, be_keep
    _check(rc)


# ---------------------------------------------------------------------------------------------
# level-3 routines on the GEMM main loop (gblas.h:506-586)
# ---------------------------------------------------------------------------------------------
class Triangle(enum.IntEnum):
    Upper = 121
    Lower = 122


class Diagonal(enum.IntEnum):
    NonUnit = 131
    Unit = 132


class Side(enum.IntEnum):
    Left = 141
    Right = 142


_SYMM, _SYRK, _TRMM, _TRSM = 1, 2, 3, 4


def _level3_workspace(routine, buf, m, n, stream):
    need = lib().dlf_b200_level3_workspace_bytes(routine, int(precision_of(buf)), m, n)
    ws = torch.empty(max(int(need), 8), dtype=torch.uint8, device=buf.device)
    ws.record_stream(stream)  # read by work queued on `stream`, which may not be the allocator's
    return ws


def symm(layout, side, triangle, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset, b_ld, beta,
         c_buffer, c_offset, c_ld, queue=None, event=None):
    """C = alpha*S*B + beta*C (Left) or alpha*B*S + beta*C (Right), S symmetric, one triangle
    stored (gpgpu::blas::symm, gblas.h:506-515)."""
    prec = precision_of(c_buffer)
    if a_buffer.dtype != c_buffer.dtype or b_buffer.dtype != c_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if m == 0 or n == 0:
        raise BLASError(StatusCode.kInvalidDimension)
    ka = m if int(side) == Side.Left else n
    row = int(layout) == Layout.RowMajor
    _test_matrix(ka, ka, a_buffer, a_offset, a_ld, StatusCode.kInvalidLeadDimA, StatusCode.kInsufficientMemoryA)
    one, two = (n, m) if row else (m, n)
    _test_matrix(one, two, b_buffer, b_offset, b_ld, StatusCode.kInvalidLeadDimB, StatusCode.kInsufficientMemoryB)
    _test_matrix(one, two, c_buffer, c_offset, c_ld, StatusCode.kInvalidLeadDimC, StatusCode.kInsufficientMemoryC)
    al, be = _scalar(alpha, c_buffer.dtype), _scalar(beta, c_buffer.dtype)
    s, sp = _stream(queue)
    ws = _level3_workspace(_SYMM, c_buffer, m, n, s)
    if event is not None:
        event.start.record(s)
    rc = lib().dlf_b200_symm(int(prec), int(layout), int(side), int(triangle), m, n, ctypes.byref(al),
                             _ptr(a_buffer, a_offset), a_ld, _ptr(b_buffer, b_offset), b_ld, ctypes.byref(be),
                             _ptr(c_buffer, c_offset), c_ld, ctypes.c_void_p(ws.data_ptr()), ws.numel(), sp)
    if event is not None:
        event.end.record(s)
    _check(rc)


def syrk(layout, triangle, a_transpose, n, k, alpha, a_buffer, a_offset, a_ld, beta, c_buffer, c_offset, c_ld,
         queue=None, event=None):
    """The named triangle of C = alpha*op(A)*op(A)^T + beta*C (gpgpu::blas::syrk, gblas.h:528-536)."""
    prec = precision_of(c_buffer)
    if a_buffer.dtype != c_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if n == 0 or k == 0:
        raise BLASError(StatusCode.kInvalidDimension)
    row = int(layout) == Layout.RowMajor
    a_rot = (row and int(a_transpose) == Transpose.NoTrans) or (not row and int(a_transpose) != Transpose.NoTrans)
    one, two = (k, n) if a_rot else (n, k)
    _test_matrix(one, two, a_buffer, a_offset, a_ld, StatusCode.kInvalidLeadDimA, StatusCode.kInsufficientMemoryA)
    _test_matrix(n, n, c_buffer, c_offset, c_ld, StatusCode.kInvalidLeadDimC, StatusCode.kInsufficientMemoryC)
    al, be = _scalar(alpha, c_buffer.dtype), _scalar(beta, c_buffer.dtype)
    s, sp = _stream(queue)
    ws = _level3_workspace(_SYRK, c_buffer, n, n, s)
    if event is not None:
        event.start.record(s)
    rc = lib().dlf_b200_syrk(int(prec), int(layout), int(triangle), int(a_transpose), n, k, ctypes.byref(al),
                             _ptr(a_buffer, a_offset), a_ld, ctypes.byref(be), _ptr(c_buffer, c_offset), c_ld,
                             ctypes.c_void_p(ws.data_ptr()), ws.numel(), sp)
    if event is not None:
        event.end.record(s)
    _check(rc)


def _triangular(fn_name, routine, layout, side, triangle, a_transpose, diagonal, m, n, alpha, a_buffer, a_offset,
                a_ld, b_buffer, b_offset, b_ld, queue, event):
    prec = precision_of(b_buffer)
    if a_buffer.dtype != b_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if m == 0 or n == 0:
        raise BLASError(StatusCode.kInvalidDimension)
    ka = m if int(side) == Side.Left else n
    row = int(layout) == Layout.RowMajor
    _test_matrix(ka, ka, a_buffer, a_offset, a_ld, StatusCode.kInvalidLeadDimA, StatusCode.kInsufficientMemoryA)
    one, two = (n, m) if row else (m, n)
    _test_matrix(one, two, b_buffer, b_offset, b_ld, StatusCode.kInvalidLeadDimB, StatusCode.kInsufficientMemoryB)
    al = _scalar(alpha, b_buffer.dtype)
    s, sp = _stream(queue)
    ws = _level3_workspace(routine, b_buffer, m, n, s)
    if event is not None:
        event.start.record(s)
    rc = getattr(lib(), fn_name)(int(prec), int(layout), int(side), int(triangle), int(a_transpose), int(diagonal),
                                 m, n, ctypes.byref(al), _ptr(a_buffer, a_offset), a_ld, _ptr(b_buffer, b_offset),
                                 b_ld, ctypes.c_void_p(ws.data_ptr()), ws.numel(), sp)
    if event is not None:
        event.end.record(s)
    _check(rc)


def trmm(layout, side, triangle, a_transpose, diagonal, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset,
         b_ld, queue=None, event=None):
    """B = alpha*op(T)*B (Left) or alpha*B*op(T) (Right), in place (gpgpu::blas::trmm, gblas.h:570-577)."""
    _triangular("dlf_b200_trmm", _TRMM, layout, side, triangle, a_transpose, diagonal, m, n, alpha, a_buffer,
                a_offset, a_ld, b_buffer, b_offset, b_ld, queue, event)


def trsm(layout, side, triangle, a_transpose, diagonal, m, n, alpha, a_buffer, a_offset, a_ld, b_buffer, b_offset,
         b_ld, queue=None, event=None):
    """Solves op(T)*X = alpha*B (Left) or X*op(T) = alpha*B (Right); X overwrites B
    (gpgpu::blas::trsm, gblas.h:579-586)."""
    _triangular("dlf_b200_trsm", _TRSM, layout, side, triangle, a_transpose, diagonal, m, n, alpha, a_buffer,
                a_offset, a_ld, b_buffer, b_offset, b_ld, queue, event)
