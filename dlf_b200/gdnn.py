"""Host-side mirror of ``gpgpu::dnn::conv2d`` (gpgpu/include/gdnn.h:201-213) plus the
``Filter2D`` geometry of dlf/include/tensor/dnn.h:9-122 that its callers use.

``conv2d`` keeps the reference's argument order. One argument is added at the end: ``bias``
(``num_kernels`` values), which the reference applies as a separate pass over Y
(``ConvOp::evaluate``, dlf/include/predict.h:1272-1281) and this backend folds into the
convolution's epilogue.
"""
import ctypes

import torch

from . import lib
from .gblas import BLASError, StatusCode, _caller_scratch, _check, _ptr, _stream, precision_of


class Filter2D:
    """Geometry of a 2-D filter: NCHW input, OIHW kernel (dnn.h:9-122)."""

    def __init__(self, input_shape, kernel_shape, group=1, kernel_w=None):
        """Filter2D(input_shape, kernel_shape, group) for convolutions, or
        Filter2D(input_shape, kernel_h, kernel_w) for pooling (dlf/src/tensor/filter.cpp:5-25)."""
        self.batches, self.channels, self.height, self.width = map(int, input_shape)
        if isinstance(kernel_shape, int):
            # pooling form: the second and third arguments are kernel_h, kernel_w
            self.kernel_h = int(kernel_shape)
            self.kernel_w = int(kernel_w if kernel_w is not None else group)
            self.num_kernels, self.group = self.channels, 1
        else:
            self.num_kernels, cpg, self.kernel_h, self.kernel_w = map(int, kernel_shape)
            self.group = int(group)
            if cpg * self.group != self.channels:
                raise ValueError("kernel channels * group != input channels")
        self.pad_top = self.pad_left = self.pad_bottom = self.pad_right = 0
        self.stride_h = self.stride_w = 1
        self.dilation_h = self.dilation_w = 1

    def pads(self, *p):
        if len(p) == 2:
            self.pad_top = self.pad_bottom = int(p[0])
            self.pad_left = self.pad_right = int(p[1])
        else:
            self.pad_top, self.pad_left, self.pad_bottom, self.pad_right = map(int, p)
        return self

    def auto_pad(self, mode):
        """dlf/src/tensor/filter.cpp:51-82."""
        if mode == "VALID":
            self.pad_top = self.pad_left = self.pad_bottom = self.pad_right = 0
        elif mode in ("SAME_UPPER", "SAME_LOWER"):
            def pad(size, kernel, stride, dilation):
                ext = (kernel - 1) * dilation + 1
                total = max(((size - 1) // stride) * stride + ext - size, 0)
                half = total >> 1
                return (half, total - half) if mode == "SAME_UPPER" else (total - half, half)
            self.pad_top, self.pad_bottom = pad(self.height, self.kernel_h, self.stride_h, self.dilation_h)
            self.pad_left, self.pad_right = pad(self.width, self.kernel_w, self.stride_w, self.dilation_w)
        return self

    def strides(self, h, w):
        self.stride_h, self.stride_w = int(h), int(w)
        return self

    def dilations(self, h, w):
        self.dilation_h, self.dilation_w = int(h), int(w)
        return self

    @property
    def output_h(self):  # dnn.h:99-103
        size = self.height + self.pad_top + self.pad_bottom
        ext = self.dilation_h * (self.kernel_h - 1) + 1
        return (size - ext) // self.stride_h + 1 if size >= ext else 1

    @property
    def output_w(self):  # dnn.h:105-109
        size = self.width + self.pad_left + self.pad_right
        ext = self.dilation_w * (self.kernel_w - 1) + 1
        return (size - ext) // self.stride_w + 1 if size >= ext else 1

    def output_shape(self):
        return (self.batches, self.num_kernels, self.output_h, self.output_w)


_WORKSPACES = {}


def _workspace(device, stream, nbytes):
    """Scratch for the packed filter bank, one buffer per (device, stream), grown on demand - the
    role the context's temporary-buffer pool plays in the reference (gpgpu/src/gpgpu.cpp:189-214).
    Calls on one stream are ordered, so they can share it."""
    own = _caller_scratch(device, nbytes)
    if own is not None:
        return own
    key = (device.index, stream.cuda_stream)
    buf = _WORKSPACES.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            # earlier convolutions queued on this stream may still read the old buffer
            buf.record_stream(stream)
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        buf.record_stream(stream)
        _WORKSPACES[key] = buf
    return buf


def conv2d(batches, channels, height, width, output_h, output_w, num_kernels, group, kernel_h,
           kernel_w, pad_top, pad_left, pad_bottom, pad_right, stride_h, stride_w, dilation_h,
           dilation_w, im_buffer, kernel_buffer, result_buffer, queue=None, event=None, bias=None,
           residual=None, activation=None):
    """NCHW cross-correlation into result_buffer (gpgpu::dnn::conv2d, gdnn.h:201-213).

    ``bias``, ``residual`` (a tensor shaped like the result, may be the result itself) and
    ``activation`` (None or "relu") fuse what dlf's graph runtime runs as separate passes after
    the convolution: the bias add of ConvOp (dlf/include/predict.h:1272-1281), the Add of a
    residual connection and the Relu that follows it."""
    prec = precision_of(result_buffer)
    if im_buffer.dtype != result_buffer.dtype or kernel_buffer.dtype != result_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if bias is not None and bias.dtype != result_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if group < 1 or channels % group or num_kernels % group:
        raise BLASError(StatusCode.kInvalidDimension)
    if im_buffer.numel() < batches * channels * height * width:
        raise BLASError(StatusCode.kInsufficientMemoryA)
    if kernel_buffer.numel() < num_kernels * (channels // group) * kernel_h * kernel_w:
        raise BLASError(StatusCode.kInsufficientMemoryB)
    if result_buffer.numel() < batches * num_kernels * output_h * output_w:
        raise BLASError(StatusCode.kInsufficientMemoryC)
    if bias is not None and bias.numel() < num_kernels:
        raise BLASError(StatusCode.kInvalidValue)
    if residual is not None and (residual.dtype != result_buffer.dtype or
                                 residual.numel() < batches * num_kernels * output_h * output_w):
        raise BLASError(StatusCode.kInvalidValue)
    if activation not in (None, "relu"):
        raise BLASError(StatusCode.kInvalidValue)
    s, sp = _stream(queue)
    ws = _workspace(result_buffer.device, s, lib().dlf_b200_conv2d_workspace_bytes(
        int(prec), batches, channels, height, width, output_h, output_w, num_kernels, group,
        kernel_h, kernel_w))
    if event is not None:
        event.start.record(s)
    null = ctypes.c_void_p(0)
    rc = lib().dlf_b200_conv2d_fused(
        int(prec), batches, channels, height, width, output_h, output_w, num_kernels, group,
        kernel_h, kernel_w, pad_top, pad_left, pad_bottom, pad_right, stride_h, stride_w,
        dilation_h, dilation_w, _ptr(im_buffer), _ptr(kernel_buffer),
        _ptr(bias) if bias is not None else null,
        _ptr(residual) if residual is not None else null, 1 if activation == "relu" else 0,
        _ptr(result_buffer), ctypes.c_void_p(ws.data_ptr()), ws.numel(), sp)
    if event is not None:
        event.end.record(s)
    _check(rc)


def conv2d_filter(X, W, Y, filt, bias=None, queue=None, event=None, residual=None, activation=None):
    """dlf::dnn::conv2d(X, W, Y, filter) for device tensors (dlf/include/tensor/dnn_detail.h:154-166)."""
    conv2d(filt.batches, filt.channels, filt.height, filt.width, filt.output_h, filt.output_w,
           filt.num_kernels, filt.group, filt.kernel_h, filt.kernel_w, filt.pad_top,
           filt.pad_left, filt.pad_bottom, filt.pad_right, filt.stride_h, filt.stride_w,
           filt.dilation_h, filt.dilation_w, X, W, Y, queue=queue, event=event, bias=bias,
           residual=residual, activation=activation)


def _pool(fn_name, extra, batches, channels, height, width, output_h, output_w, kernel_h, kernel_w, pad_top,
          pad_left, pad_bottom, pad_right, stride_h, stride_w, dilation_h, dilation_w, x_buffer, y_buffer,
          queue, event):
    prec = precision_of(y_buffer)
    if x_buffer.dtype != y_buffer.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if x_buffer.numel() < batches * channels * height * width:
        raise BLASError(StatusCode.kInsufficientMemoryA)
    if y_buffer.numel() < batches * channels * output_h * output_w:
        raise BLASError(StatusCode.kInsufficientMemoryC)
    s, sp = _stream(queue)
    if event is not None:
        event.start.record(s)
    rc = getattr(lib(), fn_name)(
        int(prec), batches, channels, height, width, output_h, output_w, kernel_h, kernel_w, pad_top,
        pad_left, pad_bottom, pad_right, stride_h, stride_w, dilation_h, dilation_w, *extra,
        _ptr(x_buffer), _ptr(y_buffer), sp)
    if event is not None:
        event.end.record(s)
    _check(rc)


def maxpool(batches, channels, height, width, output_h, output_w, kernel_h, kernel_w, pad_top, pad_left,
            pad_bottom, pad_right, stride_h, stride_w, dilation_h, dilation_w, x_buffer, y_buffer,
            queue=None, event=None):
    """gpgpu::dnn::maxpool, in the argument order of its definition and of its callers
    (gpgpu/src/gdnn.cpp:1667-1676; dlf/include/tensor/dnn.h:218-229)."""
    _pool("dlf_b200_maxpool", (), batches, channels, height, width, output_h, output_w, kernel_h, kernel_w,
          pad_top, pad_left, pad_bottom, pad_right, stride_h, stride_w, dilation_h, dilation_w, x_buffer,
          y_buffer, queue, event)


def avgpool(batches, channels, height, width, output_h, output_w, kernel_h, kernel_w, pad_top, pad_left,
            pad_bottom, pad_right, stride_h, stride_w, dilation_h, dilation_w, count_include_pad, x_buffer,
            y_buffer, queue=None, event=None):
    """gpgpu::dnn::avgpool (gpgpu/src/gdnn.cpp:1728-1738; dlf/include/tensor/dnn.h:249-261)."""
    _pool("dlf_b200_avgpool", (1 if count_include_pad else 0,), batches, channels, height, width, output_h,
          output_w, kernel_h, kernel_w, pad_top, pad_left, pad_bottom, pad_right, stride_h, stride_w,
          dilation_h, dilation_w, x_buffer, y_buffer, queue, event)


def _filter_args(f):
    return (f.batches, f.channels, f.height, f.width, f.output_h, f.output_w, f.kernel_h, f.kernel_w,
            f.pad_top, f.pad_left, f.pad_bottom, f.pad_right, f.stride_h, f.stride_w, f.dilation_h,
            f.dilation_w)


def max_pooling(X, Y, filt, queue=None, event=None):
    """dlf::dnn::max_pooling(X, Y, filter) for device tensors (dlf/include/tensor/dnn.h:217-229)."""
    maxpool(*_filter_args(filt), X, Y, queue=queue, event=event)


def average_pooling(X, Y, filt, count_include_pad, queue=None, event=None):
    """dlf::dnn::average_pooling(X, Y, filter, count_include_pad) (dnn.h:248-262)."""
    avgpool(*_filter_args(filt), count_include_pad, X, Y, queue=queue, event=event)


def global_max_pooling(X, Y, queue=None, event=None):
    """dlf::dnn::global_max_pooling for device tensors: max_pooling with the whole plane as the
    window (dlf/include/tensor/dnn.h:346-351)."""
    h, w = int(X.shape[2]), int(X.shape[3])
    max_pooling(X, Y, Filter2D(X.shape, h, w).strides(h, w), queue=queue, event=event)


def global_average_pooling(X, Y, queue=None, event=None):
    """dlf::dnn::global_average_pooling for device tensors (dnn.h:361-375)."""
    h, w = int(X.shape[2]), int(X.shape[3])
    average_pooling(X, Y, Filter2D(X.shape, h, w).strides(h, w), False, queue=queue, event=event)


# ---------------------------------------------------------------------------------------------
# Channels-last operators (16-bit, (N, H, W, C) with C a multiple of 8): what an operator-list
# runtime that owns its intermediate tensors uses between its operators. The reference's operators
# are NCHW; these compute the same functions on the permuted tensors.

NHWC, NCHW = 0, 1


def nhwc_supported(filt, dtype, y_layout=NHWC):
    """Whether conv2d_nhwc serves this convolution (the limits of the tensor-map unit's im2col mode;
    the C entry returns kNotImplemented otherwise and launches nothing)."""
    f = filt
    return (dtype in (torch.float16, torch.bfloat16) and f.group == 1 and f.channels % 8 == 0 and
            (y_layout == NCHW or f.num_kernels % 8 == 0) and f.kernel_h <= 16 and f.kernel_w <= 16 and
            f.pad_top < 128 and f.pad_left < 128 and f.stride_h <= 8 and f.stride_w <= 8 and
            f.dilation_h * (f.kernel_h - 1) < 256 and f.dilation_w * (f.kernel_w - 1) < 256 and f.batches < 65536 and
            (f.output_w - 1) * f.stride_w + 1 - f.width - f.pad_left <= 127 and
            (f.output_h - 1) * f.stride_h + 1 - f.height - f.pad_top <= 127)


def pack_filters_nhwc(W, queue=None):
    """OIHW filter bank -> (Cout, KH*KW, Ck), Ck = C rounded up to 64 (zero-filled): the K-major operand
    conv2d_nhwc reads."""
    prec = precision_of(W)
    co, c, kh, kw = (int(d) for d in W.shape)
    n = lib().dlf_b200_nhwc_filter_elems(c, co, kh, kw)
    out = torch.empty(n, dtype=W.dtype, device=W.device)
    _, sp = _stream(queue)
    _check(lib().dlf_b200_pack_filters_nhwc(int(prec), c, co, kh, kw, _ptr(W.contiguous()), _ptr(out), sp))
    return out


def nchw_to_nhwc(X, Y=None, queue=None):
    """(N, C, H, W) -> (N, H, W, C') with C' = C rounded up to 8 (the added channels zero)."""
    prec = precision_of(X)
    n, c, h, w = (int(d) for d in X.shape)
    cp = (c + 7) // 8 * 8
    if Y is None:
        Y = torch.empty((n, h, w, cp), dtype=X.dtype, device=X.device)
    elif Y.numel() < n * h * w * cp or Y.dtype != X.dtype:
        raise BLASError(StatusCode.kInsufficientMemoryC)
    _, sp = _stream(queue)
    _check(lib().dlf_b200_nchw_to_nhwc(int(prec), n, c, h, w, _ptr(X), _ptr(Y), sp))
    return Y


def conv2d_nhwc(X, W_packed, Y, filt, bias=None, residual=None, activation=None, y_layout=NHWC, queue=None):
    """Y = act(conv2d(X, W) + bias + residual) with X (N, H, W, C), the filter bank as
    pack_filters_nhwc writes it, and Y / residual in ``y_layout``. One launch, no scratch."""
    f = filt
    prec = precision_of(Y)
    if X.dtype != Y.dtype or W_packed.dtype != Y.dtype or (bias is not None and bias.dtype != Y.dtype) or \
            (residual is not None and residual.dtype != Y.dtype):
        raise BLASError(StatusCode.kInvalidValue)
    if X.numel() < f.batches * f.channels * f.height * f.width:
        raise BLASError(StatusCode.kInsufficientMemoryA)
    if W_packed.numel() < lib().dlf_b200_nhwc_filter_elems(f.channels, f.num_kernels, f.kernel_h, f.kernel_w):
        raise BLASError(StatusCode.kInsufficientMemoryB)
    n_out = f.batches * f.num_kernels * f.output_h * f.output_w
    if Y.numel() < n_out or (residual is not None and residual.numel() < n_out):
        raise BLASError(StatusCode.kInsufficientMemoryC)
    if activation not in (None, "relu"):
        raise BLASError(StatusCode.kInvalidValue)
    _, sp = _stream(queue)
    null = ctypes.c_void_p(0)
    _check(lib().dlf_b200_conv2d_nhwc(
        int(prec), f.batches, f.channels, f.height, f.width, f.output_h, f.output_w, f.num_kernels, f.kernel_h,
        f.kernel_w, f.pad_top, f.pad_left, f.pad_bottom, f.pad_right, f.stride_h, f.stride_w, f.dilation_h,
        f.dilation_w, _ptr(X), _ptr(W_packed), _ptr(bias) if bias is not None else null,
        _ptr(residual) if residual is not None else null, 1 if activation == "relu" else 0, _ptr(Y), int(y_layout), sp))


def pool_nhwc(X, Y, filt, average=False, count_include_pad=False, queue=None):
    """max / average pooling on (N, H, W, C) tensors; ``filt`` is the pooling Filter2D of the NCHW shape."""
    f = filt
    prec = precision_of(Y)
    if f.dilation_h != 1 or f.dilation_w != 1:
        raise BLASError(StatusCode.kNotImplemented)
    if X.dtype != Y.dtype:
        raise BLASError(StatusCode.kInvalidValue)
    if X.numel() < f.batches * f.channels * f.height * f.width:
        raise BLASError(StatusCode.kInsufficientMemoryA)
    if Y.numel() < f.batches * f.channels * f.output_h * f.output_w:
        raise BLASError(StatusCode.kInsufficientMemoryC)
    _, sp = _stream(queue)
    _check(lib().dlf_b200_pool_nhwc(int(prec), 1 if average else 0, 1 if count_include_pad else 0, f.batches, f.channels,
                                    f.height, f.width, f.output_h, f.output_w, f.kernel_h, f.kernel_w, f.pad_top,
                                    f.pad_left, f.stride_h, f.stride_w, _ptr(X), _ptr(Y), sp))
