"""Operator-list execution of a model graph on the device.

This is the part of dlf's graph runtime that reaches this library's kernels: a ``Predictor``
(dlf/include/predict.h:137-163) turns the nodes of a graph into a flat list of operators over
preallocated device tensors and ``predict()`` evaluates the list in order (predict.h:2048-2070).
The operators are the ones whose work is a contraction or a pooling pass of this library -
``Conv`` (predict.h:1258-1286), ``Gemm`` (:1203-1226), ``MatMul`` (:1228-1241), ``MaxPool`` /
``AveragePool`` / ``GlobalAveragePool`` / ``GlobalMaxPool`` (:1288-1370) - plus the shape-only
``Flatten`` / ``Reshape`` / ``Identity``, and the nodes the optimizer folds into a convolution:
``BatchNormalization`` and a bias ``Add`` (dlf/src/model/passes.hpp:162-263, 330-403), the ``Add``
of a residual connection and the ``Relu`` that follows a convolution (one fused launch instead of
the reference's separate element-wise passes). A node that is none of these is refused when the
predictor is built: nothing is computed outside the library.

Once the list has run once, it is captured into a CUDA graph and later ``predict()`` calls replay
the graph: one submission instead of a launch (and its host-side argument work) per operator.

The graph is built with a small rendition of the reference's IR (dlf/include/model/graph.h:
``Graph::append / addInput / addInitializer / addOutput``, ``Node::addInput / addOutput``); reading
ONNX files is not part of this library.
"""
import enum

import numpy as np
import torch

from . import gblas, gdnn, lib
from . import tensor as linalg
from .gblas import Transpose


class DataType(enum.IntEnum):
    """Element types by their ONNX numbers, as dlf/include/model/graph.h uses them."""
    FLOAT = 1
    INT64 = 7
    FLOAT16 = 10
    DOUBLE = 11
    BFLOAT16 = 16


class ShapeInferenceError(RuntimeError):
    """dlf/include/model/graph.h:1312-1318."""


class Value:
    """An edge of the graph: a graph input, an initializer or the output of a node."""

    def __init__(self, name, dtype=None, dims=None, initializer=None):
        self.name = name
        self.dtype = dtype
        self.dims = None if dims is None else tuple(int(d) for d in dims)
        self.initializer = initializer
        self.node = None

    def has_initializer(self):
        return self.initializer is not None

    def __repr__(self):
        return "Value(%r, %r)" % (self.name, self.dims)


class Node:
    """One operator of the graph; attributes carry the ONNX names."""

    def __init__(self, kind, attrs):
        self.kind = kind
        self.attrs = dict(attrs)
        self.inputs = []
        self.outputs = []

    def addInput(self, value):
        self.inputs.append(value)
        return self

    def addOutput(self, name):
        v = Value(name)
        v.node = self
        self.outputs.append(v)
        return v

    def input(self, i=0):
        return self.inputs[i] if i < len(self.inputs) else None

    def output(self, i=0):
        return self.outputs[i]

    def get(self, name, default=None):
        return self.attrs.get(name, default)

    def __repr__(self):
        return "Node(%s -> %s)" % (self.kind, [v.name for v in self.outputs])


class Graph:
    """Nodes in evaluation order, graph inputs (initializers among them) and graph outputs."""

    def __init__(self):
        self.nodes = []
        self.inputs = []
        self.outputs = []

    def append(self, kind, **attrs):
        n = Node(kind, attrs)
        self.nodes.append(n)
        return n

    def addInput(self, name, dtype, dims):
        v = Value(name, dtype, dims)
        self.inputs.append(v)
        return v

    def addInitializer(self, name, data, dtype=None):
        a = np.asarray(data)
        if dtype is None:
            dtype = DataType.INT64 if a.dtype.kind in "iu" else (DataType.DOUBLE if a.dtype == np.float64 else DataType.FLOAT)
        v = Value(name, dtype, a.shape, a)
        self.inputs.append(v)
        return v

    def addOutput(self, value):
        self.outputs.append(value)
        return value

    # -- what the optimizer passes need ------------------------------------------------------

    def uses(self, value):
        """Number of places a value is read: node inputs (the residual operand of a fused
        convolution among them) and graph outputs."""
        n = sum(1 for node in self.nodes for v in node.inputs if v is value)
        n += sum(1 for node in self.nodes if node.attrs.get("residual") is value)
        return n + sum(1 for v in self.outputs if v is value)

    def replace_all_uses(self, old, new):
        for node in self.nodes:
            node.inputs = [new if v is old else v for v in node.inputs]
            if node.attrs.get("residual") is old:
                node.attrs["residual"] = new
        self.outputs = [new if v is old else v for v in self.outputs]

    def erase(self, node):
        self.nodes.remove(node)

    def drop_unused_inputs(self):
        self.inputs = [v for v in self.inputs if not v.has_initializer() or self.uses(v) > 0]


# ---------------------------------------------------------------------------------------------
# shape inference for the supported nodes (dlf/src/model/shape_inference.cpp)


def _pair(v, default):
    if v is None:
        return (default, default)
    v = tuple(int(x) for x in v)
    if len(v) != 2:
        raise ShapeInferenceError("only 2-D filters are supported")
    return v


def _pads(node):
    p = node.get("pads")
    if p is None:
        return (0, 0, 0, 0)
    p = tuple(int(x) for x in p)
    if len(p) != 4:
        raise ShapeInferenceError("pads must have 4 values")
    return p  # ONNX order: top, left, bottom, right


def _conv_filter(node, x_dims, w_dims):
    """dnn::Filter2D of a Conv node (predict.h:1262-1270)."""
    f = gdnn.Filter2D(x_dims, w_dims, int(node.get("group", 1)))
    ks = node.get("kernel_shape")
    if ks is not None and tuple(int(k) for k in ks) != tuple(w_dims[2:]):
        raise ShapeInferenceError("Conv: kernel_shape does not match the weights")
    mode = node.get("auto_pad", "NOTSET")
    f.strides(*_pair(node.get("strides"), 1)).dilations(*_pair(node.get("dilations"), 1))
    if mode in (None, "NOTSET"):
        f.pads(*_pads(node))
    else:
        f.auto_pad(mode)
    return f


def _pool_filter(node, x_dims):
    """dnn::Filter2D of a pooling node (predict.h:1292-1298)."""
    if int(node.get("ceil_mode", 0)) != 0:
        raise ShapeInferenceError("%s: ceil_mode is not supported" % node.kind)
    kh, kw = _pair(node.get("kernel_shape"), 1)
    f = gdnn.Filter2D(x_dims, kh, kw)
    f.strides(*_pair(node.get("strides"), 1)).dilations(*_pair(node.get("dilations"), 1))
    mode = node.get("auto_pad", "NOTSET")
    if mode in (None, "NOTSET"):
        f.pads(*_pads(node))
    else:
        f.auto_pad(mode)
    return f


def _need(node, i, what):
    v = node.input(i)
    if v is None or v.dims is None:
        raise ShapeInferenceError("%s: %s has no shape" % (node.kind, what))
    return v


def _broadcast_dims(a, b):
    out = []
    for i in range(1, max(len(a), len(b)) + 1):
        x = a[-i] if i <= len(a) else 1
        y = b[-i] if i <= len(b) else 1
        if x != y and x != 1 and y != 1:
            raise ShapeInferenceError("incompatible shapes %r and %r" % (a, b))
        out.append(max(x, y))
    return tuple(reversed(out))


def infer_shapes(graph):
    """Fills in the dims and dtype of every node output (the reference runs
    ShapeInference::infer before it builds the operators, predict.h:2051)."""
    for node in graph.nodes:
        k = node.kind
        x = _need(node, 0, "input")
        if k == "Conv":
            w = _need(node, 1, "W")
            if len(x.dims) != 4 or len(w.dims) != 4:
                raise ShapeInferenceError("Conv: only 2-D convolutions (NCHW, OIHW) are supported")
            group = int(node.get("group", 1))
            if x.dims[1] != w.dims[1] * group or w.dims[0] % group:
                raise ShapeInferenceError("Conv: channels do not match the weights")
            dims = tuple(_conv_filter(node, x.dims, w.dims).output_shape())
        elif k in ("MaxPool", "AveragePool"):
            if len(x.dims) != 4:
                raise ShapeInferenceError("%s: only 2-D pooling is supported" % k)
            dims = tuple(_pool_filter(node, x.dims).output_shape())
        elif k in ("GlobalAveragePool", "GlobalMaxPool"):
            if len(x.dims) != 4:
                raise ShapeInferenceError("%s: only 2-D pooling is supported" % k)
            dims = (x.dims[0], x.dims[1], 1, 1)
        elif k == "Gemm":
            b = _need(node, 1, "B")
            if len(x.dims) != 2 or len(b.dims) != 2:
                raise ShapeInferenceError("Gemm: A and B must be matrices")
            m, ka = x.dims if not node.get("transA", 0) else x.dims[::-1]
            kb, n = b.dims if not node.get("transB", 0) else b.dims[::-1]
            if ka != kb:
                raise ShapeInferenceError("Gemm: incompatible shapes")
            if node.input(2) is not None:
                _broadcast_dims(_need(node, 2, "C").dims, (m, n))
            dims = (m, n)
        elif k == "MatMul":
            b = _need(node, 1, "B")
            a_d, b_d = x.dims, b.dims
            if len(a_d) < 1 or len(b_d) < 1:
                raise ShapeInferenceError("MatMul: scalars are not supported")
            a2 = a_d if len(a_d) > 1 else (1,) + a_d
            b2 = b_d if len(b_d) > 1 else b_d + (1,)
            if a2[-1] != b2[-2]:
                raise ShapeInferenceError("MatMul: incompatible shapes")
            dims = _broadcast_dims(a2[:-2], b2[:-2]) + (a2[-2], b2[-1])
            if len(a_d) == 1:
                dims = dims[:-2] + dims[-1:]
            if len(b_d) == 1:
                dims = dims[:-1]
        elif k == "Flatten":
            axis = int(node.get("axis", 1))
            if axis < 0:
                axis += len(x.dims)
            dims = (int(np.prod(x.dims[:axis], dtype=np.int64)), int(np.prod(x.dims[axis:], dtype=np.int64)))
        elif k == "Reshape":
            s = node.input(1)
            if s is None or not s.has_initializer():
                raise ShapeInferenceError("Reshape: the shape must be an initializer")
            want = [int(d) for d in np.asarray(s.initializer).reshape(-1)]
            total = int(np.prod(x.dims, dtype=np.int64))
            dims = [x.dims[i] if d == 0 else d for i, d in enumerate(want)]
            if dims.count(-1) > 1:
                raise ShapeInferenceError("Reshape: more than one -1")
            if -1 in dims:
                rest = int(np.prod([d for d in dims if d != -1], dtype=np.int64))
                if rest == 0 or total % rest:
                    raise ShapeInferenceError("Reshape: cannot infer the free dimension")
                dims[dims.index(-1)] = total // rest
            if int(np.prod(dims, dtype=np.int64)) != total:
                raise ShapeInferenceError("Reshape: element count differs")
            dims = tuple(dims)
        elif k in ("Relu", "Identity", "BatchNormalization", "Dropout"):
            dims = x.dims
        elif k == "Add":
            dims = _broadcast_dims(x.dims, _need(node, 1, "B").dims)
        else:
            raise ShapeInferenceError("operator %s is outside this library's path" % k)
        out = node.output(0)
        out.dims = dims
        out.dtype = x.dtype
    return graph


# ---------------------------------------------------------------------------------------------
# optimizer passes


def _float_type(value):
    return np.float64 if value.dtype == DataType.DOUBLE else np.float32


def fuse_bn_into_conv(graph):
    """W' = W * s / sqrt(var + eps), b' = (b - mean) * s / sqrt(var + eps) + b_bn
    (dlf/src/model/passes.hpp:150-263): a BatchNormalization whose input is a convolution read by
    nothing else disappears into the convolution's initializers."""
    changed = False
    for bn in list(graph.nodes):
        if bn.kind != "BatchNormalization" or bn.input(0).node is None or bn.input(0).node.kind != "Conv":
            continue
        conv = bn.input(0).node
        if graph.uses(bn.input(0)) > 1 or len(bn.outputs) > 1 or len(bn.inputs) < 5:
            continue
        params = bn.inputs[1:5]
        cw, cb = conv.input(1), conv.input(2)
        if not all(p is not None and p.has_initializer() for p in params) or not cw.has_initializer():
            continue
        if cb is not None and not cb.has_initializer():
            continue
        ft = _float_type(cw)
        scale, b_bn, mean, var = (np.asarray(p.initializer, dtype=ft).reshape(-1) for p in params)
        w = np.asarray(cw.initializer, dtype=ft)
        if w.shape[0] != scale.shape[0]:
            continue
        b = np.asarray(cb.initializer, dtype=ft).reshape(-1) if cb is not None else np.zeros_like(scale)
        scale = scale / np.sqrt(var + ft(bn.get("epsilon", 1e-5)))
        b = (b - mean) * scale + b_bn
        cw.initializer = (w * scale.reshape((-1,) + (1,) * (w.ndim - 1))).astype(ft)
        if cb is not None:
            cb.initializer = b.astype(ft)
        else:
            conv.addInput(graph.addInitializer(conv.output(0).name + ":bias", b.astype(ft), cw.dtype))
        graph.replace_all_uses(bn.output(0), bn.input(0))
        graph.erase(bn)
        changed = True
    graph.drop_unused_inputs()
    return changed


def fuse_add_bias_into_conv(graph):
    """An Add of an initializer shaped (1, M, 1, 1) or (M, 1, 1) to a convolution read by nothing
    else becomes the convolution's bias (dlf/src/model/passes.hpp:330-403)."""
    changed = False
    for add in list(graph.nodes):
        if add.kind != "Add" or add.input(0).node is None or add.input(0).node.kind != "Conv":
            continue
        conv, val = add.input(0).node, add.input(1)
        y = conv.output(0)
        if graph.uses(y) != 1 or y.dims is None or not val.has_initializer():
            continue
        cw, cb = conv.input(1), conv.input(2)
        if cw.dims is None or (cb is not None and not cb.has_initializer()):
            continue
        m = cw.dims[0]
        vd = tuple(np.asarray(val.initializer).shape)
        if len(vd) == len(y.dims):
            ok = vd[0] == 1 and vd[1] == m and all(d == 1 for d in vd[2:])
        elif len(vd) == len(y.dims) - 1:
            ok = vd[0] == m and all(d == 1 for d in vd[1:])
        else:
            ok = False
        if not ok:
            continue
        ft = _float_type(cw)
        bias = np.asarray(val.initializer, dtype=ft).reshape(-1)
        if cb is None:
            conv.addInput(graph.addInitializer(y.name + ":bias", bias, cw.dtype))
        else:
            cb.initializer = (np.asarray(cb.initializer, dtype=ft).reshape(-1) + bias).astype(ft)
        graph.replace_all_uses(add.output(0), y)
        graph.erase(add)
        changed = True
    graph.drop_unused_inputs()
    return changed


def fuse_residual_and_relu_into_conv(graph):
    """Conv -> [Add of a residual] -> [Relu] becomes one Conv node with ``residual`` and ``relu``
    marks, which the operator hands to the fused convolution entry (bias, residual and ReLU applied
    to the accumulator before it is stored). The Add goes into whichever of its two producers is a
    convolution that nothing else reads and comes last in evaluation order, so the other operand
    exists when that convolution runs."""
    changed = False
    order = {id(n): i for i, n in enumerate(graph.nodes)}
    for node in list(graph.nodes):
        if node.kind == "Add":
            a, b = node.input(0), node.input(1)
            if a.dims is None or a.dims != b.dims or a is b:
                continue
            cands = [v for v in (a, b) if v.node is not None and v.node.kind == "Conv" and graph.uses(v) == 1 and
                     "residual" not in v.node.attrs and not v.node.attrs.get("relu")]
            if not cands:
                continue
            y = max(cands, key=lambda v: order[id(v.node)])
            other = b if y is a else a
            if other.node is not None and order[id(other.node)] > order[id(y.node)]:
                continue
            y.node.attrs["residual"] = other
            graph.replace_all_uses(node.output(0), y)
            graph.erase(node)
            changed = True
        elif node.kind == "Relu":
            x = node.input(0)
            if x.node is None or x.node.kind != "Conv" or graph.uses(x) != 1 or x.node.attrs.get("relu"):
                continue
            x.node.attrs["relu"] = True
            graph.replace_all_uses(node.output(0), x)
            graph.erase(node)
            changed = True
    return changed


def optimize(graph):
    """The passes of the reference's optimizer that end in this library's fused convolution
    (dlf/src/model/optimize.cpp registers them by name), followed by the residual / ReLU fusion."""
    fuse_bn_into_conv(graph)
    fuse_add_bias_into_conv(graph)
    for n in [n for n in graph.nodes if n.kind in ("Identity", "Dropout") and len(n.outputs) == 1]:
        graph.replace_all_uses(n.output(0), n.input(0))
        graph.erase(n)
    fuse_residual_and_relu_into_conv(graph)
    return graph


_OPERATOR_KINDS = ("Conv", "Gemm", "MatMul", "MaxPool", "AveragePool", "GlobalAveragePool", "GlobalMaxPool",
                   "Flatten", "Reshape")


def unsupported_nodes(graph):
    """Nodes of an optimized graph that no operator of this library evaluates (an element-wise node
    that could not be folded into a convolution, for instance)."""
    return [n for n in graph.nodes if n.kind not in _OPERATOR_KINDS]


# ---------------------------------------------------------------------------------------------
# operators


class Operator:
    """One entry of the operator list (predict.h:118-122)."""
    launches = True

    def evaluate(self):
        raise NotImplementedError

    def scratch_bytes(self):
        return 0


class ConvOp(Operator):
    """dnn::conv2d + the bias pass (predict.h:1258-1286), with the residual Add and the Relu that
    follow it in the graph fused into the same launch."""

    def __init__(self, X, W, B, Y, filt, residual, relu):
        self.X, self.W, self.B, self.Y, self.filter, self.residual, self.relu = X, W, B, Y, filt, residual, relu

    def evaluate(self):
        gdnn.conv2d_filter(self.X, self.W, self.Y, self.filter, bias=self.B, residual=self.residual,
                           activation="relu" if self.relu else None)

    def scratch_bytes(self):
        f = self.filter
        return int(lib().dlf_b200_conv2d_workspace_bytes(
            int(gblas.precision_of(self.Y)), f.batches, f.channels, f.height, f.width, f.output_h, f.output_w,
            f.num_kernels, f.group, f.kernel_h, f.kernel_w))


class GemmOp(Operator):
    """predict.h:1203-1226: Y = alpha * op(A) * op(B) + beta * broadcast(C)."""

    def __init__(self, A, B, C, Y, alpha, beta, transA, transB):
        self.A, self.B, self.C, self.Y = A, B, C, Y
        self.alpha, self.beta = alpha, (beta if C is not None else 0)
        self.transA = Transpose.Trans if transA else Transpose.NoTrans
        self.transB = Transpose.Trans if transB else Transpose.NoTrans

    def evaluate(self):
        linalg.gemm(self.transA, self.transB, self.alpha, self.A, self.B, self.beta, self.C, self.Y)

    def scratch_bytes(self):
        m, n = self.Y.shape
        k = self.A.shape[0] if self.transA == Transpose.Trans else self.A.shape[1]
        return int(lib().dlf_b200_gemm_workspace_bytes(int(gblas.precision_of(self.Y)), m, n, k))


class MatMulOp(Operator):
    """predict.h:1228-1241."""

    def __init__(self, A, B, C):
        self.A, self.B, self.C = A, B, C

    def evaluate(self):
        linalg.matmul(self.A, self.B, self.C)

    def scratch_bytes(self):
        m = self.A.shape[-2] if self.A.dim() > 1 else 1
        n = self.B.shape[-1] if self.B.dim() > 1 else 1
        return int(lib().dlf_b200_gemm_workspace_bytes(int(gblas.precision_of(self.C)), m, n, self.A.shape[-1]))


class MaxPoolOp(Operator):
    """predict.h:1288-1311."""

    def __init__(self, X, Y, filt):
        self.X, self.Y, self.filter = X, Y, filt

    def evaluate(self):
        gdnn.max_pooling(self.X, self.Y, self.filter)


class AveragePoolOp(Operator):
    """predict.h:1313-1338."""

    def __init__(self, X, Y, filt, count_include_pad):
        self.X, self.Y, self.filter, self.count_include_pad = X, Y, filt, bool(count_include_pad)

    def evaluate(self):
        gdnn.average_pooling(self.X, self.Y, self.filter, self.count_include_pad)


class GlobalPoolOp(Operator):
    """predict.h:1340-1370."""

    def __init__(self, X, Y, average):
        self.X, self.Y, self.average = X, Y, average

    def evaluate(self):
        (gdnn.global_average_pooling if self.average else gdnn.global_max_pooling)(self.X, self.Y)


class NhwcConvOp(Operator):
    """A convolution between channels-last tensors: X (N, H, W, C), the filter bank packed once when
    the predictor is built, Y (and the residual) channels-last or NCHW. One launch, no scratch."""

    def __init__(self, X, Wp, B, Y, filt, residual, relu, y_layout):
        self.X, self.Wp, self.B, self.Y, self.filter = X, Wp, B, Y, filt
        self.residual, self.relu, self.y_layout = residual, relu, y_layout

    def evaluate(self):
        gdnn.conv2d_nhwc(self.X, self.Wp, self.Y, self.filter, bias=self.B, residual=self.residual,
                         activation="relu" if self.relu else None, y_layout=self.y_layout)


class NhwcPoolOp(Operator):
    """Max / average / global pooling between channels-last tensors."""

    def __init__(self, X, Y, filt, average, count_include_pad):
        self.X, self.Y, self.filter, self.average, self.count_include_pad = X, Y, filt, average, count_include_pad

    def evaluate(self):
        gdnn.pool_nhwc(self.X, self.Y, self.filter, average=self.average, count_include_pad=self.count_include_pad)


class ToNhwcOp(Operator):
    """The transposing copy that brings an NCHW value into the channels-last part of the list."""

    def __init__(self, X, Y):
        self.X, self.Y = X, Y

    def evaluate(self):
        gdnn.nchw_to_nhwc(self.X, self.Y)


class ViewOp(Operator):
    """Flatten / Reshape: the output shares the input's storage (the reference's ReshapeOp aliases
    its datum the same way), so there is nothing to launch."""
    launches = False

    def evaluate(self):
        pass


_TORCH_TYPES = {torch.float32: DataType.FLOAT, torch.float16: DataType.FLOAT16, torch.bfloat16: DataType.BFLOAT16}


class Predictor:
    """``Predictor<GPU, T>(graph)``: shape inference, the optimizer, then one operator per
    remaining node over device tensors allocated once (predict.h:2048-2062). ``set(i, data)`` fills
    graph input i (initializers are not inputs here: they are uploaded when the predictor is
    built), ``predict()`` evaluates the list in order (predict.h:2064-2070), ``get(i)`` reads graph
    output i back.

    ``dtype`` is T: every floating-point value of the graph is held in it. With ``cuda_graph``
    (the default) the second ``predict()`` captures the operator list into a CUDA graph and replays
    it from then on; the first one runs the launches one by one, which also loads the kernels.

    ``channels_last`` (16-bit T only): the predictor owns the tensors between its operators, so it
    keeps those that only convolutions and poolings read as (N, H, W, C) - the layout the tensor-map
    unit fetches filter windows from - and runs those operators through the channels-last entries:
    no transposing copy in front of a convolution, TMA-fed operands and TMA stores whatever the
    plane size. Graph inputs and outputs stay NCHW; a copy is inserted where an NCHW value enters the
    channels-last part."""

    def __init__(self, graph, dtype=torch.float32, device=None, cuda_graph=True, channels_last=True):
        if dtype not in _TORCH_TYPES:
            raise TypeError("Predictor: T must be float32, float16 or bfloat16")
        self.dtype = dtype
        infer_shapes(graph)
        optimize(graph)
        left = unsupported_nodes(graph)
        if left:
            raise NotImplementedError(
                "operator %s (output %s) is not folded into a convolution and is outside this library's path"
                % (left[0].kind, left[0].output(0).name))
        self.graph = graph
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._data = {}
        self._nhwc_copy = {}
        self._pre_ops = []
        self._nhwc = self._assign_layouts(graph) if channels_last and dtype != torch.float32 else set()
        self.operators = []
        for n in graph.nodes:
            op = self._create(n)
            self.operators.extend(self._pre_ops)
            self._pre_ops = []
            self.operators.append(op)
        self._inputs = [self._alloc(v) for v in graph.inputs if not v.has_initializer()]
        self._outputs = [self._alloc(v) for v in graph.outputs]
        need = max([op.scratch_bytes() for op in self.operators] + [0])
        self._scratch = torch.empty(max(need, 256), dtype=torch.uint8, device=self.device)
        self._want_graph = bool(cuda_graph)
        self._cuda_graph = None
        self._warm = False

    # -- layouts --------------------------------------------------------------------------

    _POOLS = ("MaxPool", "AveragePool")
    _GLOBAL_POOLS = ("GlobalAveragePool", "GlobalMaxPool")

    def _native(self, n):
        """A convolution the channels-last entry serves (weights known when the list is built)."""
        return (n.kind == "Conv" and n.input(1).has_initializer() and
                (n.input(2) is None or n.input(2).has_initializer()) and
                gdnn.nhwc_supported(_conv_filter(n, n.input(0).dims, n.input(1).dims), self.dtype, gdnn.NCHW))

    def _assign_layouts(self, graph):
        """ids of the values kept channels-last. Optimistic start: every output of a convolution the
        channels-last entry serves (a multiple of 8 output channels) and of a windowed pooling over
        such a value; then values are taken back until nothing contradicts: a graph output, a value
        read by an operator that needs NCHW, a residual whose convolution writes NCHW, a pooling
        whose input is NCHW."""
        native = {id(n): self._native(n) for n in graph.nodes if n.kind == "Conv"}
        cand = set()
        for n in graph.nodes:
            out = n.output(0)
            if out.dims is None or len(out.dims) != 4 or out.dims[1] % 8:
                continue
            if (n.kind == "Conv" and native[id(n)]) or n.kind in self._POOLS:
                cand.add(id(out))
        outputs = {id(v) for v in graph.outputs}
        changed = True
        while changed:
            changed = False
            for n in graph.nodes:
                out = n.output(0)
                if id(out) not in cand:
                    continue
                drop = id(out) in outputs or (n.kind in self._POOLS and id(n.input(0)) not in cand)
                for c in graph.nodes:
                    if drop:
                        break
                    reads = any(v is out for v in c.inputs)
                    as_residual = c.attrs.get("residual") is out
                    if not reads and not as_residual:
                        continue
                    if c.kind == "Conv":
                        drop = (c.input(0) is out and not native[id(c)]) or \
                               (as_residual and id(c.output(0)) not in cand) or \
                               any(v is out for v in c.inputs[1:])
                    elif c.kind in self._POOLS:
                        drop = id(c.output(0)) not in cand
                    elif c.kind in self._GLOBAL_POOLS:
                        drop = False
                    else:
                        drop = True
                if drop:
                    cand.discard(id(out))
                    changed = True
        return cand

    def _as_nhwc(self, value):
        """The channels-last tensor of a 4-D value: its own storage, or a copy made by an inserted
        operator (once per value)."""
        t = self._alloc(value)
        if id(value) in self._nhwc:
            return t
        c = self._nhwc_copy.get(id(value))
        if c is None:
            n, ch, h, w = value.dims
            c = torch.zeros((n, h, w, (ch + 7) // 8 * 8), dtype=self.dtype, device=self.device)
            self._nhwc_copy[id(value)] = c
            self._pre_ops.append(ToNhwcOp(t, c))
        return c

    # -- datums ---------------------------------------------------------------------------

    def _alloc(self, value, like=None):
        """The device tensor of a value (OperatorFactory::alloc, predict.h:300-330): initializers
        are uploaded once, everything else is allocated once and reused by every ``predict()``."""
        if value is None:
            return None
        t = self._data.get(id(value))
        if t is None:
            if value.dims is None:
                raise ShapeInferenceError("value %s has no shape" % value.name)
            if value.has_initializer():
                t = torch.from_numpy(np.ascontiguousarray(np.asarray(value.initializer, dtype=np.float64 if
                                     value.dtype == DataType.DOUBLE else np.float32))).to(self.dtype).to(self.device)
            elif like is not None:
                t = like.view(value.dims)
            elif id(value) in self._nhwc:
                n, ch, h, w = value.dims
                t = torch.zeros((n, h, w, ch), dtype=self.dtype, device=self.device)
            else:
                t = torch.zeros(value.dims, dtype=self.dtype, device=self.device)
            self._data[id(value)] = t
        return t

    # -- operators ------------------------------------------------------------------------

    def _create(self, n):
        k = n.kind
        if k == "Conv" and self._nhwc is not None and (id(n.output(0)) in self._nhwc or
                                                        (id(n.input(0)) in self._nhwc and self._native(n))):
            filt = _conv_filter(n, n.input(0).dims, n.input(1).dims)
            X = self._as_nhwc(n.input(0))
            Wp = gdnn.pack_filters_nhwc(self._alloc(n.input(1)))
            nhwc_out = id(n.output(0)) in self._nhwc
            res = n.get("residual")
            R = None if res is None else (self._as_nhwc(res) if nhwc_out else self._alloc(res))
            return NhwcConvOp(X, Wp, self._alloc(n.input(2)), self._alloc(n.output(0)), filt, R, bool(n.get("relu")),
                              gdnn.NHWC if nhwc_out else gdnn.NCHW)
        if k in self._POOLS and id(n.output(0)) in self._nhwc:
            return NhwcPoolOp(self._alloc(n.input(0)), self._alloc(n.output(0)), _pool_filter(n, n.input(0).dims),
                              k == "AveragePool", bool(n.get("count_include_pad", 0)))
        if k in self._GLOBAL_POOLS and id(n.input(0)) in self._nhwc:
            d = n.input(0).dims
            return NhwcPoolOp(self._alloc(n.input(0)), self._alloc(n.output(0)),
                              gdnn.Filter2D(d, d[2], d[3]).strides(d[2], d[3]), k == "GlobalAveragePool", False)
        if k == "Conv":
            X, W = self._alloc(n.input(0)), self._alloc(n.input(1))
            B = self._alloc(n.input(2))
            res = self._alloc(n.get("residual")) if n.get("residual") is not None else None
            Y = self._alloc(n.output(0))
            return ConvOp(X, W, B, Y, _conv_filter(n, n.input(0).dims, n.input(1).dims), res, bool(n.get("relu")))
        if k == "Gemm":
            A, B, C = self._alloc(n.input(0)), self._alloc(n.input(1)), self._alloc(n.input(2))
            return GemmOp(A, B, C, self._alloc(n.output(0)), n.get("alpha", 1.0), n.get("beta", 1.0),
                          n.get("transA", 0), n.get("transB", 0))
        if k == "MatMul":
            return MatMulOp(self._alloc(n.input(0)), self._alloc(n.input(1)), self._alloc(n.output(0)))
        if k == "MaxPool":
            return MaxPoolOp(self._alloc(n.input(0)), self._alloc(n.output(0)), _pool_filter(n, n.input(0).dims))
        if k == "AveragePool":
            return AveragePoolOp(self._alloc(n.input(0)), self._alloc(n.output(0)), _pool_filter(n, n.input(0).dims),
                                 n.get("count_include_pad", 0))
        if k in ("GlobalAveragePool", "GlobalMaxPool"):
            return GlobalPoolOp(self._alloc(n.input(0)), self._alloc(n.output(0)), k == "GlobalAveragePool")
        if k in ("Flatten", "Reshape"):
            self._alloc(n.output(0), like=self._alloc(n.input(0)))
            return ViewOp()
        raise NotImplementedError("operator %s" % k)

    # -- the reference's interface ---------------------------------------------------------

    def set(self, i, data):
        """predict.h:148-151."""
        dst = self._inputs[i]
        src = data if isinstance(data, torch.Tensor) else torch.from_numpy(np.ascontiguousarray(data))
        if tuple(src.shape) != tuple(dst.shape):
            raise ShapeInferenceError("input %d: shape %r expected, %r given" % (i, tuple(dst.shape), tuple(src.shape)))
        dst.copy_(src.to(self.dtype), non_blocking=True)

    def input(self, i):
        """The device tensor behind graph input i, for callers that fill it on the device."""
        return self._inputs[i]

    def output(self, i):
        """The device tensor behind graph output i (valid after ``predict()`` in stream order)."""
        return self._outputs[i]

    def get(self, i):
        """predict.h:153-156: graph output i as a host array."""
        t = self._outputs[i]
        return (t.float() if t.dtype != torch.float32 else t).cpu().numpy()

    def _evaluate(self):
        with gblas.scratch(self._scratch):
            for op in self.operators:
                op.evaluate()

    def launches_per_predict(self):
        """Operators that launch work (shape-only ones do not)."""
        return sum(1 for op in self.operators if op.launches)

    def predict(self):
        """Evaluates the operator list in order on the current stream (predict.h:2064-2070)."""
        if self._cuda_graph is not None:
            self._cuda_graph.replay()
            return
        if self._want_graph and self._warm:
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self._evaluate()
            except RuntimeError:
                # an operator that cannot be captured (a MatMul that uploads offset tables from the
                # host): the list keeps running launch by launch
                self._want_graph = False
                torch.cuda.synchronize(self.device)
            else:
                self._cuda_graph = g
                g.replay()
                return
        self._evaluate()
        self._warm = True
