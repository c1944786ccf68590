"""The operator-list runtime (dlf_b200.predict): graph passes and shape inference on the CPU, and on
the GPU the reference's PredictTest vectors (dlf/test/model/PredictTest.cpp:74-117) plus a small
residual network evaluated node by node with the CPU oracle. Tolerances as in the parity suite:
fp32 <= 1e-5 relative Frobenius error per operator (1e-4 for the chained network); for the chained
network in 16 bits 4e-3 (fp16) and 3e-2 (bf16) relative Frobenius error."""
import numpy as np
import pytest
import torch

import oracle
from support import load_goldens, rel_fro, tensor_of

from dlf_b200 import predict as P

G = load_goldens()


def _conv(g, x, name, cout, k, stride, pad, rng, bias=False, bn=True, cin=None):
    cin = cin if cin is not None else x.dims[1]
    n = g.append("Conv", pads=[pad] * 4, strides=[stride, stride], kernel_shape=[k, k])
    n.addInput(x).addInput(g.addInitializer(name + ".W", (np.sqrt(2.0 / (cin * k * k)) *
                                            rng.normal(size=(cout, cin, k, k))).astype(np.float32)))
    if bias:
        n.addInput(g.addInitializer(name + ".B", rng.uniform(-0.1, 0.1, cout).astype(np.float32)))
    y = n.addOutput(name)
    if bn:
        b = g.append("BatchNormalization", epsilon=1e-5)
        b.addInput(y)
        b.addInput(g.addInitializer(name + ".scale", rng.uniform(0.5, 1.5, cout).astype(np.float32)))
        b.addInput(g.addInitializer(name + ".beta", rng.uniform(-0.2, 0.2, cout).astype(np.float32)))
        b.addInput(g.addInitializer(name + ".mean", rng.uniform(-0.2, 0.2, cout).astype(np.float32)))
        b.addInput(g.addInitializer(name + ".var", rng.uniform(0.5, 1.5, cout).astype(np.float32)))
        y = b.addOutput(name + ".bn")
    return y


def _relu(g, x, name):
    n = g.append("Relu")
    n.addInput(x)
    return n.addOutput(name)


def small_resnet(batch, size, rng, classes=10):
    """Stem 7x7 stride 2 + BN + ReLU, 3x3 max pool stride 2, a bottleneck block with a projection
    shortcut (listed after the main path, as exporters do), an identity block, global average
    pool, Flatten, Gemm: every operator kind a ResNet forward uses."""
    g = P.Graph()
    x = g.addInput("image", P.DataType.FLOAT, (batch, 3, size, size))
    t = _relu(g, _conv(g, x, "stem", 16, 7, 2, 3, rng, cin=3), "stem.relu")
    mp = g.append("MaxPool", kernel_shape=[3, 3], strides=[2, 2], pads=[1, 1, 1, 1])
    mp.addInput(t)
    t = mp.addOutput("pool")
    # block 1: projection shortcut
    a = _relu(g, _conv(g, t, "b1.c1", 8, 1, 1, 0, rng, cin=16), "b1.r1")
    a = _relu(g, _conv(g, a, "b1.c2", 8, 3, 1, 1, rng, cin=8), "b1.r2")
    a = _conv(g, a, "b1.c3", 32, 1, 1, 0, rng, cin=8)
    sc = _conv(g, t, "b1.down", 32, 1, 1, 0, rng, cin=16)
    add = g.append("Add")
    add.addInput(a).addInput(sc)
    t = _relu(g, add.addOutput("b1.add"), "b1.out")
    # block 2: identity shortcut, stride-2 3x3 inside, bias instead of BN on the last convolution
    a = _relu(g, _conv(g, t, "b2.c1", 8, 1, 1, 0, rng, cin=32), "b2.r1")
    a = _relu(g, _conv(g, a, "b2.c2", 8, 3, 1, 1, rng, cin=8), "b2.r2")
    a = _conv(g, a, "b2.c3", 32, 1, 1, 0, rng, bias=True, bn=False, cin=8)
    add = g.append("Add")
    add.addInput(t).addInput(a)
    t = _relu(g, add.addOutput("b2.add"), "b2.out")
    gap = g.append("GlobalAveragePool")
    gap.addInput(t)
    fl = g.append("Flatten", axis=1)
    fl.addInput(gap.addOutput("gap"))
    fc = g.append("Gemm", transB=1)
    fc.addInput(fl.addOutput("flat"))
    fc.addInput(g.addInitializer("fc.W", (rng.normal(size=(classes, 32)) / np.sqrt(32)).astype(np.float32)))
    fc.addInput(g.addInitializer("fc.B", rng.uniform(-0.1, 0.1, classes).astype(np.float32)))
    g.addOutput(fc.addOutput("logits"))
    g.addOutput(t)
    return g


def oracle_evaluate(graph, feeds, rnd=lambda a: a):
    """The unoptimized graph node by node on the CPU, the way the reference's Predictor<CPU> runs
    it: one pass per node, every result rounded to the storage type by ``rnd``."""
    env = {}
    for v in graph.inputs:
        env[id(v)] = rnd(np.asarray(v.initializer, dtype=np.float32)) if v.has_initializer() and \
            v.dtype != P.DataType.INT64 else None
    it = iter(feeds)
    for v in graph.inputs:
        if not v.has_initializer():
            env[id(v)] = rnd(np.asarray(next(it), dtype=np.float32))
    for n in graph.nodes:
        a = [env[id(v)] if v is not None else None for v in n.inputs]
        k = n.kind
        if k == "Conv":
            s = n.get("strides", [1, 1])
            y = oracle.conv2d(a[0], a[1], group=n.get("group", 1), pads=tuple(n.get("pads", (0,) * 4)),
                              strides=tuple(s), bias=a[2] if len(a) > 2 else None, wide=True)
        elif k == "BatchNormalization":
            sh = (1, -1, 1, 1)
            y = ((a[0] - a[3].reshape(sh)) / np.sqrt(a[4].reshape(sh) + np.float32(n.get("epsilon", 1e-5))) *
                 a[1].reshape(sh) + a[2].reshape(sh)).astype(np.float32)
        elif k == "Relu":
            y = np.maximum(a[0], np.float32(0))
        elif k == "Add":
            y = (a[0] + a[1]).astype(np.float32)
        elif k == "MaxPool":
            y = oracle.pool2d(a[0], tuple(n.get("kernel_shape")), "max", tuple(n.get("pads", (0,) * 4)),
                              tuple(n.get("strides", (1, 1))))
        elif k == "GlobalAveragePool":
            y = oracle.global_pool(a[0], "avg", wide=True)
        elif k == "Flatten":
            y = a[0].reshape(a[0].shape[0], -1)
        elif k == "Gemm":
            A = a[0].T if n.get("transA", 0) else a[0]
            B = a[1].T if n.get("transB", 0) else a[1]
            y = (n.get("alpha", 1.0) * (A.astype(np.float64) @ B.astype(np.float64)) +
                 n.get("beta", 1.0) * a[2].astype(np.float64)).astype(np.float32)
        else:
            raise AssertionError(k)
        env[id(n.output(0))] = rnd(y)
    return [env[id(v)] for v in graph.outputs]


# ---------------------------------------------------------------------------------------------
# CPU: the graph passes


def test_passes_fold_a_residual_network_into_fused_convolutions():
    g = small_resnet(2, 32, np.random.default_rng(0))
    P.infer_shapes(g)
    assert g.outputs[0].dims == (2, 10) and g.outputs[1].dims == (2, 32, 8, 8)
    P.optimize(g)
    kinds = [n.kind for n in g.nodes]
    assert kinds == ["Conv", "MaxPool"] + ["Conv"] * 7 + ["GlobalAveragePool", "Flatten", "Gemm"]
    assert not P.unsupported_nodes(g)
    by_name = {n.output(0).name: n for n in g.nodes}
    # BatchNormalization left a bias behind on every convolution it followed
    assert all(len(n.inputs) == 3 for n in g.nodes if n.kind == "Conv")
    # the Add went into the producer that comes last: the projection shortcut, then block 2's c3
    assert by_name["b1.down"].get("residual") is by_name["b1.c3"].output(0) and by_name["b1.down"].get("relu")
    assert by_name["b1.c3"].get("residual") is None and not by_name["b1.c3"].get("relu")
    assert by_name["b2.c3"].get("residual") is by_name["b1.down"].output(0) and by_name["b2.c3"].get("relu")
    assert by_name["stem"].get("relu") and by_name["b2.c2"].get("relu")
    assert g.outputs[1] is by_name["b2.c3"].output(0)


def test_bn_folding_matches_the_formula():
    rng = np.random.default_rng(3)
    g = P.Graph()
    x = g.addInput("x", P.DataType.FLOAT, (1, 4, 6, 6))
    y = _conv(g, x, "c", 5, 3, 1, 1, rng, bias=True, bn=True, cin=4)
    g.addOutput(y)
    init = {v.name: np.array(v.initializer, dtype=np.float64) for v in g.inputs if v.has_initializer()}
    P.infer_shapes(g)
    assert P.fuse_bn_into_conv(g)
    conv = g.nodes[0]
    assert [n.kind for n in g.nodes] == ["Conv"] and g.outputs[0] is conv.output(0)
    s = init["c.scale"] / np.sqrt(init["c.var"] + 1e-5)
    np.testing.assert_allclose(conv.input(1).initializer, init["c.W"] * s.reshape(-1, 1, 1, 1), rtol=1e-6)
    np.testing.assert_allclose(conv.input(2).initializer, (init["c.B"] - init["c.mean"]) * s + init["c.beta"], rtol=1e-6)
    assert sorted(v.name for v in g.inputs) == ["c.B", "c.W", "x"]


def test_add_of_a_channel_initializer_becomes_the_bias():
    rng = np.random.default_rng(4)
    for shape in ((1, 5, 1, 1), (5, 1, 1)):
        g = P.Graph()
        x = g.addInput("x", P.DataType.FLOAT, (2, 4, 6, 6))
        y = _conv(g, x, "c", 5, 3, 1, 1, rng, bn=False, cin=4)
        add = g.append("Add")
        b = rng.normal(size=shape).astype(np.float32)
        add.addInput(y).addInput(g.addInitializer("b", b))
        g.addOutput(add.addOutput("out"))
        P.infer_shapes(g)
        assert P.fuse_add_bias_into_conv(g)
        assert [n.kind for n in g.nodes] == ["Conv"]
        np.testing.assert_array_equal(g.nodes[0].input(2).initializer, b.reshape(-1))
    # a bias of another shape stays an Add, which no operator of the library evaluates
    g = P.Graph()
    x = g.addInput("x", P.DataType.FLOAT, (2, 4, 6, 6))
    y = _conv(g, x, "c", 5, 3, 1, 1, rng, bn=False, cin=4)
    add = g.append("Add")
    add.addInput(y).addInput(g.addInitializer("b", np.ones((6, 6), np.float32)))
    g.addOutput(add.addOutput("out"))
    P.optimize(P.infer_shapes(g))
    assert [n.kind for n in P.unsupported_nodes(g)] == ["Add"]


def test_shape_inference_rules_and_refusals():
    g = P.Graph()
    x = g.addInput("x", P.DataType.FLOAT, (2, 3, 9, 11))
    mp = g.append("MaxPool", kernel_shape=[3, 2], strides=[2, 1], pads=[1, 0, 1, 1])
    mp.addInput(x)
    y = mp.addOutput("p")
    rs = g.append("Reshape")
    rs.addInput(y).addInput(g.addInitializer("shape", np.array([0, -1, 11], dtype=np.int64)))
    z = rs.addOutput("r")
    mm = g.append("MatMul")
    mm.addInput(z).addInput(g.addInitializer("w", np.ones((11, 7), np.float32)))
    g.addOutput(mm.addOutput("m"))
    P.infer_shapes(g)
    assert y.dims == (2, 3, 5, 11) and z.dims == (2, 15, 11) and g.outputs[0].dims == (2, 15, 7)
    bad = P.Graph()
    s = bad.append("Softmax")
    s.addInput(bad.addInput("x", P.DataType.FLOAT, (2, 3)))
    bad.addOutput(s.addOutput("y"))
    with pytest.raises(P.ShapeInferenceError):
        P.infer_shapes(bad)
    bad = P.Graph()
    c = bad.append("Conv")
    c.addInput(bad.addInput("x", P.DataType.FLOAT, (2, 3, 8, 8))).addInput(
        bad.addInitializer("w", np.ones((4, 2, 3, 3), np.float32)))
    bad.addOutput(c.addOutput("y"))
    with pytest.raises(P.ShapeInferenceError):
        P.infer_shapes(bad)


def _layout_names(graph, dtype=torch.float16):
    """Names of the values a predictor of ``dtype`` would keep channels-last (no device needed: the
    assignment only looks at the graph)."""
    P.infer_shapes(graph)
    P.optimize(graph)
    pred = object.__new__(P.Predictor)
    pred.dtype = dtype
    ids = pred._assign_layouts(graph)
    names = {}
    for n in graph.nodes:
        names[id(n.output(0))] = n.output(0).name
    return {names[i] for i in ids}


def test_channels_last_assignment_follows_the_readers():
    # every operator of the residual network after the stem's pool reads and writes channels-last,
    # except what ends in the NCHW graph output: the last block's residual chain
    got = _layout_names(small_resnet(2, 32, np.random.default_rng(0)))
    assert got == {"b1.c1", "b1.c2", "b2.c1", "b2.c2"}
    # with only the logits as output, the whole trunk is channels-last; the 3-channel stem is not
    # (its input has 3 channels) and neither is its pool (a pooling follows its input's layout)
    g = small_resnet(2, 32, np.random.default_rng(0))
    g.outputs = g.outputs[:1]
    got = _layout_names(g)
    assert got == {"b1.c1", "b1.c2", "b1.c3", "b1.down", "b2.c1", "b2.c2", "b2.c3"}
    # fp32 predictors never use the channels-last entries: decided before the assignment runs
    rng = np.random.default_rng(1)
    g = P.Graph()
    x = g.addInput("x", P.DataType.FLOAT, (1, 16, 8, 8))
    a = _conv(g, x, "a", 16, 3, 1, 1, rng, bn=False, cin=16)          # channels-last: read by b and by the pool
    b = _conv(g, a, "b", 12, 1, 1, 0, rng, bn=False, cin=16)          # 12 output channels: not a multiple of 8 -> NCHW
    mp = g.append("MaxPool", kernel_shape=[2, 2], strides=[2, 2])
    mp.addInput(a)
    c = _conv(g, mp.addOutput("p"), "c", 8, 1, 1, 0, rng, bn=False, cin=16)
    g.addOutput(b)
    g.addOutput(c)
    assert _layout_names(g) == {"a", "p"}
    # a value that a non-native convolution reads (grouped) must stay NCHW, and so must what feeds its pool
    g = P.Graph()
    x = g.addInput("x", P.DataType.FLOAT, (1, 16, 8, 8))
    a = _conv(g, x, "a", 16, 3, 1, 1, rng, bn=False, cin=16)
    n = g.append("Conv", group=2, kernel_shape=[1, 1])
    n.addInput(a).addInput(g.addInitializer("gw", np.ones((8, 8, 1, 1), np.float32)))
    g.addOutput(n.addOutput("grouped"))
    assert _layout_names(g) == set()


def test_a_relu_that_follows_no_convolution_is_refused():
    g = P.Graph()
    x = g.addInput("x", P.DataType.FLOAT, (1, 2, 4, 4))
    mp = g.append("MaxPool", kernel_shape=[2, 2], strides=[2, 2])
    mp.addInput(x)
    g.addOutput(_relu(g, mp.addOutput("p"), "r"))
    with pytest.raises(NotImplementedError):
        P.Predictor(g)


# ---------------------------------------------------------------------------------------------
# GPU


@pytest.fixture
def device_lib():
    import dlf_b200
    yield dlf_b200
    assert dlf_b200.device_status() == 0, "a device-side bounded wait timed out"


@pytest.mark.gpu
def test_predict_gemm_vector_through_the_predictor(device_lib):
    """PredictTest.Gemm (dlf/test/model/PredictTest.cpp:74-90), bit for bit."""
    p = G["predict"]["gemm"]
    g = P.Graph()
    n = g.append("Gemm", alpha=1.0, beta=1.0)
    for nm in "ABC":
        n.addInput(g.addInput(nm, P.DataType.FLOAT, p[nm]["shape"]))
    g.addOutput(n.addOutput("Y"))
    pred = P.Predictor(g)
    for i, nm in enumerate("ABC"):
        pred.set(i, tensor_of(p[nm]).numpy())
    for _ in range(3):  # launch by launch, captured, replayed
        pred.predict()
        np.testing.assert_array_equal(pred.get(0), tensor_of(p["Y"]).numpy())


@pytest.mark.gpu
def test_predict_conv_vector_through_the_predictor(device_lib):
    """PredictTest.Conv (PredictTest.cpp:92-117): bias as an initializer, X and W as inputs."""
    p = G["predict"]["conv"]
    g = P.Graph()
    n = g.append("Conv", pads=p["pads"])
    n.addInput(g.addInput("X", P.DataType.FLOAT, p["X"]["shape"]))
    n.addInput(g.addInput("W", P.DataType.FLOAT, p["W"]["shape"]))
    n.addInput(g.addInitializer("B", tensor_of(p["bias"]).numpy()))
    g.addOutput(n.addOutput("Y"))
    pred = P.Predictor(g)
    pred.set(0, tensor_of(p["X"]).numpy())
    pred.set(1, tensor_of(p["W"]).numpy())
    for _ in range(3):
        pred.predict()
        np.testing.assert_array_equal(pred.get(0), tensor_of(p["Y"]).numpy())


def _round_fn(dtype):
    if dtype == torch.float32:
        return lambda a: a
    return lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dtype).float().numpy()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,channels_last", [(torch.float32, False), (torch.float16, False), (torch.float16, True),
                                                 (torch.bfloat16, False), (torch.bfloat16, True)],
                         ids=["f32", "f16-nchw", "f16-channels-last", "bf16-nchw", "bf16-channels-last"])
def test_small_residual_network_against_the_oracle(device_lib, dtype, channels_last):
    """Every predict() - the first launch by launch, the second captured into a CUDA graph, the
    later ones replays - on fresh inputs against the unoptimized graph evaluated node by node on
    the CPU. Eleven operators launch work (Flatten does not)."""
    rng = np.random.default_rng(11)
    reference_graph = small_resnet(3, 40, np.random.default_rng(5))
    pred = P.Predictor(small_resnet(3, 40, np.random.default_rng(5)), dtype=dtype, channels_last=channels_last)
    kinds = [type(op).__name__ for op in pred.operators]
    if channels_last:
        # the stem (3 channels) and its pool stay NCHW, one copy brings the pool's output into the
        # channels-last part, the last block writes NCHW again (its output is a graph output)
        assert kinds.count("ToNhwcOp") >= 1 and kinds.count("NhwcConvOp") >= 4 and kinds.count("NhwcPoolOp") == 0
    else:
        assert pred.launches_per_predict() == 11 and "NhwcConvOp" not in kinds
    rnd = _round_fn(dtype)
    deltas = []
    for step in range(4):
        x = rng.normal(size=(3, 3, 40, 40)).astype(np.float32)
        want = oracle_evaluate(reference_graph, [x], rnd)
        before = device_lib.launch_count()
        pred.set(0, x)
        pred.predict()
        got = [pred.get(0), pred.get(1)]
        deltas.append(device_lib.launch_count() - before)
        for a, b in zip(got, want):
            if dtype == torch.float32:
                assert rel_fro(a, b) <= 1e-4
            else:
                # 16-bit: every operator's output is rounded to the storage type on both sides, but
                # at different places (the device rounds once per fused launch, the oracle after
                # every node; the folded weights are rounded products). Nine layers of rounding
                # noise of 2^-11 (2^-8) per element: a few units of that in the Frobenius norm.
                assert rel_fro(a, b) <= (4e-3 if dtype == torch.float16 else 3e-2)
    # kernel launches of the library: at least one per operator launch by launch, the same number
    # again while the list is captured, none when the graph is replayed
    assert deltas[0] >= pred.launches_per_predict() and deltas[1] == deltas[0] and deltas[2] == 0 and deltas[3] == 0


@pytest.mark.gpu
def test_graph_replay_equals_launch_by_launch(device_lib):
    """The same input through a predictor that replays a CUDA graph and through one that does not:
    identical bits, and the replay makes no call into the library (its launch counter stands)."""
    x = np.random.default_rng(2).normal(size=(2, 3, 32, 32)).astype(np.float32)
    outs = []
    for use_graph in (True, False):
        pred = P.Predictor(small_resnet(2, 32, np.random.default_rng(9)), dtype=torch.float16, cuda_graph=use_graph)
        pred.set(0, x)
        before = device_lib.launch_count()
        pred.predict()
        first = device_lib.launch_count() - before
        pred.predict()
        pred.predict()
        before = device_lib.launch_count()
        pred.predict()
        torch.cuda.synchronize()
        assert device_lib.launch_count() - before == (0 if use_graph else first)
        outs.append(pred.output(0).clone())
    assert torch.equal(outs[0], outs[1])


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,channels_last", [(torch.float32, False), (torch.float16, False), (torch.float16, True)],
                         ids=["f32", "f16-nchw", "f16-channels-last"])
def test_resnet50_operator_list_against_the_oracle(device_lib, dtype, channels_last):
    """All 53 convolutions of ResNet-50 v1 chained with their residual connections, the pools and
    the FC layer, at 64x64 so that the CPU evaluation takes seconds: launch by launch, captured
    and replayed, against the unoptimized graph on the CPU."""
    from bench import resnet50_graph
    pred = P.Predictor(resnet50_graph(2, size=64, classes=100, seed=3), dtype=dtype, channels_last=channels_last)
    kinds = [type(op).__name__ for op in pred.operators]
    if channels_last:
        # everything after the stem's pool is channels-last: 52 convolutions and the global pool, one copy
        assert kinds.count("NhwcConvOp") == 52 and kinds.count("ToNhwcOp") == 1 and kinds.count("NhwcPoolOp") == 1
    else:
        assert pred.launches_per_predict() == 56
    reference_graph = resnet50_graph(2, size=64, classes=100, seed=3)
    rnd = _round_fn(dtype)
    rng = np.random.default_rng(8)
    for step in range(3):
        x = rng.normal(size=(2, 3, 64, 64)).astype(np.float32)
        want = oracle_evaluate(reference_graph, [x], rnd)[0]
        pred.set(0, x)
        pred.predict()
        # 16-bit: 50 layers of rounding noise on both sides, at different places
        assert rel_fro(pred.get(0), want) <= (1e-4 if dtype == torch.float32 else 1e-2)
