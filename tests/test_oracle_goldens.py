"""CPU suite, part 1: the oracle reproduces every golden vector the reference's unit tests hold
for the gemm / matmul / conv2d path (bit-exact: all goldens are small integers)."""
import numpy as np
import pytest
import torch

import oracle
from dlf_b200 import tensor as dt
from dlf_b200.gblas import Transpose
from support import OracleBlas, UNSUPPORTED_EXPR, evaluate, load_goldens, tensor_of

G = load_goldens()
T, N = oracle.TRANS, oracle.NO_TRANS


@pytest.mark.parametrize("case", G["gemm"], ids=lambda c: c["source"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64, np.int32, np.int64])
def test_gemm_golden_generic_path(case, dtype):
    """gemm_serial ordering (int types in the reference) for all four transpose combinations."""
    A, At, B, Bt, C, R = (np.array(tensor_of(case[k], torch.float64).numpy(), dtype=dtype).ravel()
                          for k in ("A", "A_t", "B", "B_t", "C", "R"))
    for ta, tb, a, lda, b, ldb in ((N, N, A, 6, B, 4), (T, N, At, 3, B, 4), (N, T, A, 6, Bt, 6),
                                   (T, T, At, 3, Bt, 6)):
        c = C.copy()
        oracle.gemm_generic(ta, tb, 3, 4, 6, case["alpha"], a, lda, b, ldb, case["beta"], c, 4)
        assert c.tolist() == R.tolist()


@pytest.mark.parametrize("case", G["gemm"], ids=lambda c: c["source"])
@pytest.mark.parametrize("layout", [oracle.ROW_MAJOR, oracle.COL_MAJOR])
def test_gemm_golden_blas_path(case, layout):
    """cblas_sgemm semantics, row- and column-major, with element offsets."""
    A, At, B, Bt, C, R = (tensor_of(case[k]).numpy() for k in ("A", "A_t", "B", "B_t", "C", "R"))
    row = layout == oracle.ROW_MAJOR
    for ta, tb, a, b in ((N, N, A, B), (T, N, At, B), (N, T, A, Bt), (T, T, At, Bt)):
        # a column-major caller stores the transposed arrays
        sa, sb, sc = (a, b, C) if row else (a.T, b.T, C.T)
        fa = np.concatenate([np.zeros(5, np.float32), np.ascontiguousarray(sa).ravel()])
        fb = np.concatenate([np.zeros(7, np.float32), np.ascontiguousarray(sb).ravel()])
        fc = np.concatenate([np.zeros(3, np.float32), np.ascontiguousarray(sc).ravel()])
        oracle.gblas_sgemm(layout, ta, tb, 3, 4, 6, 2.0, fa, 5, sa.shape[1], fb, 7, sb.shape[1],
                           3.0, fc, 3, sc.shape[1])
        got = fc[3:].reshape(sc.shape)
        got = got if row else got.T
        assert np.array_equal(got, R)


def _supported(case):
    text = " ".join(c["a"] + c["b"] for c in case["checks"]) + \
        " ".join(v.get("expr", "") for v in case["vars"].values())
    return not any(u in text for u in UNSUPPORTED_EXPR)


@pytest.mark.parametrize("case", G["matmul"], ids=lambda c: c["name"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.int32])
def test_matmul_goldens_through_front_end(case, dtype):
    """dlf::matmul routing (broadcast, transposes from strides, reorder, strided vs offset-table
    batching) driven on CPU tensors with the oracle as the BLAS: results equal the literals."""
    if not _supported(case):
        pytest.skip("expression form not modelled: " + str(case["checks"]))
    env = dict(case["vars"])
    env["__dtype__"] = dtype
    for chk in case["checks"]:
        A, B = evaluate(chk["a"], env), evaluate(chk["b"], env)
        expect = evaluate(chk["expect"], env)
        be = OracleBlas()
        got = dt.matmul(A, B, backend=be)
        assert list(got.shape) == list(expect.shape)
        assert torch.equal(got, expect), (case["name"], chk)


@pytest.mark.parametrize("case", G["dot"], ids=lambda c: c["name"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.int32])
def test_dot_goldens_through_front_end(case, dtype):
    """dlf::dot / multi_dot known answers (TensorTest.Dot, UniformTest.Dot / MultiDot*, the
    GPGPUTest vector / matrix dots) on CPU tensors with the oracle as the BLAS."""
    args = [tensor_of(a, dtype) for a in case["args"]]
    expect = tensor_of(case["expected"], dtype)
    be = OracleBlas()
    got = dt.dot(args[0], args[1], backend=be) if len(args) == 2 else dt.multi_dot(*args, backend=be)
    assert list(got.shape) == list(expect.shape)
    assert torch.equal(got, expect), case["name"]


def test_multi_dot_picks_the_cheapest_order():
    """(10x2)(2x10)(10x2): multiplying the last two first costs 80 multiplications instead of
    400; the split table must say so (detail::matrix_chain_order, linalg_detail.h:1701-1720)."""
    assert dt._matrix_chain_order([10, 2, 10, 2])[0][2] == 0
    assert dt._matrix_chain_order([2, 10, 2, 10])[0][2] == 1
    with pytest.raises(dt.ShapeError):
        dt.multi_dot(torch.zeros(2, 3), torch.zeros(4, 5))
    with pytest.raises(dt.ShapeError):
        dt.multi_dot(torch.zeros(2, 3), torch.zeros(3), torch.zeros(3, 4))


def test_matmul_routing_choices():
    """The three branches of detail::matmul (linalg_detail.h:1573-1662)."""
    A = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)
    B = torch.arange(40, dtype=torch.float32).reshape(2, 4, 5)
    tr = []
    dt.matmul(A[0], B[0], backend=OracleBlas(), trace=tr)
    dt.matmul(A, B, backend=OracleBlas(), trace=tr)
    dt.matmul(A, B[0], backend=OracleBlas(), trace=tr)  # broadcast B: batch stride 0
    X = torch.arange(2 * 2 * 3 * 4, dtype=torch.float32).reshape(2, 2, 3, 4)
    Y = torch.arange(2 * 2 * 4 * 5, dtype=torch.float32).reshape(2, 2, 4, 5)
    dt.matmul(X.transpose(0, 1), Y, backend=OracleBlas(), trace=tr)  # prefix not collapsible
    assert tr == ["gemm", "gemmStridedBatched", "gemmStridedBatched", "gemmBatched"]
    ref = torch.matmul(X.transpose(0, 1), Y)
    assert torch.equal(dt.matmul(X.transpose(0, 1), Y, backend=OracleBlas()), ref)


def test_gemm_front_end_golden():
    case = G["gemm"][0]
    A, At, B, Bt, C, R = (tensor_of(case[k]) for k in ("A", "A_t", "B", "B_t", "C", "R"))
    NT, TR = Transpose.NoTrans, Transpose.Trans
    for ta, tb, a, b in ((NT, NT, A, B), (TR, NT, At, B), (NT, TR, A, Bt), (TR, TR, At, Bt)):
        got = dt.gemm(ta, tb, 2.0, a, b, 3.0, C, backend=OracleBlas())
        assert torch.equal(got, R)
    # PredictTest.Gemm: C {2} broadcast over rows, alpha = beta = 1
    p = G["predict"]["gemm"]
    got = dt.gemm(NT, NT, 1.0, tensor_of(p["A"]), tensor_of(p["B"]), 1.0, tensor_of(p["C"]),
                  backend=OracleBlas())
    assert torch.equal(got, tensor_of(p["Y"]))


@pytest.mark.parametrize("case", G["conv2d"], ids=lambda c: c["name"])
def test_conv2d_goldens(case):
    X, W = tensor_of(case["X"]).numpy(), tensor_of(case["W"]).numpy()
    f = case["filter"]
    Y = oracle.conv2d(X, W, group=f["group"], pads=tuple(f["pads"]), strides=tuple(f["strides"]))
    if "R" in case:
        assert np.array_equal(Y, tensor_of(case["R"]).numpy())
    # independent check of every case (also the four without literals) against torch's conv
    import torch.nn.functional as F
    pt, pl, pb, pr = f["pads"]
    ref = F.conv2d(F.pad(torch.from_numpy(X).double(), (pl, pr, pt, pb)),
                   torch.from_numpy(W).double(), stride=tuple(f["strides"]), groups=f["group"])
    assert np.array_equal(Y.astype(np.float64), ref.numpy())


def test_predict_conv_with_bias_golden():
    p = G["predict"]["conv"]
    Y = oracle.conv2d(tensor_of(p["X"]).numpy(), tensor_of(p["W"]).numpy(), pads=tuple(p["pads"]),
                      bias=tensor_of(p["bias"]).numpy())
    assert np.array_equal(Y, tensor_of(p["Y"]).numpy())


def test_oracle_sgemm_matches_float64_on_random_inputs():
    rng = np.random.default_rng(0)
    for (m, n, k) in ((37, 53, 129), (128, 64, 300)):
        A = rng.uniform(-1, 1, (m, k)).astype(np.float32)
        B = rng.uniform(-1, 1, (k, n)).astype(np.float32)
        C = rng.normal(size=(m, n)).astype(np.float32)
        ref = 0.5 * A.astype(np.float64) @ B.astype(np.float64) + 0.5 * C
        for wide in (False, True):
            c = C.copy().ravel()
            oracle.gblas_sgemm(oracle.ROW_MAJOR, N, N, m, n, k, 0.5, A.ravel(), 0, k, B.ravel(), 0,
                               n, 0.5, c, 0, n, wide=wide)
            assert np.linalg.norm(c.reshape(m, n) - ref) / np.linalg.norm(ref) < 1e-6
        # transposed storage gives the same numbers
        c = C.copy().ravel()
        oracle.gblas_sgemm(oracle.ROW_MAJOR, T, T, m, n, k, 0.5, np.ascontiguousarray(A.T).ravel(),
                           0, m, np.ascontiguousarray(B.T).ravel(), 0, k, 0.5, c, 0, n)
        assert np.linalg.norm(c.reshape(m, n) - ref) / np.linalg.norm(ref) < 1e-6


def test_host_cblas_agrees_with_oracle():
    fn, desc = oracle.find_host_cblas()
    if fn is None:
        pytest.skip(desc)
    rng = np.random.default_rng(1)
    A = rng.uniform(-1, 1, (64, 96)).astype(np.float32)
    B = rng.uniform(-1, 1, (96, 48)).astype(np.float32)
    c1 = np.zeros(64 * 48, np.float32)
    c2 = np.zeros(64 * 48, np.float32)
    oracle.host_sgemm(fn, oracle.ROW_MAJOR, N, N, 64, 48, 96, 1.0, A, 96, B, 48, 0.0, c1, 48)
    oracle.gblas_sgemm(oracle.ROW_MAJOR, N, N, 64, 48, 96, 1.0, A.ravel(), 0, 96, B.ravel(), 0, 48,
                       0.0, c2, 0, 48)
    assert np.linalg.norm(c1 - c2) / np.linalg.norm(c2) < 1e-6


def _pool_filter(X_shape, cfg):
    from dlf_b200 import gdnn
    f = gdnn.Filter2D(X_shape, cfg["kernel"][0], cfg["kernel"][1])
    for name, arg in cfg["calls"]:
        getattr(f, name)(*arg) if isinstance(arg, list) else getattr(f, name)(arg)
    return f


@pytest.mark.parametrize("case", G["pool"]["maxpool"], ids=lambda c: c["name"])
def test_maxpool_goldens(case):
    """TEST(MaxPool, *) of the reference (dlf/test/DNNTest.cpp:625-731), including the
    SAME_UPPER auto-padding of Filter2D (dlf/src/tensor/filter.cpp:51-82)."""
    X = tensor_of(case["X"]).numpy()
    f = _pool_filter(X.shape, case["filter"])
    Y = oracle.pool2d(X, (f.kernel_h, f.kernel_w), "max", (f.pad_top, f.pad_left, f.pad_bottom, f.pad_right),
                      (f.stride_h, f.stride_w), (f.dilation_h, f.dilation_w))
    R = tensor_of(case["R"]).numpy()
    assert Y.shape == R.shape == (f.batches, f.channels, f.output_h, f.output_w)
    assert np.array_equal(Y, R)


def test_global_pooling_golden():
    """TEST(DNNTest, GlobalPooling) (dlf/test/DNNTest.cpp:769-794), through the plane reduction
    and through pooling with the whole plane as the window (the device route of the reference)."""
    g = G["pool"]["global"]
    X = tensor_of(g["X"]).numpy()
    assert oracle.global_pool(X, "max").ravel().tolist() == g["max_R"]
    assert oracle.global_pool(X, "avg").ravel().tolist() == g["avg_R"]
    assert oracle.pool2d(X, X.shape[2:], "max", strides=X.shape[2:]).ravel().tolist() == g["max_R"]
    assert oracle.pool2d(X, X.shape[2:], "avg", strides=X.shape[2:]).ravel().tolist() == g["avg_R"]


def test_average_pool_counts():
    """count_include_pad divides by kernel_h*kernel_w, otherwise by the taps inside the image
    (dnn_detail.h:205-221)."""
    X = np.ones((1, 1, 4, 4), np.float32)
    a = oracle.pool2d(X, (3, 3), "avg", (1, 1, 1, 1))
    b = oracle.pool2d(X, (3, 3), "avg", (1, 1, 1, 1), count_include_pad=True)
    assert np.all(a == 1.0)
    assert b[0, 0, 0, 0] == np.float32(4.0 / 9.0) and b[0, 0, 1, 1] == 1.0


# ------------------------------------------------------------------------------------------
# level-3 routines built on GEMM
# ------------------------------------------------------------------------------------------
_SIDE = {"Left": oracle.LEFT, "Right": oracle.RIGHT}
_TRI = {"Upper": oracle.UPPER, "Lower": oracle.LOWER}
_TRANS = {"NoTrans": oracle.NO_TRANS, "Trans": oracle.TRANS}
_DIAG = {"NonUnit": oracle.NON_UNIT, "Unit": oracle.UNIT}


def _level3_operand(spec):
    if spec.get("identity"):
        return np.eye(spec["shape"][0], dtype=np.float32)
    return tensor_of(spec).numpy().astype(np.float32)


@pytest.mark.parametrize("case", G["level3"]["symm"], ids=lambda c: c["side"] + c["triangle"])
def test_symm_goldens(case):
    """symm_test of dlf/test/GPGPUTest.cpp:307-351: the oracle's symm reproduces the literals."""
    A, B = _level3_operand(case["A"]), _level3_operand(case["B"])
    m, n = B.shape
    C = np.zeros((m, n), np.float32)
    oracle.symm(_SIDE[case["side"]], _TRI[case["triangle"]], m, n, 1.0, A, A.shape[1], B, n, 0.0, C, n)
    assert C.flatten().tolist() == [float(v) for v in case["expected"]["values"]]


@pytest.mark.parametrize("case", G["level3"]["trmm"],
                         ids=lambda c: c["side"] + c["triangle"] + c["transpose"] + c["diagonal"])
def test_trmm_goldens(case):
    """trmm_test of dlf/test/GPGPUTest.cpp:361-470; trsm must undo each of them."""
    A, B = _level3_operand(case["A"]), _level3_operand(case["B"])
    m, n = B.shape
    args = (_SIDE[case["side"]], _TRI[case["triangle"]], _TRANS[case["transpose"]], _DIAG[case["diagonal"]])
    X = B.copy()
    oracle.trmm(*args, m, n, 1.0, A, A.shape[1], X, n)
    assert X.flatten().tolist() == [float(v) for v in case["expected"]["values"]]
    oracle.trsm(*args, m, n, 1.0, A, A.shape[1], X, n, wide=True)
    assert np.allclose(X, B, atol=1e-5)
