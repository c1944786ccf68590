"""GPU suite: the CUDA path, called through the C-ABI (dlf_b200.gblas / gdnn are ctypes shims over
libdlf_b200.so), against the reference's golden vectors and against the CPU oracle on seeded
inputs. Tolerances: bit-exact for the integer-valued goldens; fp32 <= 1e-5 relative Frobenius
error; fp16 / bf16 <= 2e-2 max relative error (relative to max(|y|, 1e-2*max|y|))."""
import itertools
import threading

import numpy as np
import pytest
import torch

import oracle
from support import evaluate, load_goldens, max_rel, rel_fro, tensor_of, UNSUPPORTED_EXPR

pytestmark = pytest.mark.gpu

G = load_goldens()
FP32_TOL = 1e-5
HALF_TOL = 2e-2


@pytest.fixture(scope="module")
def lib():
    import dlf_b200
    return dlf_b200


@pytest.fixture(autouse=True)
def _device_status_clean(lib):
    yield
    assert lib.device_status() == 0, "a device-side bounded wait timed out"


def _gb():
    from dlf_b200 import gblas
    return gblas


def _rand(rng, shape, dist="uniform"):
    if dist == "uniform":
        return rng.uniform(-1, 1, shape).astype(np.float32)
    return rng.normal(size=shape).astype(np.float32)


def _round_to(x, dtype):
    """float32 array rounded (nearest-even) to the storage type and back."""
    return torch.from_numpy(x).to(dtype).to(torch.float32).numpy()


# ------------------------------------------------------------------------------------------
# golden vectors of the reference's tests, through the C-ABI
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", G["gemm"], ids=lambda c: c["source"])
def test_gemm_goldens(case, dtype):
    gb = _gb()
    A, At, B, Bt, C, R = (tensor_of(case[k], dtype) for k in ("A", "A_t", "B", "B_t", "C", "R"))
    N, T = gb.Transpose.NoTrans, gb.Transpose.Trans
    for ta, tb, a, b in ((N, N, A, B), (T, N, At, B), (N, T, A, Bt), (T, T, At, Bt)):
        c = C.clone().cuda()
        gb.gemm(gb.Layout.RowMajor, ta, tb, 3, 4, 6, 2, a.cuda().reshape(-1), 0, a.shape[1],
                b.cuda().reshape(-1), 0, b.shape[1], 3, c.reshape(-1), 0, 4)
        assert torch.equal(c.cpu(), R)
        # the same product for a column-major caller (transposed storage)
        c = C.t().contiguous().cuda()
        gb.gemm(gb.Layout.ColMajor, ta, tb, 3, 4, 6, 2, a.t().contiguous().cuda().reshape(-1), 0,
                a.shape[0], b.t().contiguous().cuda().reshape(-1), 0, b.shape[0], 3,
                c.reshape(-1), 0, 3)
        assert torch.equal(c.cpu().t(), R)


def _supported(case):
    text = " ".join(c["a"] + c["b"] for c in case["checks"]) + \
        " ".join(v.get("expr", "") for v in case["vars"].values())
    return not any(u in text for u in UNSUPPORTED_EXPR)


@pytest.mark.parametrize("case", G["matmul"], ids=lambda c: c["name"])
def test_matmul_goldens(case):
    from dlf_b200 import tensor as dt
    if not _supported(case):
        pytest.skip("expression form not modelled")
    env = dict(case["vars"])
    # build the views on the device from device-resident base tensors
    for k, v in list(env.items()):
        if "expr" not in v:
            env[k] = tensor_of(v).cuda()
    for chk in case["checks"]:
        A, B = evaluate(chk["a"], env), evaluate(chk["b"], env)
        expect = evaluate(chk["expect"], env)
        if not A.is_cuda:
            A = A.cuda()
        if not B.is_cuda:
            B = B.cuda()
        got = dt.matmul(A, B)
        assert list(got.shape) == list(expect.shape)
        assert torch.equal(got.cpu(), expect.cpu()), (case["name"], chk)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", G["dot"], ids=lambda c: c["name"])
def test_dot_goldens(case, dtype):
    """dlf::dot / multi_dot on device tensors: TensorTest.Dot, UniformTest.Dot / MultiDot* and the
    GPGPUTest vector / matrix dots, bit-exact (all values are small integers)."""
    from dlf_b200 import tensor as dt
    expect = tensor_of(case["expected"], dtype)
    if dtype == torch.float16 and float(expect.float().abs().max()) > 2048:
        pytest.skip("expected values are not exactly representable in fp16")
    args = [tensor_of(a, dtype).cuda() for a in case["args"]]
    got = dt.dot(args[0], args[1]) if len(args) == 2 else dt.multi_dot(*args)
    assert list(got.shape) == list(expect.shape)
    assert torch.equal(got.cpu(), expect), case["name"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", G["conv2d"], ids=lambda c: c["name"])
def test_conv2d_goldens(case, dtype):
    from dlf_b200 import gdnn
    X, W = tensor_of(case["X"], dtype), tensor_of(case["W"], dtype)
    f = case["filter"]
    filt = gdnn.Filter2D(X.shape, W.shape, f["group"]).pads(*f["pads"]).strides(*f["strides"])
    Y = torch.full(filt.output_shape(), float("nan"), dtype=dtype).cuda()
    gdnn.conv2d_filter(X.cuda(), W.cuda(), Y, filt)
    ref = oracle.conv2d(X.float().numpy(), W.float().numpy(), group=f["group"],
                        pads=tuple(f["pads"]), strides=tuple(f["strides"]))
    if "R" in case:
        assert np.array_equal(ref, tensor_of(case["R"]).numpy())
    if dtype == torch.float32 or np.abs(ref).max() <= 2048:
        assert np.array_equal(Y.float().cpu().numpy(), ref)
    else:
        assert max_rel(Y.float().cpu().numpy(), ref) <= HALF_TOL


def test_predict_conv_bias_golden():
    from dlf_b200 import gdnn
    p = G["predict"]["conv"]
    X, W, b = tensor_of(p["X"]), tensor_of(p["W"]), tensor_of(p["bias"])
    filt = gdnn.Filter2D(X.shape, W.shape).pads(*p["pads"])
    Y = torch.empty(filt.output_shape()).cuda()
    gdnn.conv2d_filter(X.cuda(), W.cuda(), Y, filt, bias=b.cuda())
    assert torch.equal(Y.cpu(), tensor_of(p["Y"]))


def test_predict_gemm_golden():
    from dlf_b200 import tensor as dt
    gb = _gb()
    p = G["predict"]["gemm"]
    got = dt.gemm(gb.Transpose.NoTrans, gb.Transpose.NoTrans, 1.0, tensor_of(p["A"]).cuda(),
                  tensor_of(p["B"]).cuda(), 1.0, tensor_of(p["C"]).cuda())
    assert torch.equal(got.cpu(), tensor_of(p["Y"]))


# ------------------------------------------------------------------------------------------
# seeded random parity against the oracle
# ------------------------------------------------------------------------------------------
def _gemm_case(rng, dtype, layout, ta, tb, m, n, k, alpha, beta, pad, offs, nan_c=False):
    gb = _gb()
    row = layout == gb.Layout.RowMajor
    a_one, a_two, b_one, b_two, c_one, c_two = gb._dims(layout, ta, tb, m, n, k)
    lda, ldb, ldc = a_one + pad[0], b_one + pad[1], c_one + pad[2]
    A = _round_to(_rand(rng, offs[0] + lda * a_two), dtype)
    B = _round_to(_rand(rng, offs[1] + ldb * b_two), dtype)
    C = _round_to(_rand(rng, offs[2] + ldc * c_two, "normal"), dtype)
    ref = C.copy()
    oracle.gblas_sgemm(int(layout), int(ta), int(tb), m, n, k, alpha, A, offs[0], lda, B, offs[1],
                       ldb, beta, ref, offs[2], ldc, wide=True)
    dC = torch.from_numpy(C).to(dtype).cuda()
    if nan_c:
        dC.fill_(float("nan"))
    before = dC.clone()
    gb.gemm(layout, ta, tb, m, n, k, alpha, torch.from_numpy(A).to(dtype).cuda(), offs[0], lda,
            torch.from_numpy(B).to(dtype).cuda(), offs[1], ldb, beta, dC, offs[2], ldc)
    got = dC.float().cpu().numpy()
    # elements outside the m x n window (padding, offset prefix) must be untouched
    mask = np.zeros(C.shape, bool)
    for j in range(c_two):
        mask[offs[2] + j * ldc: offs[2] + j * ldc + c_one] = True
    b4 = before.float().cpu().numpy()
    assert np.array_equal(got[~mask], b4[~mask], equal_nan=True)
    return got[mask], ref[mask]


SHAPES = [(1, 1, 1), (3, 4, 6), (127, 65, 33), (128, 256, 64), (130, 260, 70), (257, 31, 500),
          (64, 1, 96), (1, 300, 64)]


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_fp32_all_layouts(m, n, k):
    gb = _gb()
    rng = np.random.default_rng(m * 1000003 + n * 1009 + k)
    combos = itertools.product((gb.Layout.RowMajor, gb.Layout.ColMajor),
                               (gb.Transpose.NoTrans, gb.Transpose.Trans),
                               (gb.Transpose.NoTrans, gb.Transpose.Trans))
    for i, (layout, ta, tb) in enumerate(combos):
        pad = (0, 0, 0) if i % 2 == 0 else (3, 5, 1)
        offs = (0, 0, 0) if i % 3 == 0 else (7, 2, 9)
        got, ref = _gemm_case(rng, torch.float32, layout, ta, tb, m, n, k, 0.5, 0.5, pad, offs)
        assert rel_fro(got, ref) <= FP32_TOL, (layout, ta, tb)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_half_all_layouts(dtype, m, n, k):
    """Covers both operand loaders: aligned leading dimensions take the TMA producer, the padded /
    offset variants (odd element offsets) take the generic loader warps."""
    gb = _gb()
    rng = np.random.default_rng(m * 7919 + n * 104729 + k)
    combos = itertools.product((gb.Layout.RowMajor, gb.Layout.ColMajor),
                               (gb.Transpose.NoTrans, gb.Transpose.Trans),
                               (gb.Transpose.NoTrans, gb.Transpose.Trans))
    for i, (layout, ta, tb) in enumerate(combos):
        pad = ((0, 0, 0), (8, 16, 8), (3, 5, 1))[i % 3]
        offs = ((0, 0, 0), (8, 16, 24), (7, 2, 9))[i % 3]
        got, ref = _gemm_case(rng, dtype, layout, ta, tb, m, n, k, 0.125, 0.0, pad, offs)
        assert max_rel(got, ref) <= HALF_TOL, (layout, ta, tb)


def test_gemm_aligned_shapes_take_both_loaders(lib):
    """Same aligned problem through the TMA producer and through the forced generic loader."""
    gb = _gb()
    rng = np.random.default_rng(5)
    outs = []
    for generic in (False, True):
        lib.set_tuning(0, generic)
        try:
            got, ref = _gemm_case(np.random.default_rng(5), torch.float16, gb.Layout.RowMajor,
                                  gb.Transpose.NoTrans, gb.Transpose.Trans, 384, 520, 264, 1.0,
                                  0.0, (0, 0, 0), (0, 0, 0))
        finally:
            lib.set_tuning(0, False)
        assert max_rel(got, ref) <= HALF_TOL
        outs.append(got)
    assert np.array_equal(outs[0], outs[1])  # same tiles, same accumulation order
    del rng


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_gemm_every_tile_width(lib, bn):
    gb = _gb()
    lib.set_tuning(bn, False)
    try:
        got, ref = _gemm_case(np.random.default_rng(bn), torch.float16, gb.Layout.ColMajor,
                              gb.Transpose.NoTrans, gb.Transpose.NoTrans, 520, 776, 328, 1.0, 0.0,
                              (0, 0, 0), (0, 0, 0))
        assert max_rel(got, ref) <= HALF_TOL
        if bn != 256:
            got, ref = _gemm_case(np.random.default_rng(bn), torch.float32, gb.Layout.RowMajor,
                                  gb.Transpose.Trans, gb.Transpose.NoTrans, 300, 520, 200, 0.5,
                                  0.5, (0, 0, 0), (0, 0, 0))
            assert rel_fro(got, ref) <= FP32_TOL
    finally:
        lib.set_tuning(0, False)


@pytest.mark.parametrize("bn,flags", [(96, 3), (160, 3), (192, 3), (224, 3), (192, 3 | 0x400), (256, 3)])
def test_tensor_memory_operand_kernel_tile_widths(lib, bn, flags):
    """The kernel that keeps operand A in tensor memory takes any tile width that is a multiple of
    32, with one or two accumulators (two whenever two operand slots remain; 0x400 asks for
    three). fp16 GEMM in both operand orders, fp32 GEMM (widths up to 192 fit two accumulators)
    and a 1x1 convolution, against the oracle."""
    from dlf_b200 import gdnn
    gb = _gb()
    lib.set_tuning(bn, flags)
    try:
        for ta in (gb.Transpose.NoTrans, gb.Transpose.Trans):
            got, ref = _gemm_case(np.random.default_rng(bn), torch.float16, gb.Layout.ColMajor,
                                  ta, gb.Transpose.NoTrans, 390, 500, 200, 1.0, 0.0, (0, 0, 0), (0, 0, 0))
            assert max_rel(got, ref) <= HALF_TOL
        # B stored n-contiguous (MN-major tile made of whole 64-column groups: widths that end
        # inside a group are rounded down), odd leading dimensions keep it off the TMA kernel
        got, ref = _gemm_case(np.random.default_rng(bn + 1), torch.float16, gb.Layout.RowMajor,
                              gb.Transpose.Trans, gb.Transpose.NoTrans, 281, 303, 323, 0.125, 0.0,
                              (0, 0, 0), (0, 0, 0))
        assert max_rel(got, ref) <= HALF_TOL
        got, ref = _gemm_case(np.random.default_rng(bn), torch.float32, gb.Layout.RowMajor,
                              gb.Transpose.Trans, gb.Transpose.NoTrans, 300, 520, 200, 0.5, 0.5,
                              (0, 0, 0), (0, 0, 0))
        assert rel_fro(got, ref) <= FP32_TOL
        for dtype in (torch.float16, torch.float32):
            rng = np.random.default_rng(bn)
            X = _round_to(rng.normal(size=(3, 72, 14, 14)).astype(np.float32), dtype)
            Wt = _round_to((0.1 * rng.normal(size=(424, 72, 1, 1))).astype(np.float32), dtype)
            ref = oracle.conv2d(X, Wt, group=1, pads=(0, 0, 0, 0), strides=(1, 1), dilations=(1, 1), wide=True)
            filt = gdnn.Filter2D(X.shape, Wt.shape)
            Y = torch.full(ref.shape, float("nan"), dtype=dtype, device="cuda")
            gdnn.conv2d_filter(torch.from_numpy(X).to(dtype).cuda(), torch.from_numpy(Wt).to(dtype).cuda(), Y, filt)
            got = Y.float().cpu().numpy()
            if dtype == torch.float32:
                assert rel_fro(got, ref) <= FP32_TOL
            else:
                assert max_rel(got, ref) <= HALF_TOL
    finally:
        lib.set_tuning(0, 0)


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("n", [96, 160, 200, 264, 520])
def test_gemm_tma_store_box_widths(lib, bn, n):
    """The TMA-fed kernel writes 16-bit outputs as TMA stores of 32 x 64 blocks (two staged 32 x 32
    blocks per store) when tiles are 128 columns or wider, else 32 x 32; N values whose last block
    pair is half empty or cut by the matrix edge must come out identical in both forms, with
    nothing written beyond column N."""
    gb = _gb()
    outs = []
    for flags in (0, 0x100):
        lib.set_tuning(bn, flags)
        try:
            got, ref = _gemm_case(np.random.default_rng(n), torch.float16, gb.Layout.ColMajor,
                                  gb.Transpose.NoTrans, gb.Transpose.Trans, 328, n, 136, 1.0, 0.0,
                                  (0, 0, 8), (0, 0, 0))
        finally:
            lib.set_tuning(0, 0)
        assert max_rel(got, ref) <= HALF_TOL
        outs.append(got)
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("m", [85, 88, 381])
def test_gemm_padded_c_keeps_its_padding_with_tma_compatible_strides(lib, m):
    """C has a leading dimension that is a multiple of 16 bytes but a contiguous extent that is
    not (m = 85 or 381 with ld = m + 3): a TMA store would be clipped only at the next 16-byte
    boundary and overwrite the padding, so such outputs must take the plain stores. The helper
    checks that nothing outside the m x n window changes."""
    gb = _gb()
    for dtype in (torch.float16, torch.bfloat16):
        got, ref = _gemm_case(np.random.default_rng(m), dtype, gb.Layout.ColMajor, gb.Transpose.NoTrans,
                              gb.Transpose.Trans, m, 200, 136, -2.0, 0.0, (3, 0, 3), (0, 8, 0))
        assert max_rel(got, ref) <= HALF_TOL
        # the same for loads: K-major operands whose rows hold k = 133 values and 3 of padding
        # (ld = 136): the TMA loads must zero-fill from element 133 on, not from the next
        # 16-byte boundary
        got, ref = _gemm_case(np.random.default_rng(m + 1), dtype, gb.Layout.RowMajor, gb.Transpose.NoTrans,
                              gb.Transpose.Trans, 96, 72, 133, 1.0, 0.0, (3, 3, 0), (8, 0, 0))
        assert max_rel(got, ref) <= HALF_TOL


@pytest.mark.parametrize("m,n,k", [(512, 512, 264), (300, 520, 200), (1000, 264, 72)])
def test_gemm_cta_pair_kernel(lib, m, n, k):
    """The cta_group::2 variant (two CTAs share 256 x 256 tiles; opt-in, tuning bit 0x200) on all
    four transpose combinations, with a ragged M whose second half-tile is partly or wholly
    outside the matrix; the result must equal the single-CTA kernel's bit for bit."""
    gb = _gb()
    for ta, tb in itertools.product((gb.Transpose.NoTrans, gb.Transpose.Trans), repeat=2):
        outs = []
        for flag in (0, 0x200):
            lib.set_tuning(256, flag)
            try:
                got, ref = _gemm_case(np.random.default_rng(m + n), torch.float16, gb.Layout.RowMajor,
                                      ta, tb, m, n, k, 1.0, 0.0, (0, 0, 0), (0, 0, 0))
            finally:
                lib.set_tuning(0, 0)
            assert max_rel(got, ref) <= HALF_TOL
            outs.append(got)
        assert np.array_equal(outs[0], outs[1])


def test_beta_zero_never_reads_c():
    """beta == 0 must overwrite C without reading it (xgemm_part2.cl:87-126): NaNs in C vanish."""
    gb = _gb()
    rng = np.random.default_rng(11)
    for dtype, tol, metric in ((torch.float32, FP32_TOL, rel_fro), (torch.float16, HALF_TOL, max_rel)):
        got, ref = _gemm_case(rng, dtype, gb.Layout.RowMajor, gb.Transpose.NoTrans,
                              gb.Transpose.NoTrans, 100, 72, 40, 1.0, 0.0, (0, 0, 0), (0, 0, 0),
                              nan_c=True)
        assert not np.isnan(got).any()
        assert metric(got, ref) <= tol


@pytest.mark.parametrize("flags", [0, 1], ids=["tma-store-epilogue", "generic-epilogue"])
def test_nan_in_an_operand_stays_nan(lib, flags):
    """A NaN in A reaches every output it contributes to, and only those, on the TMA-fed kernel
    (whose epilogue writes through TMA stores) as on the loader-warp kernel - the oracle's
    positions exactly. (fmaxf drops a NaN operand: the ReLU clamp must not run without ReLU.)"""
    gb = _gb()
    m, n, k = 160, 136, 72
    rng = np.random.default_rng(99)
    A = _round_to(_rand(rng, m * k), torch.float16)
    B = _round_to(_rand(rng, k * n), torch.float16)
    A[5 * k + 3] = np.nan   # row 5
    A[130 * k + 70] = np.nan  # row 130
    ref = np.zeros(m * n, np.float32)
    oracle.gblas_sgemm(oracle.ROW_MAJOR, oracle.NO_TRANS, oracle.NO_TRANS, m, n, k, 1.0, A, 0, k, B, 0, n,
                       0.0, ref, 0, n)
    C = torch.zeros(m * n, dtype=torch.float16, device="cuda")
    lib.set_tuning(0, flags)
    try:
        gb.gemm(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, m, n, k, 1.0,
                torch.from_numpy(A).half().cuda(), 0, k, torch.from_numpy(B).half().cuda(), 0, n, 0.0, C, 0, n)
        torch.cuda.synchronize()
    finally:
        lib.set_tuning(0, 0)
    got = C.float().cpu().numpy()
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    assert np.isnan(got).sum() == 2 * n
    ok = ~np.isnan(ref)
    assert max_rel(got[ok], ref[ok]) <= HALF_TOL


def test_calls_on_a_queue_that_is_not_the_current_stream(lib):
    """gemmBatched and conv2d on an explicit queue while another stream is current: their scratch
    (offset tables, packed filter bank) is allocated by the caller's allocator and must stay alive
    until the queue has passed the work that reads it."""
    from dlf_b200 import gdnn
    gb = _gb()
    q = torch.cuda.Stream()
    rng = np.random.default_rng(21)
    m, n, k, batch = 48, 40, 56, 6
    A = torch.from_numpy(_rand(rng, batch * m * k)).cuda()
    B = torch.from_numpy(_rand(rng, batch * k * n)).cuda()
    X = torch.from_numpy(_rand(rng, (2, 8, 12, 12), "normal")).cuda()
    W = torch.from_numpy(0.1 * _rand(rng, (16, 8, 3, 3), "normal")).cuda()
    f = gdnn.Filter2D(X.shape, W.shape).pads(1, 1)
    torch.cuda.synchronize()
    outs = []
    for _ in range(3):
        C = torch.zeros(batch * m * n, device="cuda")
        Y = torch.empty(f.output_shape(), device="cuda")
        q.wait_stream(torch.cuda.current_stream())
        gb.gemmBatched(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, m, n, k, [1.0] * batch,
                       A, [i * m * k for i in range(batch)], k, B, [i * k * n for i in range(batch)], n,
                       [0.0] * batch, C, [i * m * n for i in range(batch)], n, batch, queue=q)
        gdnn.conv2d_filter(X, W, Y, f, queue=q)
        # allocator traffic on the current stream while the queue may still be working
        junk = [torch.full((1 << 16,), 7.0, device="cuda") for _ in range(8)]
        del junk
        outs.append((C, Y))
    q.synchronize()
    torch.cuda.synchronize()
    refC = torch.bmm(A.view(batch, m, k).double(), B.view(batch, k, n).double()).float().flatten()
    refY = oracle.conv2d(X.cpu().numpy(), W.cpu().numpy(), pads=(1, 1, 1, 1), wide=True)
    for C, Y in outs:
        assert rel_fro(C.cpu().numpy(), refC.cpu().numpy()) <= FP32_TOL
        assert rel_fro(Y.cpu().numpy(), refY) <= FP32_TOL


def test_conv2d_dilation_beyond_16_bits_takes_the_wide_index_kernel(lib):
    """(KH-1)*dilation_h = 40000 does not fit the 16-bit tap offsets of the tensor-memory-operand
    kernel's k table: the call must be served by the kernel with wide indices (one launch, no
    packing grid) and give the oracle's result (only the kh = 0 tap lies inside the image)."""
    from dlf_b200 import gdnn
    rng = np.random.default_rng(40000)
    X = _rand(rng, (2, 3, 6, 9), "normal")
    Wt = _rand(rng, (5, 3, 2, 2), "normal")
    ref = oracle.conv2d(X, Wt, dilations=(40000, 1), wide=True)
    filt = gdnn.Filter2D(X.shape, Wt.shape).dilations(40000, 1)
    assert tuple(filt.output_shape()) == ref.shape
    Y = torch.full(ref.shape, float("nan"), device="cuda")
    n0 = lib.launch_count()
    gdnn.conv2d_filter(torch.from_numpy(X).cuda(), torch.from_numpy(Wt).cuda(), Y, filt)
    assert lib.launch_count() - n0 == 1
    assert rel_fro(Y.cpu().numpy(), ref) <= FP32_TOL


@pytest.mark.parametrize("k", [1056, 4096])
def test_gemm_fp32_long_k_stays_accurate(k):
    """The tensor core truncates when it adds into its fp32 accumulator; without countermeasure the
    3xTF32 result drifts by about 6e-9*K (1e-4 at K = 16384). Long K is therefore accumulated in
    chunks that are summed with ordinary fp32 adds: the error must stay well inside 1e-5."""
    gb = _gb()
    rng = np.random.default_rng(k)
    for (layout, ta, tb, m, n) in ((gb.Layout.RowMajor, gb.Transpose.Trans, gb.Transpose.NoTrans, 200, 136),
                                   (gb.Layout.ColMajor, gb.Transpose.NoTrans, gb.Transpose.Trans, 130, 300)):
        got, ref = _gemm_case(rng, torch.float32, layout, ta, tb, m, n, k, 0.5, 0.5, (0, 0, 0), (0, 0, 0))
        assert rel_fro(got, ref) <= 4e-6


@pytest.mark.parametrize("chunked", [True, False], ids=["chunked", "one-accumulator"])
def test_gemm_config5_shape_at_k_16384(lib, chunked):
    """BASELINE config 5 at its own K: row-major, A stored K x M and passed Trans, alpha = beta =
    0.5, K = 16384 (M, N kept small so that the oracle finishes in seconds). With the K-chunked
    accumulation the error stays inside the 1e-5 tolerance; accumulating all of K in one
    tensor-core accumulator (tuning bit 0x1000) shows the truncation drift the chunks remove."""
    gb = _gb()
    m, n, k = 256, 384, 16384
    rng = np.random.default_rng(5)
    A = _rand(rng, k * m)
    B = _rand(rng, k * n)
    C0 = rng.normal(size=m * n).astype(np.float32)
    ref = C0.copy()
    oracle.gblas_sgemm(oracle.ROW_MAJOR, oracle.TRANS, oracle.NO_TRANS, m, n, k, 0.5, A, 0, m, B, 0, n,
                       0.5, ref, 0, n, wide=True)
    C = torch.from_numpy(C0.copy()).cuda()
    lib.set_tuning(0, 0 if chunked else 0x1000)
    try:
        gb.gemm(gb.Layout.RowMajor, gb.Transpose.Trans, gb.Transpose.NoTrans, m, n, k, 0.5,
                torch.from_numpy(A).cuda(), 0, m, torch.from_numpy(B).cuda(), 0, n, 0.5, C, 0, n)
        torch.cuda.synchronize()
    finally:
        lib.set_tuning(0, 0)
    err = rel_fro(C.cpu().numpy(), ref)
    if chunked:
        assert err <= 4e-6, err
        test_gemm_config5_shape_at_k_16384.chunked_err = err
    else:
        assert err > getattr(test_gemm_config5_shape_at_k_16384, "chunked_err", 4e-6), err


def test_gemm_config1_sgemm_1024():
    """BASELINE config 1: fp32 row-major 1024^3, alpha 1, beta 0, U[-1,1] seed 0, C zero."""
    gb = _gb()
    rng = np.random.default_rng(0)
    A, B = _rand(rng, 1024 * 1024), _rand(rng, 1024 * 1024)
    ref = np.zeros(1024 * 1024, np.float32)
    oracle.gblas_sgemm(oracle.ROW_MAJOR, oracle.NO_TRANS, oracle.NO_TRANS, 1024, 1024, 1024, 1.0,
                       A, 0, 1024, B, 0, 1024, 0.0, ref, 0, 1024)
    C = torch.zeros(1024 * 1024, device="cuda")
    gb.gemm(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, 1024, 1024, 1024, 1.0,
            torch.from_numpy(A).cuda(), 0, 1024, torch.from_numpy(B).cuda(), 0, 1024, 0.0, C, 0, 1024)
    assert rel_fro(C.cpu().numpy(), ref) <= FP32_TOL


# ------------------------------------------------------------------------------------------
# batched
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_strided_batched_including_shared_operand(dtype):
    gb = _gb()
    rng = np.random.default_rng(21)
    m, n, k, batch = 70, 90, 50, 5
    for a_stride, ta, tb in ((m * k + 8, gb.Transpose.NoTrans, gb.Transpose.NoTrans),
                             (0, gb.Transpose.NoTrans, gb.Transpose.Trans),
                             (m * k, gb.Transpose.Trans, gb.Transpose.NoTrans)):
        lda = k if ta == gb.Transpose.NoTrans else m
        ldb = n if tb == gb.Transpose.NoTrans else k
        b_stride, c_stride = k * n + 16, m * n
        A = _round_to(_rand(rng, a_stride * (batch - 1) + m * k + 3), dtype)
        B = _round_to(_rand(rng, b_stride * (batch - 1) + k * n + 5), dtype)
        C = _round_to(_rand(rng, c_stride * batch), dtype)
        ref = C.copy()
        oracle.gblas_sgemm_strided_batched(oracle.ROW_MAJOR, int(ta), int(tb), m, n, k, 0.5, A, 3,
                                           lda, a_stride, B, 5, ldb, b_stride, 0.25, ref, 0, n,
                                           c_stride, batch, wide=True)
        dC = torch.from_numpy(C).to(dtype).cuda()
        gb.gemmStridedBatched(gb.Layout.RowMajor, ta, tb, m, n, k, 0.5,
                              torch.from_numpy(A).to(dtype).cuda(), 3, lda, a_stride,
                              torch.from_numpy(B).to(dtype).cuda(), 5, ldb, b_stride, 0.25, dC, 0,
                              n, c_stride, batch)
        got = dC.float().cpu().numpy()
        if dtype == torch.float32:
            assert rel_fro(got, ref) <= FP32_TOL
        else:
            assert max_rel(got, ref) <= HALF_TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(256, 384, 64, 3), (136, 200, 72, 2), (128, 128, 256, 1), (520, 136, 40, 2)],
                         ids=lambda s: "x".join(map(str, s)))
def test_short_k_products_computed_transposed(lib, shape, dtype):
    """A 16-bit product with K <= 256 and N >= 128 whose result can leave through TMA stores is
    computed as D^T = Bu * Au^T (the lanes hold D's columns, the epilogue writes 16-byte pieces of
    D's contiguous direction); bit 30 of the tile-width word turns that off. Both ways against the
    oracle for every transpose combination in both layouts, padded leading dimension and batch
    stride of C, beta = 0 with C pre-filled (it must not be read), nothing outside the m x n windows
    touched, and the two ways bit-identical (the same products summed in the same order)."""
    gb = _gb()
    m, n, k, batch = shape
    rng = np.random.default_rng(sum(shape))
    for layout in (gb.Layout.RowMajor, gb.Layout.ColMajor):
        for ta in (gb.Transpose.NoTrans, gb.Transpose.Trans):
            for tb in (gb.Transpose.NoTrans, gb.Transpose.Trans):
                a_one, a_two, b_one, b_two, c_one, c_two = gb._dims(layout, ta, tb, m, n, k)
                lda, ldb, ldc = a_one, b_one, c_one + 8
                a_stride, b_stride, c_stride = lda * a_two, ldb * b_two + 16, ldc * c_two + 24
                A = _round_to(_rand(rng, a_stride * batch), dtype)
                B = _round_to(_rand(rng, b_stride * batch), dtype)
                C = np.full(c_stride * batch, 7.0, dtype=np.float32)
                ref = C.copy()
                oracle.gblas_sgemm_strided_batched(int(layout), int(ta), int(tb), m, n, k, 0.5, A, 0, lda, a_stride,
                                                   B, 0, ldb, b_stride, 0.0, ref, 0, ldc, c_stride, batch, wide=True)
                dA, dB = torch.from_numpy(A).to(dtype).cuda(), torch.from_numpy(B).to(dtype).cuda()
                outs = []
                for route in (0, 0x40000000):
                    dC = torch.full((c_stride * batch,), float("nan"), dtype=dtype, device="cuda")
                    lib.set_tuning(route, 0)
                    try:
                        gb.gemmStridedBatched(layout, ta, tb, m, n, k, 0.5, dA, 0, lda, a_stride, dB, 0, ldb, b_stride,
                                              0.0, dC, 0, ldc, c_stride, batch)
                        torch.cuda.synchronize()
                    finally:
                        lib.set_tuning(0, 0)
                    got = dC.float().cpu().numpy()
                    win = np.zeros(c_stride * batch, dtype=bool)  # the elements of the m x n windows
                    for bb in range(batch):
                        for line in range(c_two):
                            win[bb * c_stride + line * ldc: bb * c_stride + line * ldc + c_one] = True
                    assert np.isnan(got[~win]).all(), "padding touched"
                    assert max_rel(got[win], ref[win]) <= HALF_TOL
                    outs.append(dC)
                assert torch.equal(outs[0][torch.from_numpy(win).cuda()], outs[1][torch.from_numpy(win).cuda()])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_gemm_batched_affine_tables_take_the_strided_path(lib, dtype):
    """Offset tables that are affine in the batch index (one alpha, one beta) run as a strided batch;
    16-bit tables of the form base + idx * stride with 16-byte aligned base and stride (one entry out
    of line by 8 elements; the same matrices in a shuffled order) and beta == 0 keep the
    tensor-map-fed kernel with idx as the batch coordinate; bit 18 of the tile-width word sends
    everything through the offset tables. All against the oracle and equal to each other."""
    gb = _gb()
    rng = np.random.default_rng(77)
    m, n, k, batch = 64, 136, 72, 5
    a_offs = [8 + i * (m * k + 16) for i in range(batch)]
    b_offs = [0] * batch                                    # stride 0: one B for every product
    c_offs = [16 + i * (m * n + 8) for i in range(batch)]
    A = _round_to(_rand(rng, a_offs[-1] + m * k + 64), dtype)
    B = _round_to(_rand(rng, k * n), dtype)
    C = _round_to(_rand(rng, c_offs[-1] + m * n + 40), dtype)
    shuffled = [a_offs[i] for i in (3, 0, 4, 1, 2)]
    dA, dB = torch.from_numpy(A).to(dtype).cuda(), torch.from_numpy(B).to(dtype).cuda()
    for offs_a in (a_offs, a_offs[:3] + [a_offs[3] + 8] + a_offs[4:], shuffled):
        for beta in (0.25, 0.0):
            ref = C.copy()
            oracle.gblas_sgemm_batched(oracle.ROW_MAJOR, oracle.NO_TRANS, oracle.NO_TRANS, m, n, k, [0.5] * batch, A,
                                       offs_a, k, B, b_offs, n, [beta] * batch, ref, c_offs, n, batch, wide=True)
            outs = []
            for route in (0, 0x40000):
                dC = torch.from_numpy(C).to(dtype).cuda()
                lib.set_tuning(route, 0)
                try:
                    gb.gemmBatched(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, m, n, k,
                                   [0.5] * batch, dA, offs_a, k, dB, b_offs, n, [beta] * batch, dC, c_offs, n, batch)
                    torch.cuda.synchronize()
                finally:
                    lib.set_tuning(0, 0)
                got = dC.float().cpu().numpy()
                assert (rel_fro(got, ref) <= FP32_TOL) if dtype == torch.float32 else (max_rel(got, ref) <= HALF_TOL)
                outs.append(got)
            if dtype == torch.float32:
                assert rel_fro(outs[0], outs[1]) <= FP32_TOL
            else:
                assert max_rel(outs[0], outs[1]) <= HALF_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_batched_offset_tables(dtype):
    gb = _gb()
    rng = np.random.default_rng(31)
    m, n, k, batch = 33, 45, 27, 6
    a_offs = [7 + i * (m * k + 3) for i in range(batch)]
    b_offs = [(batch - 1 - i) * (k * n + 1) for i in range(batch)]  # reversed order
    c_offs = [2 + i * (m * n + 4) for i in range(batch)]
    alphas = [0.5 + 0.25 * i for i in range(batch)]
    betas = [0.0 if i % 2 == 0 else 0.5 for i in range(batch)]
    A = _round_to(_rand(rng, a_offs[-1] + m * k), dtype)
    B = _round_to(_rand(rng, b_offs[0] + k * n), dtype)
    C = _round_to(_rand(rng, c_offs[-1] + m * n), dtype)
    ref = C.copy()
    oracle.gblas_sgemm_batched(oracle.COL_MAJOR, oracle.NO_TRANS, oracle.TRANS, m, n, k, alphas, A,
                               a_offs, m, B, b_offs, n, betas, ref, c_offs, m, batch, wide=True)
    dC = torch.from_numpy(C).to(dtype).cuda()
    gb.gemmBatched(gb.Layout.ColMajor, gb.Transpose.NoTrans, gb.Transpose.Trans, m, n, k, alphas,
                   torch.from_numpy(A).to(dtype).cuda(), a_offs, m,
                   torch.from_numpy(B).to(dtype).cuda(), b_offs, n, betas, dC, c_offs, m, batch)
    got = dC.float().cpu().numpy()
    if dtype == torch.float32:
        assert rel_fro(got, ref) <= FP32_TOL
    else:
        assert max_rel(got, ref) <= HALF_TOL


def test_config4_attention_like_batched_half():
    """BASELINE config 4 shapes at a reduced batch for the element-wise check, both operand
    storage orders; alpha = 1/sqrt(64), beta = 0."""
    gb = _gb()
    rng = np.random.default_rng(4)
    for (m, n, k) in ((512, 512, 64), (512, 64, 512)):
        batch = 6
        for ta, tb in itertools.product((gb.Transpose.NoTrans, gb.Transpose.Trans), repeat=2):
            A = _round_to((0.1 * rng.normal(size=batch * m * k)).astype(np.float32), torch.float16)
            B = _round_to((0.1 * rng.normal(size=batch * k * n)).astype(np.float32), torch.float16)
            lda = k if ta == gb.Transpose.NoTrans else m
            ldb = n if tb == gb.Transpose.NoTrans else k
            ref = np.zeros(batch * m * n, np.float32)
            oracle.gblas_sgemm_strided_batched(oracle.ROW_MAJOR, int(ta), int(tb), m, n, k, 0.125,
                                               A, 0, lda, m * k, B, 0, ldb, k * n, 0.0, ref, 0, n,
                                               m * n, batch, wide=True)
            dC = torch.full((batch * m * n,), float("nan"), dtype=torch.float16, device="cuda")
            gb.gemmStridedBatched(gb.Layout.RowMajor, ta, tb, m, n, k, 0.125,
                                  torch.from_numpy(A).half().cuda(), 0, lda, m * k,
                                  torch.from_numpy(B).half().cuda(), 0, ldb, k * n, 0.0, dC, 0, n,
                                  m * n, batch)
            assert max_rel(dC.float().cpu().numpy(), ref) <= HALF_TOL


# ------------------------------------------------------------------------------------------
# convolution
# ------------------------------------------------------------------------------------------
CONV_CASES = [
    # N, C, H, W, Cout, KH, KW, pads(t,l,b,r), strides, dilations, group
    (2, 64, 56, 56, 64, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 1),     # config 2 at batch 2
    (2, 3, 37, 41, 16, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1), 1),      # stem-like, K = 147
    (3, 32, 14, 14, 48, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 1),     # 1x1
    (3, 64, 8, 16, 80, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 1),      # 1x1, 16-byte-aligned planes: batched-GEMM route
    (2, 16, 12, 12, 320, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 1),    # wide output: 256-column tiles
    (3, 32, 14, 14, 64, 1, 1, (0, 0, 0, 0), (2, 2), (1, 1), 1),     # 1x1 stride 2
    (2, 8, 13, 11, 12, 3, 2, (1, 2, 2, 1), (2, 1), (1, 2), 2),      # odd everything + groups
    (5, 16, 7, 7, 40, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 4),       # tiles straddle images
    (1, 4, 9, 9, 4, 3, 3, (0, 0, 0, 0), (1, 1), (2, 2), 4),         # depthwise, dilated
    (3, 8, 11, 37, 20, 5, 3, (2, 0, 2, 1), (2, 1), (2, 1), 1),      # row form: 5x3, stride_h 2, dilation_h 2, one-sided pad
    (2, 6, 6, 70, 150, 2, 7, (0, 3, 1, 3), (1, 1), (1, 1), 1),      # row form: 7 taps per row, several channel tiles
    (2, 12, 8, 8, 24, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 3),       # row form with groups
    (1, 4, 5, 40, 8, 1, 4, (0, 0, 0, 0), (1, 1), (1, 1), 1),        # row form, no padding: OW < W
    (1, 192, 9, 12, 40, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1), 1),     # row form, K' = 576: chunked accumulation in fp32
    (1, 72, 9, 12, 24, 3, 3, (1, 1, 2, 2), (2, 2), (1, 2), 1),      # im2col form (dilation_w 2), K = 648: chunked accumulation in fp32
    (3, 70, 7, 7, 36, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 1),       # 1x1, odd plane (49 pixels), K tail: affine addressing
    (2, 40, 9, 9, 24, 1, 1, (0, 0, 1, 1), (2, 2), (1, 1), 2),       # 1x1 stride 2, trailing padding reaches outside: table lookup
    (2, 24, 14, 14, 72, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 1),     # 1x1, even plane (196): paired 32-bit stores for 16-bit outputs
    (2, 16, 15, 23, 40, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1), 1),     # strided row form: 3x3 stride 2, odd width (2 shifts, 2 column phases)
    (3, 6, 13, 30, 20, 5, 5, (2, 2, 2, 2), (1, 3), (1, 1), 2),      # strided row form: stride_w 3, groups
    (2, 5, 9, 26, 12, 2, 4, (0, 0, 1, 0), (1, 2), (1, 1), 1),       # strided row form: no left padding (shifts 0..1), KW = 4
    (1, 7, 8, 67, 24, 1, 8, (0, 1, 0, 5), (1, 4), (1, 1), 1),       # strided row form: stride_w 4, KW = 8, wide right padding
    (2, 3, 20, 33, 64, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1), 1),      # stem shape with 64 output channels: 4 shifts x 64 = one 256-column tile
    (2, 36, 25, 21, 36, 5, 7, (3, 0, 1, 3), (1, 1), (2, 1), 1),     # row form, 7 taps x 32 channels = 224 columns: in fp32 four stages would overflow shared memory by the table padding
    (3, 96, 7, 7, 32, 7, 7, (3, 1, 1, 1), (1, 1), (1, 1), 1),       # row form, K' = 672 chunked in fp32 with 7 taps x 16 channels = 112 columns: the sum array is not a multiple of 32 columns
    (2, 120, 9, 10, 24, 5, 5, (2, 2, 2, 2), (1, 1), (1, 1), 1),     # same with 5 taps x 16 channels = 80 columns
    (3, 70, 7, 7, 150, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 1),      # widening 1x1 on odd planes, 70 channels: channels-last copy by funnel shifts, repacked filters
    (2, 24, 9, 9, 64, 1, 1, (0, 0, 0, 0), (2, 2), (1, 1), 1),       # widening 1x1 stride 2, odd output width: per-pixel copy
    (2, 64, 17, 12, 136, 1, 1, (0, 0, 0, 0), (2, 2), (1, 1), 1),    # widening 1x1 stride 2, OW = 6: copy in groups of two kept pixels
    (2, 64, 9, 16, 128, 1, 1, (0, 0, 0, 0), (1, 2), (1, 1), 1),     # widening 1x1, stride_w 2 only, OW = 8: groups of four
    (2, 64, 15, 15, 40, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1), 1),     # 3x3 stride 2, 64 channels: im2col-mode loads with traversal strides
    (2, 4, 13, 18, 24, 2, 4, (0, 1, 1, 2), (1, 2), (1, 1), 1),      # 4 channels, even KH, KW = 4, stride_w 2: small-channel route
    (1, 1, 9, 30, 8, 3, 8, (1, 3, 1, 3), (3, 4), (1, 1), 1),        # 1 channel, KW = 8, strides (3, 4)
    (1, 3, 6, 530, 16, 3, 3, (1, 1, 1, 1), (1, 2), (1, 1), 1),      # 3 channels, 265 outputs per row: three tiles per row
]


# 16-bit convolutions of one group take the channels-last route (transposing copy + tensor-map-fed
# operand) when the caller passes scratch; bit 16 of the tile-width word keeps them on the kernels
# that gather the operand themselves. Both are the product (the second serves callers without scratch).
NO_CL = 0x10000
ROUTES = [(torch.float32, 0), (torch.float16, 0), (torch.float16, NO_CL), (torch.bfloat16, 0),
          (torch.bfloat16, NO_CL)]
ROUTE_IDS = ["f32", "f16-channels-last", "f16-gather", "bf16-channels-last", "bf16-gather"]


@pytest.mark.parametrize("dtype,route", ROUTES, ids=ROUTE_IDS)
@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: "x".join(map(str, c[:7])))
def test_conv2d_random_parity(lib, case, dtype, route):
    from dlf_b200 import gdnn
    N, C, H, W, Co, KH, KW, pads, strides, dil, group = case
    rng = np.random.default_rng(abs(hash(case)) % (2 ** 32))
    X = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
    std = np.sqrt(2.0 / (C // group * KH * KW))
    Wt = _round_to((std * rng.normal(size=(Co, C // group, KH, KW))).astype(np.float32), dtype)
    bias = _round_to(rng.uniform(-0.1, 0.1, Co).astype(np.float32), dtype)
    ref = oracle.conv2d(X, Wt, group=group, pads=pads, strides=strides, dilations=dil, bias=bias,
                        wide=True)
    filt = gdnn.Filter2D(X.shape, Wt.shape, group).pads(*pads).strides(*strides).dilations(*dil)
    assert tuple(filt.output_shape()) == ref.shape
    Y = torch.full(ref.shape, float("nan"), dtype=dtype, device="cuda")
    lib.set_tuning(route, 0)
    try:
        gdnn.conv2d_filter(torch.from_numpy(X).to(dtype).cuda(), torch.from_numpy(Wt).to(dtype).cuda(),
                           Y, filt, bias=torch.from_numpy(bias).to(dtype).cuda())
    finally:
        lib.set_tuning(0, 0)
    got = Y.float().cpu().numpy()
    if dtype == torch.float32:
        assert rel_fro(got, ref) <= FP32_TOL
    else:
        assert max_rel(got, ref) <= HALF_TOL


def _resnet_shapes():
    from bench import RESNET50_SHAPES
    return RESNET50_SHAPES


@pytest.mark.parametrize("route", [0, NO_CL], ids=["channels-last", "gather"])
@pytest.mark.parametrize("shape", _resnet_shapes(), ids=lambda c: "x".join(map(str, c[:6])))
def test_conv2d_resnet50_layer_shapes_vs_oracle(lib, shape, route):
    """BASELINE config 3 at its real layer shapes: every one of the 20 distinct ResNet-50 v1
    convolutions (224 x 224 input), fp16 with bias, two images, against the oracle with a wide
    accumulator. Inputs follow the configuration: activations |N(0,1)|, He-normal weights."""
    from dlf_b200 import gdnn
    cin, h, cout, k, s, p, _count = shape
    rng = np.random.default_rng(cin * 1000 + cout + k)
    X = _round_to(np.abs(rng.normal(size=(2, cin, h, h))).astype(np.float32), torch.float16)
    Wt = _round_to((np.sqrt(2.0 / (cin * k * k)) * rng.normal(size=(cout, cin, k, k))).astype(np.float32),
                   torch.float16)
    bias = _round_to(rng.uniform(-0.1, 0.1, cout).astype(np.float32), torch.float16)
    ref = oracle.conv2d(X, Wt, pads=(p,) * 4, strides=(s, s), bias=bias, wide=True)
    filt = gdnn.Filter2D(X.shape, Wt.shape).pads(p, p).strides(s, s)
    Y = torch.full(ref.shape, float("nan"), dtype=torch.float16, device="cuda")
    lib.set_tuning(route, 0)
    try:
        gdnn.conv2d_filter(torch.from_numpy(X).half().cuda(), torch.from_numpy(Wt).half().cuda(), Y, filt,
                           bias=torch.from_numpy(bias).half().cuda())
    finally:
        lib.set_tuning(0, 0)
    assert max_rel(Y.float().cpu().numpy(), ref) <= HALF_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,n,k,ta,tb", [(256, 1000, 2048, False, False), (200, 136, 4096, True, False),
                                         (96, 520, 1024, False, True), (64, 64, 8192, True, True)])
def test_gemm_k_split_matches_unsplit(lib, dtype, m, n, k, ta, tb):
    """Products with few output tiles and a long K are cut along K when the caller gives scratch
    (dlf_b200_gemm_ex): the result must agree with the oracle and, up to fp32 rounding of the slice
    sums, with the unsplit kernel (tuning bit 0x20000000 switches the split off); beta and alpha
    apply once, in the reduction."""
    gb = _gb()
    rng = np.random.default_rng(m + n + k)
    A = _round_to(_rand(rng, m * k), dtype)
    B = _round_to(_rand(rng, k * n), dtype)
    C0 = _round_to(_rand(rng, m * n, "normal"), dtype)
    TA = gb.Transpose.Trans if ta else gb.Transpose.NoTrans
    TB = gb.Transpose.Trans if tb else gb.Transpose.NoTrans
    lda, ldb = (m if ta else k), (k if tb else n)
    ref = C0.copy()
    oracle.gblas_sgemm(oracle.ROW_MAJOR, int(TA), int(TB), m, n, k, 0.5, A, 0, lda, B, 0, ldb, 0.25, ref, 0, n, wide=True)
    outs = []
    for flags in (0, 0x20000000):
        C = torch.from_numpy(C0.copy()).to(dtype).cuda()
        lib.set_tuning(0, flags)
        try:
            n0 = lib.launch_count()
            gb.gemm(gb.Layout.RowMajor, TA, TB, m, n, k, 0.5, torch.from_numpy(A).to(dtype).cuda(), 0, lda,
                    torch.from_numpy(B).to(dtype).cuda(), 0, ldb, 0.25, C, 0, n)
            torch.cuda.synchronize()
            launches = lib.launch_count() - n0
        finally:
            lib.set_tuning(0, 0)
        assert launches == (2 if flags == 0 else 1)  # split: product + reduction
        outs.append(C.float().cpu().numpy())
        if dtype == torch.float32:
            assert rel_fro(outs[-1], ref) <= FP32_TOL
        else:
            assert max_rel(outs[-1], ref) <= HALF_TOL
    if dtype == torch.float32:
        assert rel_fro(outs[0], outs[1]) <= 6e-6


def test_resnet50_fc_gemm_vs_oracle():
    """The final fully connected layer of config 3 as a GEMM: 256 x 1000 x 2048, fp16."""
    gb = _gb()
    m, n, k = 256, 1000, 2048
    rng = np.random.default_rng(2048)
    A = _round_to(np.abs(rng.normal(size=m * k)).astype(np.float32), torch.float16)
    B = _round_to((np.sqrt(2.0 / k) * rng.normal(size=k * n)).astype(np.float32), torch.float16)
    ref = np.zeros(m * n, np.float32)
    oracle.gblas_sgemm(oracle.ROW_MAJOR, oracle.NO_TRANS, oracle.NO_TRANS, m, n, k, 1.0, A, 0, k, B, 0, n,
                       0.0, ref, 0, n, wide=True)
    C = torch.full((m * n,), float("nan"), dtype=torch.float16, device="cuda")
    gb.gemm(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, m, n, k, 1.0,
            torch.from_numpy(A).half().cuda(), 0, k, torch.from_numpy(B).half().cuda(), 0, n, 0.0, C, 0, n)
    assert max_rel(C.float().cpu().numpy(), ref) <= HALF_TOL


STORE_MODE_CASES = [
    # N, C, H, W, Cout, k, pad, stride
    (2, 16, 24, 24, 32, 3, 1, 1),    # plane of 576 pixels: image-aligned tiles + TMA stores when forced for stride 1
    (3, 16, 14, 14, 40, 3, 1, 1),    # 196-pixel planes: tiles cross images, two runs, 8-byte-aligned planes
    (5, 8, 7, 7, 24, 3, 1, 1),       # 49-pixel planes: up to four runs per tile, 2-byte-aligned planes
    (3, 32, 14, 14, 72, 1, 0, 1),    # 1x1 on the plain epilogue
    (5, 24, 7, 7, 40, 1, 0, 1),      # 1x1, odd planes
    (2, 3, 40, 48, 64, 7, 3, 2),     # strided row form (stem-like): TMA stores by default
    (2, 8, 9, 40, 16, 3, 0, 1),      # no padding: output rows shorter than the position rows
    (40, 4, 3, 3, 8, 3, 1, 1),       # 9-pixel planes: more images per tile than the staging handles -> direct stores
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", STORE_MODE_CASES, ids=lambda c: "x".join(map(str, c)))
def test_conv2d_output_store_modes_agree(lib, case, dtype):
    """The two ways 16-bit results of the row-form convolution leave the SM - one element per lane,
    or TMA stores of image-aligned tiles (default for the strided row form, measurement bit
    128 << 16 for stride 1) - give the same bits, with and without a residual + ReLU, and touch
    nothing outside Y."""
    from dlf_b200 import gdnn
    N, C, H, W, Co, k, p, s = case
    rng = np.random.default_rng(sum(case))
    X = torch.from_numpy(_rand(rng, (N, C, H, W), "normal")).to(dtype).cuda()
    Wt = torch.from_numpy(0.2 * _rand(rng, (Co, C, k, k), "normal")).to(dtype).cuda()
    bias = torch.from_numpy(_rand(rng, Co)).to(dtype).cuda()
    f = gdnn.Filter2D(X.shape, Wt.shape).pads(p, p).strides(s, s)
    n_out = int(np.prod(f.output_shape()))
    R = torch.from_numpy(_rand(rng, f.output_shape(), "normal")).to(dtype).cuda()
    for fused in (False, True):
        outs = []
        for flags in (0, 128 << 16):
            buf = torch.full((n_out + 64,), 3.0, dtype=dtype, device="cuda")  # guard band on both sides
            Y = buf[32:32 + n_out].view(f.output_shape())
            lib.set_tuning(NO_CL, flags)  # both on the row-form kernel
            try:
                if fused:
                    gdnn.conv2d_filter(X, Wt, Y, f, bias=bias, residual=R, activation="relu")
                else:
                    gdnn.conv2d_filter(X, Wt, Y, f, bias=bias)
                torch.cuda.synchronize()
            finally:
                lib.set_tuning(0, 0)
            assert bool((buf[:32] == 3.0).all()) and bool((buf[32 + n_out:] == 3.0).all())
            outs.append(Y.clone())
        for o in outs[1:]:
            assert torch.equal(outs[0], o)
    ref = oracle.conv2d(X.float().cpu().numpy(), Wt.float().cpu().numpy(), pads=(p,) * 4, strides=(s, s),
                        bias=bias.float().cpu().numpy(), wide=True)
    lib.set_tuning(0, 128 << 16)
    try:
        Y = torch.empty(f.output_shape(), dtype=dtype, device="cuda")
        gdnn.conv2d_filter(X, Wt, Y, f, bias=bias)
    finally:
        lib.set_tuning(0, 0)
    assert max_rel(Y.float().cpu().numpy(), ref) <= HALF_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_conv2d_pointwise_table_lookup_matches_affine(lib, dtype):
    """1x1 filters without padding address the image affinely in k; the table lookup used for
    every other filter must give the same bits."""
    from dlf_b200 import gdnn
    for case in (CONV_CASES[2], CONV_CASES[5], CONV_CASES[15]):
        N, C, H, W, Co, KH, KW, pads, strides, dil, group = case
        rng = np.random.default_rng(11)
        X = torch.from_numpy(rng.normal(size=(N, C, H, W)).astype(np.float32)).to(dtype).cuda()
        Wt = torch.from_numpy((0.1 * rng.normal(size=(Co, C // group, KH, KW))).astype(np.float32)).to(dtype).cuda()
        filt = gdnn.Filter2D(X.shape, Wt.shape, group).pads(*pads).strides(*strides).dilations(*dil)
        outs = []
        for flags in (0, 0x2000):
            lib.set_tuning(NO_CL, flags)  # both on the gathering kernel
            try:
                Y = torch.full(filt.output_shape(), float("nan"), dtype=dtype, device="cuda")
                gdnn.conv2d_filter(X, Wt, Y, filt)
                outs.append(Y.cpu())
            finally:
                lib.set_tuning(0, 0)
        assert torch.equal(outs[0], outs[1]), case


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", [
    (3, 64, 14, 14, 136, 3, 1, 1),   # 196-pixel planes: vectors of 4
    (3, 64, 9, 10, 72, 3, 1, 1),     # 90-pixel planes: vectors of 2
    (2, 64, 12, 12, 300, 1, 1, 0),   # 1x1, 144-pixel planes take the batched-GEMM route (not swapped)
    (5, 32, 10, 10, 64, 1, 2, 0),    # 1x1 stride 2: 25-pixel planes, odd: never swapped
    (2, 96, 16, 12, 40, 3, 1, 1),    # 192-pixel planes: vectors of 8, two images in one 256-pixel tile
], ids=lambda c: "x".join(map(str, c)))
def test_conv2d_swapped_roles_every_vector_width(lib, case, dtype):
    """The channels-last route with the roles swapped (lanes = output channels, columns = pixels,
    each lane storing vectors of consecutive pixels) is the default only for planes of a multiple of
    8 pixels; bit 17 of the tile-width word turns it on for vectors of 4 and 2 as well. All of them against
    the oracle, with a residual and ReLU, and nothing outside Y touched."""
    from dlf_b200 import gdnn
    N, C, H, W, Co, k, s, p = case
    rng = np.random.default_rng(sum(case))
    Xh = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
    Wh = _round_to((np.sqrt(2.0 / (C * k * k)) * rng.normal(size=(Co, C, k, k))).astype(np.float32), dtype)
    bh = _round_to(rng.uniform(-0.1, 0.1, Co).astype(np.float32), dtype)
    X, Wt, b = (torch.from_numpy(a).to(dtype).cuda() for a in (Xh, Wh, bh))
    f = gdnn.Filter2D(X.shape, Wt.shape).pads(p, p).strides(s, s)
    Rh = _round_to(rng.normal(size=tuple(f.output_shape())).astype(np.float32), dtype)
    R = torch.from_numpy(Rh).to(dtype).cuda()
    n_out = int(np.prod(f.output_shape()))
    ref = oracle.conv2d_fused(Xh, Wh, residual=Rh, relu=True, bias=bh, pads=(p,) * 4, strides=(s, s), wide=True)
    for route in (0, 0x20000):
        buf = torch.full((n_out + 64,), 3.0, dtype=dtype, device="cuda")
        Y = buf[32:32 + n_out].view(f.output_shape())
        lib.set_tuning(route, 0)
        try:
            gdnn.conv2d_filter(X, Wt, Y, f, bias=b, residual=R, activation="relu")
            torch.cuda.synchronize()
        finally:
            lib.set_tuning(0, 0)
        assert bool((buf[:32] == 3.0).all()) and bool((buf[32 + n_out:] == 3.0).all())
        assert max_rel(Y.float().cpu().numpy(), ref) <= HALF_TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", [(3, 64, 8, 16, 136), (2, 72, 28, 28, 520), (5, 128, 5, 8, 128), (2, 64, 12, 12, 200),
                                  (3, 64, 8, 16, 64), (2, 32, 16, 16, 72)],  # idle lane quadrants: skipped whole or in part
                         ids=lambda c: "x".join(map(str, c)))
def test_conv2d_pointwise_batched_gemm_both_orientations(lib, case, dtype):
    """A 1x1 stride-1 convolution on 16-byte-aligned planes is a batched GEMM over the images; with
    64 output channels or more it runs with the roles swapped (lanes = output channels, TMA stores
    of [channel][pixel] boxes; planes that are not a multiple of 32 pixels end in a box clipped by
    the hardware or in per-lane stores). Both orientations against the oracle, with residual and
    ReLU, nothing outside Y touched."""
    from dlf_b200 import gdnn
    N, C, H, W, Co = case
    rng = np.random.default_rng(sum(case))
    Xh = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
    Wh = _round_to((np.sqrt(2.0 / C) * rng.normal(size=(Co, C, 1, 1))).astype(np.float32), dtype)
    bh = _round_to(rng.uniform(-0.1, 0.1, Co).astype(np.float32), dtype)
    X, Wt, b = (torch.from_numpy(a).to(dtype).cuda() for a in (Xh, Wh, bh))
    f = gdnn.Filter2D(X.shape, Wt.shape)
    Rh = _round_to(rng.normal(size=tuple(f.output_shape())).astype(np.float32), dtype)
    R = torch.from_numpy(Rh).to(dtype).cuda()
    n_out = int(np.prod(f.output_shape()))
    ref = oracle.conv2d_fused(Xh, Wh, residual=Rh, relu=True, bias=bh, wide=True)
    for route in (0, 0x80000):
        buf = torch.full((n_out + 64,), 3.0, dtype=dtype, device="cuda")
        Y = buf[32:32 + n_out].view(f.output_shape())
        lib.set_tuning(route, 0)
        try:
            gdnn.conv2d_filter(X, Wt, Y, f, bias=b, residual=R, activation="relu")
            torch.cuda.synchronize()
        finally:
            lib.set_tuning(0, 0)
        assert bool((buf[:32] == 3.0).all()) and bool((buf[32 + n_out:] == 3.0).all())
        assert max_rel(Y.float().cpu().numpy(), ref) <= HALF_TOL


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", [
    (2, 64, 16, 16, 64, 3, 3, 1),     # the default case of this kernel: <= 64 output channels, rows of 8k outputs
    (2, 64, 56, 56, 48, 3, 3, 1),     # 56x56: tiles of 4 rows, two tiles of weights unused
    (3, 128, 28, 28, 128, 3, 3, 1),   # two 64-channel blocks per tile, 7 rows per tile
    (5, 256, 14, 14, 300, 3, 3, 1),   # four blocks, three tiles of output channels, the last one ragged
    (2, 64, 18, 18, 200, 3, 3, 1),    # rows of 18 outputs: per-lane vector stores instead of TMA boxes
    (3, 64, 10, 10, 72, 3, 3, 0),     # no padding: 8x8 outputs, the bordered copy has no border
    (2, 64, 30, 30, 64, 5, 5, 2),     # 5x5
    (1, 64, 70, 70, 136, 7, 7, 3),    # 7x7, 70 outputs per row: 3 rows per tile, ragged last tile
    (2, 128, 9, 12, 40, 3, 5, 1),     # KH != KW, output narrower than the input
], ids=lambda c: "x".join(map(str, c)))
def test_conv2d_halo_tile_kernel(lib, case, dtype):
    """Stride-1 filters larger than 1x1 over a multiple of 64 channels can run on the halo-tile kernel
    (bordered channel-group-major copy, a tile's rows fetched once, the filter taps as descriptor
    offsets into them). It is the default with at most 64 output channels and rows of a multiple of 8
    outputs; bit 24 of the tile-width word takes it wherever it can serve, bit 23 never. Both against
    the oracle with bias, residual and ReLU; nothing outside Y touched; the two routes agree to
    rounding of the 16-bit output."""
    from dlf_b200 import gdnn
    N, C, H, W, Co, kh, kw, p = case
    rng = np.random.default_rng(sum(case))
    Xh = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
    Wh = _round_to((np.sqrt(2.0 / (C * kh * kw)) * rng.normal(size=(Co, C, kh, kw))).astype(np.float32), dtype)
    bh = _round_to(rng.uniform(-0.1, 0.1, Co).astype(np.float32), dtype)
    X, Wt, b = (torch.from_numpy(a).to(dtype).cuda() for a in (Xh, Wh, bh))
    f = gdnn.Filter2D(X.shape, Wt.shape).pads(p, p)
    Rh = _round_to(rng.normal(size=tuple(f.output_shape())).astype(np.float32), dtype)
    R = torch.from_numpy(Rh).to(dtype).cuda()
    n_out = int(np.prod(f.output_shape()))
    ref = oracle.conv2d_fused(Xh, Wh, residual=Rh, relu=True, bias=bh, pads=(p,) * 4, wide=True)
    for route in (0x1000000, 0x800000):
        buf = torch.full((n_out + 64,), 3.0, dtype=dtype, device="cuda")
        Y = buf[32:32 + n_out].view(f.output_shape())
        lib.set_tuning(route, 0)
        try:
            gdnn.conv2d_filter(X, Wt, Y, f, bias=b, residual=R, activation="relu")
            torch.cuda.synchronize()
        finally:
            lib.set_tuning(0, 0)
        assert bool((buf[:32] == 3.0).all()) and bool((buf[32 + n_out:] == 3.0).all())
        assert max_rel(Y.float().cpu().numpy(), ref) <= HALF_TOL


FUSED_CASES = [
    CONV_CASES[0],    # row form 3x3
    CONV_CASES[3],    # 1x1 with aligned planes: TMA-fed GEMM route, TMA-store epilogue
    CONV_CASES[17],   # 1x1 14x14: affine gather, paired stores
    CONV_CASES[14],   # implicit im2col (dilation_w 2), chunked fp32
    CONV_CASES[7],    # groups, tiles straddle images
    CONV_CASES[18],   # strided row form
    (2, 32, 8, 16, 300, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1), 1),  # TMA route, ragged last column block
]


@pytest.fixture
def _route(lib, request):
    lib.set_tuning(request.param, 0)
    yield request.param
    lib.set_tuning(0, 0)


@pytest.mark.parametrize("dtype,_route", ROUTES, ids=ROUTE_IDS, indirect=["_route"])
@pytest.mark.parametrize("case", FUSED_CASES + [CONV_CASES[13], CONV_CASES[7][:10] + (1,)],
                         ids=lambda c: "x".join(map(str, c[:7])))
def test_conv2d_fused_residual_relu(lib, case, dtype, _route):
    """Y = relu(conv(X, W) + bias + R) in one launch, on every epilogue of the library, against
    the oracle's conv -> bias -> Add -> Relu chain; also each part alone, and R aliasing Y."""
    from dlf_b200 import gdnn
    N, C, H, W, Co, KH, KW, pads, strides, dil, group = case
    rng = np.random.default_rng(23)
    Xh = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
    Wh = _round_to((np.sqrt(2.0 / (C // group * KH * KW)) * rng.normal(size=(Co, C // group, KH, KW))).astype(np.float32), dtype)
    bh = _round_to(rng.uniform(-0.1, 0.1, Co).astype(np.float32), dtype)
    X, Wt, b = (torch.from_numpy(a).to(dtype).cuda() for a in (Xh, Wh, bh))
    filt = gdnn.Filter2D(X.shape, Wt.shape, group).pads(*pads).strides(*strides).dilations(*dil)
    Rh = _round_to(rng.normal(size=tuple(filt.output_shape())).astype(np.float32), dtype)
    R = torch.from_numpy(Rh).to(dtype).cuda()
    kw = dict(group=group, pads=pads, strides=strides, dilations=dil, wide=True)

    def check(got, ref):
        got = got.float().cpu().numpy()
        if dtype == torch.float32:
            assert rel_fro(got, ref) <= FP32_TOL
        else:
            assert max_rel(got, ref) <= HALF_TOL

    for use_bias, use_res, relu in ((True, True, True), (False, False, True), (False, True, False)):
        Y = torch.full(filt.output_shape(), float("nan"), dtype=dtype, device="cuda")
        gdnn.conv2d_filter(X, Wt, Y, filt, bias=b if use_bias else None, residual=R if use_res else None,
                           activation="relu" if relu else None)
        ref = oracle.conv2d_fused(Xh, Wh, residual=Rh if use_res else None, relu=relu,
                                  bias=bh if use_bias else None, **kw)
        check(Y, ref)
        if relu:
            assert float(Y.float().min()) >= 0.0
    # in place: Y holds the residual on entry
    Y = R.clone()
    gdnn.conv2d_filter(X, Wt, Y, filt, bias=b, residual=Y, activation="relu")
    check(Y, oracle.conv2d_fused(Xh, Wh, residual=Rh, relu=True, bias=bh, **kw))
    assert lib.device_status() == 0
    with pytest.raises(_gb().BLASError):
        gdnn.conv2d_filter(X, Wt, Y, filt, activation="gelu")


@pytest.mark.parametrize("path", [5, 0x8005, 0x8000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_conv2d_strided_row_form_variants(lib, path, dtype):
    """stride_w > 1 takes the row form with the input columns split into stride_w phases; path 5
    sends the same cases through the implicit-im2col gather instead, 0x8000 makes the loader
    warps gather the (phase-split) filter bank instead of streaming a packed copy."""
    from dlf_b200 import gdnn
    lib.set_tuning(0, path)
    try:
        for case in CONV_CASES[18:23] + [CONV_CASES[1]]:
            N, C, H, W, Co, KH, KW, pads, strides, dil, group = case
            rng = np.random.default_rng(17)
            X = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
            Wt = _round_to((0.1 * rng.normal(size=(Co, C // group, KH, KW))).astype(np.float32), dtype)
            ref = oracle.conv2d(X, Wt, group=group, pads=pads, strides=strides, dilations=dil, wide=True)
            filt = gdnn.Filter2D(X.shape, Wt.shape, group).pads(*pads).strides(*strides).dilations(*dil)
            Y = torch.full(ref.shape, float("nan"), dtype=dtype, device="cuda")
            gdnn.conv2d_filter(torch.from_numpy(X).to(dtype).cuda(), torch.from_numpy(Wt).to(dtype).cuda(), Y, filt)
            got = Y.float().cpu().numpy()
            if dtype == torch.float32:
                assert rel_fro(got, ref) <= FP32_TOL, case
            else:
                assert max_rel(got, ref) <= HALF_TOL, case
    finally:
        lib.set_tuning(0, 0)
    assert lib.device_status() == 0


@pytest.mark.parametrize("path", [2, 4, 0x8000, 0x8004])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_conv2d_every_kernel_variant(lib, path, dtype):
    """Convolutions normally take the row form (horizontal taps as GEMM columns) when stride_w =
    dilation_w = 1 and the plain implicit-im2col gather otherwise; the loader-warp kernel with
    both operands in shared memory is the fallback for very long K. Force each of the other two
    on cases the row form would take, and compare all of them with the oracle."""
    from dlf_b200 import gdnn
    lib.set_tuning(0, path)
    try:
        for case in (CONV_CASES[0], CONV_CASES[7], CONV_CASES[11]):
            N, C, H, W, Co, KH, KW, pads, strides, dil, group = case
            rng = np.random.default_rng(7)
            X = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
            Wt = _round_to((0.1 * rng.normal(size=(Co, C // group, KH, KW))).astype(np.float32), dtype)
            ref = oracle.conv2d(X, Wt, group=group, pads=pads, strides=strides, dilations=dil, wide=True)
            filt = gdnn.Filter2D(X.shape, Wt.shape, group).pads(*pads).strides(*strides).dilations(*dil)
            Y = torch.full(ref.shape, float("nan"), dtype=dtype, device="cuda")
            gdnn.conv2d_filter(torch.from_numpy(X).to(dtype).cuda(), torch.from_numpy(Wt).to(dtype).cuda(), Y, filt)
            got = Y.float().cpu().numpy()
            if dtype == torch.float32:
                assert rel_fro(got, ref) <= FP32_TOL, case
            else:
                assert max_rel(got, ref) <= HALF_TOL, case
    finally:
        lib.set_tuning(0, 0)


def test_conv2d_config2_full_size_properties():
    """BASELINE config 2 at its full size (N=64): every image against the oracle would take long
    on the CPU, so four images are checked element-wise and the whole batch through two
    size-independent properties: (i) images are independent (a permuted batch gives the permuted
    output, bit for bit), (ii) linearity in the weights."""
    from dlf_b200 import gdnn
    rng = np.random.default_rng(0)
    X = rng.normal(size=(64, 64, 56, 56)).astype(np.float32)
    Wt = (np.sqrt(2.0 / 576) * rng.normal(size=(64, 64, 3, 3))).astype(np.float32)
    bias = rng.uniform(-0.1, 0.1, 64).astype(np.float32)
    filt = gdnn.Filter2D(X.shape, Wt.shape).pads(1, 1)
    dX, dW, db = torch.from_numpy(X).cuda(), torch.from_numpy(Wt).cuda(), torch.from_numpy(bias).cuda()
    Y = torch.empty(filt.output_shape(), device="cuda")
    gdnn.conv2d_filter(dX, dW, Y, filt, bias=db)
    pick = [0, 17, 42, 63]
    ref = oracle.conv2d(X[pick], Wt, pads=(1, 1, 1, 1), bias=bias, wide=True)
    assert rel_fro(Y[pick].cpu().numpy(), ref) <= FP32_TOL
    perm = torch.randperm(64, generator=torch.Generator().manual_seed(1)).cuda()
    Yp = torch.empty_like(Y)
    gdnn.conv2d_filter(dX[perm].contiguous(), dW, Yp, filt, bias=db)
    assert torch.equal(Yp, Y[perm])
    Y2 = torch.empty_like(Y)
    gdnn.conv2d_filter(dX, (2.0 * dW).contiguous(), Y2, filt)  # exact scaling by 2, no bias
    Y1 = torch.empty_like(Y)
    gdnn.conv2d_filter(dX, dW, Y1, filt)
    assert torch.equal(Y2, 2.0 * Y1)


# ------------------------------------------------------------------------------------------
# errors, threads
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,flags", [(torch.float16, 0), (torch.float32, 0), (torch.float16, 3)],
                         ids=["tma-fed", "tensor-memory-operand-f32", "tensor-memory-operand-f16-staged-stores"])
def test_device_side_wait_runs_out_and_reports(lib, dtype, flags):
    """The bounded waits of the kernels, made to run out once without faulting anything: with the
    test aid 0x10000000 a single-tile launch withholds the commit that hands the accumulator to
    the epilogue and waits about a millisecond. The call returns, the device status reports the
    time-out exactly once, C keeps its old contents, and the next ordinary call is correct."""
    gb = _gb()
    m, n, k = 64, 64, 128  # one tile
    rng = np.random.default_rng(7)
    A = torch.from_numpy(_round_to(_rand(rng, m * k), dtype)).to(dtype).cuda()
    B = torch.from_numpy(_round_to(_rand(rng, k * n), dtype)).to(dtype).cuda()
    C = torch.full((m * n,), 5.0, dtype=dtype, device="cuda")
    assert lib.device_status() == 0
    lib.set_tuning(0, 0x10000000 | flags)
    try:
        gb.gemm(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, m, n, k, 1.0, A, 0, k, B, 0, n, 0.0,
                C, 0, n)
        torch.cuda.synchronize()
    finally:
        lib.set_tuning(0, flags)
    try:
        assert lib.device_status() == 1   # bit 0: a bounded wait gave up
        assert lib.device_status() == 0   # reported once
        assert bool((C == 5.0).all())     # the epilogue never ran
        gb.gemm(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, m, n, k, 1.0, A, 0, k, B, 0, n, 0.0,
                C, 0, n)
        torch.cuda.synchronize()
    finally:
        lib.set_tuning(0, 0)
    ref = (A.double().view(m, k) @ B.double().view(k, n)).flatten().cpu().numpy()
    got = C.double().cpu().numpy()
    assert (rel_fro(got, ref) <= FP32_TOL) if dtype == torch.float32 else (max_rel(got, ref) <= HALF_TOL)
    assert lib.device_status() == 0


def test_argument_errors_have_reference_status_codes():
    gb = _gb()
    a = torch.zeros(64, device="cuda")
    L, N = gb.Layout.RowMajor, gb.Transpose.NoTrans
    with pytest.raises(gb.BLASError) as e:
        gb.gemm(L, N, N, 0, 4, 4, 1.0, a, 0, 4, a, 0, 4, 0.0, a, 0, 4)
    assert e.value.status == gb.StatusCode.kInvalidDimension
    with pytest.raises(gb.BLASError) as e:
        gb.gemm(L, N, N, 4, 4, 4, 1.0, a, 0, 3, a, 0, 4, 0.0, a, 0, 4)
    assert e.value.status == gb.StatusCode.kInvalidLeadDimA
    with pytest.raises(gb.BLASError) as e:
        gb.gemm(L, N, N, 4, 4, 4, 1.0, a, 0, 4, a, 0, 4, 0.0, a, 60, 4)
    assert e.value.status == gb.StatusCode.kInsufficientMemoryC
    with pytest.raises(gb.BLASError) as e:
        gb.gemmStridedBatched(L, N, N, 4, 4, 4, 1.0, a, 0, 4, 16, a, 0, 4, 16, 0.0, a, 0, 4, 16, 0)
    assert e.value.status == gb.StatusCode.kInvalidBatchCount


def test_two_host_threads_each_with_its_own_queue():
    """Mirror of GPGPU.MultipleThreadContextActivation (dlf/test/GPGPUTest.cpp:716-733)."""
    gb = _gb()
    rng = np.random.default_rng(3)
    A, B = _rand(rng, 96 * 80), _rand(rng, 80 * 72)
    ref = np.zeros(96 * 72, np.float32)
    oracle.gblas_sgemm(oracle.ROW_MAJOR, oracle.NO_TRANS, oracle.NO_TRANS, 96, 72, 80, 1.0, A, 0,
                       80, B, 0, 72, 0.0, ref, 0, 72, wide=True)
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    results = [None, None]

    def work(i):
        s = torch.cuda.Stream()
        C = torch.zeros(96 * 72, device="cuda")
        for _ in range(20):
            gb.gemm(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, 96, 72, 80,
                    1.0, dA, 0, 80, dB, 0, 72, 0.0, C, 0, 72, queue=s)
        s.synchronize()
        results[i] = C.cpu().numpy()

    ts = [threading.Thread(target=work, args=(i,)) for i in range(2)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    for r in results:
        assert rel_fro(r, ref) <= FP32_TOL


def test_event_brackets_the_launch():
    gb = _gb()
    a = torch.randn(512 * 512, device="cuda")
    c = torch.empty(512 * 512, device="cuda")
    ev = gb.Event()
    gb.gemm(gb.Layout.RowMajor, gb.Transpose.NoTrans, gb.Transpose.NoTrans, 512, 512, 512, 1.0, a,
            0, 512, a, 0, 512, 0.0, c, 0, 512, event=ev)
    assert ev.elapsed_ms() > 0.0


# ---------------------------------------------------------------------------------------------
# pooling
# ---------------------------------------------------------------------------------------------
def _pool_filter(X_shape, cfg):
    from dlf_b200 import gdnn
    f = gdnn.Filter2D(X_shape, cfg["kernel"][0], cfg["kernel"][1])
    for name, arg in cfg["calls"]:
        getattr(f, name)(*arg) if isinstance(arg, list) else getattr(f, name)(arg)
    return f


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", G["pool"]["maxpool"], ids=lambda c: c["name"])
def test_maxpool_goldens_bit_exact(case, dtype):
    from dlf_b200 import gdnn
    X = tensor_of(case["X"]).to(dtype).cuda()
    f = _pool_filter(X.shape, case["filter"])
    Y = torch.full((f.batches, f.channels, f.output_h, f.output_w), float("nan"), dtype=dtype, device="cuda")
    gdnn.max_pooling(X, Y, f)
    assert torch.equal(Y.float().cpu(), tensor_of(case["R"]))


def test_global_pooling_golden_gpu():
    from dlf_b200 import gdnn
    g = G["pool"]["global"]
    X = tensor_of(g["X"]).cuda()
    Y = torch.empty(2, 3, 1, 1, device="cuda")
    gdnn.global_max_pooling(X, Y)
    assert Y.cpu().ravel().tolist() == g["max_R"]
    gdnn.global_average_pooling(X, Y)
    assert Y.cpu().ravel().tolist() == g["avg_R"]


POOL_CASES = [
    # N, C, H, W, KH, KW, pads(t,l,b,r), strides, dilations
    (2, 3, 100, 100, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),     # the reference's multi-channel test shape
    (3, 16, 112, 112, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1)),    # ResNet stem pool
    (2, 5, 13, 17, 2, 3, (0, 2, 1, 0), (2, 1), (1, 2)),       # odd everything, asymmetric pads, dilation
    (2, 4, 9, 9, 5, 5, (4, 4, 4, 4), (3, 3), (1, 1)),         # windows mostly in the padding
    (4, 7, 7, 7, 7, 7, (0, 0, 0, 0), (7, 7), (1, 1)),         # whole plane: one-warp-per-plane reduction
    (2, 3, 4, 5, 4, 5, (0, 0, 0, 0), (1, 1), (1, 1)),         # whole plane smaller than a warp
    (3, 14, 8, 24, 8, 24, (0, 0, 0, 0), (8, 24), (1, 1)),     # whole plane of 768 bytes in fp32: 64 planes fill the 48 KB of staging exactly
]


@pytest.mark.parametrize("flags", [0, 0x100 << 16], ids=["staged", "plain"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("case", POOL_CASES, ids=lambda c: "x".join(map(str, c[:6])))
def test_pooling_random_parity(lib, case, dtype, flags):
    """max: bit-exact for every type (a maximum of stored values); average: bit-exact in fp32 for
    windowed pooling (same order of additions as the reference), tolerance for 16-bit types and
    for the plane reduction (the reference's own reduction order is unspecified there)."""
    from dlf_b200 import gdnn
    N, C, H, W, KH, KW, pads, strides, dil = case
    lib.set_tuning(0, flags)
    try:
        _pooling_case(lib, case, dtype, flags)
    finally:
        lib.set_tuning(0, 0)


def _pooling_case(lib, case, dtype, flags):
    from dlf_b200 import gdnn
    N, C, H, W, KH, KW, pads, strides, dil = case
    rng = np.random.default_rng(31)
    Xh = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
    X = torch.from_numpy(Xh).to(dtype).cuda()
    f = gdnn.Filter2D(X.shape, KH, KW).pads(*pads).strides(*strides).dilations(*dil)
    shape = (N, C, f.output_h, f.output_w)
    Y = torch.full(shape, float("nan"), dtype=dtype, device="cuda")
    gdnn.max_pooling(X, Y, f)
    ref = oracle.pool2d(Xh, (KH, KW), "max", pads, strides, dil)
    assert np.array_equal(Y.float().cpu().numpy(), ref)
    whole = shape[2:] == (1, 1) and (KH, KW) == (H, W)
    for cip in (False, True):
        Y = torch.full(shape, float("nan"), dtype=dtype, device="cuda")
        gdnn.average_pooling(X, Y, f, cip)
        ref = oracle.pool2d(Xh, (KH, KW), "avg", pads, strides, dil, count_include_pad=cip)
        got = Y.float().cpu().numpy()
        if dtype == torch.float32 and not (whole and not flags):
            assert np.array_equal(got, ref, equal_nan=True)
        else:
            if dtype == torch.float32:
                assert rel_fro(got, ref) <= FP32_TOL
            else:
                assert max_rel(got, ref) <= HALF_TOL
    assert lib.device_status() == 0


def test_pooling_argument_errors(lib):
    from dlf_b200 import gdnn
    gb = _gb()
    X = torch.zeros(1, 1, 4, 4, device="cuda")
    Y = torch.zeros(1, 1, 1, 1, device="cuda")
    f = gdnn.Filter2D(X.shape, 2, 2)
    with pytest.raises(gb.BLASError):
        gdnn.max_pooling(X, Y, f)  # Y too small for the 3 x 3 output
    with pytest.raises(gb.BLASError):
        gdnn.max_pooling(X.half(), torch.zeros(1, 1, 3, 3, device="cuda"), f)  # mixed types


@pytest.mark.parametrize("shape", [
    # Cin, H, Cout, k, stride, pad: ResNet-50 layers that run on the tensor-memory-operand kernel
    (3, 224, 64, 7, 2, 3), (64, 56, 64, 3, 1, 1), (128, 28, 128, 3, 1, 1), (256, 14, 256, 3, 1, 1),
    (512, 7, 512, 3, 1, 1), (256, 14, 1024, 1, 1, 0), (1024, 14, 2048, 1, 2, 0), (2048, 7, 512, 1, 1, 0),
])
@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
def test_conv2d_workspace_bound_covers_the_packed_filter_bank(lib, shape, dtype):
    """dlf_b200_conv2d_workspace_bytes is an upper bound over the tilings the library may choose:
    with that much scratch the filter bank is packed (two launches per call: packing + main);
    with none the same call still works (one launch, loader warps gather the filter bank) and
    gives the same bits."""
    from dlf_b200 import gdnn
    cin, h, cout, k, s, p = shape
    X = torch.randn(2, cin, h, h, device="cuda").to(dtype)
    W = (torch.randn(cout, cin, k, k, device="cuda") * 0.05).to(dtype)
    f = gdnn.Filter2D(X.shape, W.shape).pads(p, p).strides(s, s)
    Y = torch.empty(f.output_shape(), device="cuda", dtype=dtype)
    lib.set_tuning(NO_CL, 0)  # the kernels that gather the activations themselves
    try:
        n0 = lib.launch_count()
        gdnn.conv2d_filter(X, W, Y, f)
        assert lib.launch_count() - n0 == 2
    finally:
        lib.set_tuning(0, 0)
    lib.set_tuning(0, 0x8000)
    try:
        Y2 = torch.empty_like(Y)
        n0 = lib.launch_count()
        gdnn.conv2d_filter(X, W, Y2, f)
        assert lib.launch_count() - n0 == 1
    finally:
        lib.set_tuning(0, 0)
    assert torch.equal(Y, Y2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
def test_conv2d_very_long_k_falls_back_to_shared_memory_operands(lib, dtype):
    """K = C*KH*KW = 12600 needs a 100 KB k table, more than the tensor-memory-operand kernel
    reserves: the call must take the loader-warp kernel with both operands in shared memory by
    itself (dilation_w = 2 keeps it off the row form) and still meet the tolerance."""
    from dlf_b200 import gdnn
    rng = np.random.default_rng(5)
    N, C, H, W, Co, KH, KW = 1, 1400, 6, 9, 24, 3, 3
    X = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
    Wt = _round_to((rng.normal(size=(Co, C, KH, KW)) / np.sqrt(C * KH * KW)).astype(np.float32), dtype)
    pads, strides, dil = (1, 2, 1, 2), (1, 1), (1, 2)
    ref = oracle.conv2d(X, Wt, pads=pads, strides=strides, dilations=dil, wide=True)
    f = gdnn.Filter2D(X.shape, Wt.shape).pads(*pads).strides(*strides).dilations(*dil)
    Y = torch.full(f.output_shape(), float("nan"), dtype=dtype, device="cuda")
    gdnn.conv2d_filter(torch.from_numpy(X).to(dtype).cuda(), torch.from_numpy(Wt).to(dtype).cuda(), Y, f)
    got = Y.float().cpu().numpy()
    if dtype == torch.float32:
        assert rel_fro(got, ref) <= FP32_TOL
    else:
        assert max_rel(got, ref) <= HALF_TOL
    assert lib.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("stride", [1, 2])
def test_conv2d_pointwise_with_very_many_channels(lib, dtype, stride):
    """A 1x1 filter over 13000 channels: K is beyond what a k table could hold, but affine
    addressing needs none, so the call stays on the tensor-memory-operand kernel (packing launch
    + one main launch) and, in fp32, keeps its K-chunked accumulation."""
    from dlf_b200 import gdnn
    rng = np.random.default_rng(9)
    N, C, H, W, Co = 2, 13000, 5, 6, 40
    X = _round_to(rng.normal(size=(N, C, H, W)).astype(np.float32), dtype)
    Wt = _round_to((rng.normal(size=(Co, C, 1, 1)) / np.sqrt(C)).astype(np.float32), dtype)
    ref = oracle.conv2d(X, Wt, strides=(stride, stride), wide=True)
    f = gdnn.Filter2D(X.shape, Wt.shape).strides(stride, stride)
    Y = torch.full(f.output_shape(), float("nan"), dtype=dtype, device="cuda")
    n0 = lib.launch_count()
    gdnn.conv2d_filter(torch.from_numpy(X).to(dtype).cuda(), torch.from_numpy(Wt).to(dtype).cuda(), Y, f)
    assert lib.launch_count() - n0 == 2
    got = Y.float().cpu().numpy()
    if dtype == torch.float32:
        assert rel_fro(got, ref) <= FP32_TOL
    else:
        assert max_rel(got, ref) <= HALF_TOL
    assert lib.device_status() == 0


# ------------------------------------------------------------------------------------------
# level-3 routines on the GEMM main loop: symm, syrk, trmm, trsm
# ------------------------------------------------------------------------------------------
def _l3_operand(spec, dtype):
    if spec.get("identity"):
        return torch.eye(spec["shape"][0], dtype=dtype)
    return tensor_of(spec, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", G["level3"]["symm"], ids=lambda c: c["side"] + c["triangle"])
def test_symm_goldens(case, dtype):
    """symm_test of dlf/test/GPGPUTest.cpp:307-351 through the front-end, bit-exact."""
    from dlf_b200 import tensor as dt
    gb = _gb()
    A, B = _l3_operand(case["A"], dtype).cuda(), _l3_operand(case["B"], dtype).cuda()
    got = dt.symm(gb.Side[case["side"]], gb.Triangle[case["triangle"]], A, B)
    assert torch.equal(got.cpu(), tensor_of(case["expected"], dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("case", G["level3"]["trmm"],
                         ids=lambda c: c["side"] + c["triangle"] + c["transpose"] + c["diagonal"])
def test_trmm_goldens_and_trsm_inverts_them(case, dtype):
    """trmm_test of dlf/test/GPGPUTest.cpp:361-470, bit-exact; trsm with the same arguments gives
    the identity back (fp32: the values are small integers, the solve is exact up to rounding)."""
    from dlf_b200 import tensor as dt
    gb = _gb()
    A, B = _l3_operand(case["A"], dtype).cuda(), _l3_operand(case["B"], dtype).cuda()
    args = (gb.Side[case["side"]], gb.Triangle[case["triangle"]], gb.Transpose[case["transpose"]],
            gb.Diagonal[case["diagonal"]])
    got = dt.trmm(*args, A, B)
    assert torch.equal(got.cpu(), tensor_of(case["expected"], dtype))
    if dtype == torch.float32:
        back = dt.trsm(*args, A, got)
        assert torch.allclose(back.cpu(), B.cpu(), atol=1e-5)


L3_SHAPES = [(5, 7), (64, 64), (100, 100), (130, 257), (300, 70)]


@pytest.mark.parametrize("layout", ["RowMajor", "ColMajor"])
@pytest.mark.parametrize("m,n", L3_SHAPES)
def test_symm_and_syrk_random_parity(lib, layout, m, n):
    """symm (both sides, both triangles) and syrk (both triangles, both transpositions) on seeded
    inputs with padded leading dimensions and element offsets, fp32, against the oracle; the
    triangle of C that syrk does not own must keep its values. Column-major calls are checked
    through the transposed row-major problem."""
    gb = _gb()
    rng = np.random.default_rng(m * 1000 + n)
    lay = gb.Layout[layout]
    row = layout == "RowMajor"
    for side in (gb.Side.Left, gb.Side.Right):
        for tri in (gb.Triangle.Upper, gb.Triangle.Lower):
            ka = m if side == gb.Side.Left else n
            lda, ldb, ldc = ka + 3, (n if row else m) + 2, (n if row else m) + 5
            A = _rand(rng, 7 + lda * ka)
            B = _rand(rng, 3 + ldb * (m if row else n))
            C0 = _rand(rng, 1 + ldc * (m if row else n))
            got = torch.from_numpy(C0.copy()).cuda()
            gb.symm(lay, side, tri, m, n, 0.75, torch.from_numpy(A).cuda(), 7, lda, torch.from_numpy(B).cuda(), 3, ldb,
                    -0.5, got, 1, ldc)
            ref = C0.copy()
            if row:
                oracle.symm(int(side), int(tri), m, n, 0.75, A[7:], lda, B[3:], ldb, -0.5, ref[1:], ldc, wide=True)
            else:  # C^T = B^T S (Left) / S B^T (Right), the other triangle of the row-major view of A
                oracle.symm(oracle.RIGHT if side == gb.Side.Left else oracle.LEFT,
                            oracle.LOWER if tri == gb.Triangle.Upper else oracle.UPPER, n, m, 0.75, A[7:], lda, B[3:],
                            ldb, -0.5, ref[1:], ldc, wide=True)
            assert rel_fro(got.cpu().numpy(), ref) <= FP32_TOL
    k = n
    for tri in (gb.Triangle.Upper, gb.Triangle.Lower):
        for ta in (gb.Transpose.NoTrans, gb.Transpose.Trans):
            a_rot = (row and ta == gb.Transpose.NoTrans) or (not row and ta != gb.Transpose.NoTrans)
            one, two = (k, m) if a_rot else (m, k)
            lda, ldc = one + 4, m + 3
            A = _rand(rng, 5 + lda * two)
            C0 = _rand(rng, 2 + ldc * m)
            got = torch.from_numpy(C0.copy()).cuda()
            gb.syrk(lay, tri, ta, m, k, 1.25, torch.from_numpy(A).cuda(), 5, lda, 0.5, got, 2, ldc)
            ref = C0.copy()
            if row:
                oracle.syrk(int(tri), int(ta), m, k, 1.25, A[5:], lda, 0.5, ref[2:], ldc, wide=True)
            else:
                oracle.syrk(oracle.LOWER if tri == gb.Triangle.Upper else oracle.UPPER,
                            oracle.TRANS if ta == gb.Transpose.NoTrans else oracle.NO_TRANS, m, k, 1.25, A[5:], lda,
                            0.5, ref[2:], ldc, wide=True)
            g = got.cpu().numpy()
            assert rel_fro(g, ref) <= FP32_TOL
            # outside the owned triangle nothing changed, bit for bit
            changed = g != C0
            idx = np.nonzero(changed)[0] - 2
            r, c = idx // ldc, idx % ldc
            owned_upper = (tri == gb.Triangle.Upper) == row
            assert np.all((c < m) & ((r <= c) if owned_upper else (r >= c)))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16])
@pytest.mark.parametrize("layout", ["RowMajor", "ColMajor"])
@pytest.mark.parametrize("m,n", L3_SHAPES)
def test_trmm_and_trsm_random_parity(lib, layout, m, n, dtype):
    """All sixteen (side, triangle, transposition, diagonal) forms of trmm and trsm on seeded
    inputs (padded leading dimensions, offsets) against the oracle; the triangle of A that the
    call does not name is filled with NaN and must never be read. trsm operands are made
    diagonally dominant so that the systems are well conditioned."""
    gb = _gb()
    rng = np.random.default_rng(m * 31 + n)
    lay = gb.Layout[layout]
    row = layout == "RowMajor"
    tol = FP32_TOL if dtype == torch.float32 else None
    for side in (gb.Side.Left, gb.Side.Right):
        ka = m if side == gb.Side.Left else n
        for tri in (gb.Triangle.Upper, gb.Triangle.Lower):
            for ta in (gb.Transpose.NoTrans, gb.Transpose.Trans):
                for diag in (gb.Diagonal.NonUnit, gb.Diagonal.Unit):
                    lda, ldb = ka + 2, (n if row else m) + 3
                    Am = (0.5 / np.sqrt(ka)) * rng.uniform(-1, 1, (ka, lda)).astype(np.float32)
                    Am[np.arange(ka), np.arange(ka)] = rng.uniform(1.0, 2.0, ka).astype(np.float32)
                    # the stored triangle in the layout's own view; everything else is poison
                    ii, jj = np.indices((ka, lda))
                    stored_upper = (tri == gb.Triangle.Upper) == row
                    keep = (jj < ka) & ((ii <= jj) if stored_upper else (ii >= jj))
                    if diag == gb.Diagonal.Unit:
                        keep &= ii != jj
                    Am = _round_to(Am, dtype)
                    A_clean = np.where(keep, Am, 0.0).astype(np.float32)
                    A_dev = np.where(keep, Am, np.nan).astype(np.float32)
                    B0 = _round_to(_rand(rng, 4 + ldb * (m if row else n)), dtype)
                    o_side = int(side) if row else (oracle.RIGHT if side == gb.Side.Left else oracle.LEFT)
                    o_tri = int(tri) if row else (oracle.LOWER if tri == gb.Triangle.Upper else oracle.UPPER)
                    om, on = (m, n) if row else (n, m)
                    for name in ("trmm", "trsm"):
                        got = torch.from_numpy(B0.copy()).to(dtype).cuda()
                        getattr(gb, name)(lay, side, tri, ta, diag, m, n, 0.5, torch.from_numpy(A_dev.ravel()).to(dtype).cuda(),
                                          0, lda, got, 4, ldb)
                        ref = B0.copy()
                        getattr(oracle, name)(o_side, o_tri, int(ta), int(diag), om, on, 0.5, A_clean.ravel(), lda,
                                              ref[4:], ldb, wide=True)
                        g = got.float().cpu().numpy()
                        assert np.isfinite(g).all(), (name, side, tri, ta, diag)
                        if dtype == torch.float32:
                            assert rel_fro(g, ref) <= tol, (name, side, tri, ta, diag)
                        else:
                            assert max_rel(g, ref) <= (HALF_TOL if name == "trmm" else 5e-2), (name, side, tri, ta, diag)


def test_level3_argument_errors(lib):
    gb = _gb()
    a = torch.zeros(64, device="cuda")
    with pytest.raises(gb.BLASError) as e:
        gb.symm(gb.Layout.RowMajor, gb.Side.Left, gb.Triangle.Upper, 4, 4, 1.0, a, 0, 3, a, 0, 4, 0.0, a, 0, 4)
    assert e.value.status == gb.StatusCode.kInvalidLeadDimA
    with pytest.raises(gb.BLASError) as e:
        gb.trsm(gb.Layout.RowMajor, gb.Side.Right, gb.Triangle.Upper, gb.Transpose.NoTrans, gb.Diagonal.Unit, 4, 0, 1.0,
                a, 0, 4, a, 0, 4)
    assert e.value.status == gb.StatusCode.kInvalidDimension
    with pytest.raises(gb.BLASError) as e:
        gb.syrk(gb.Layout.RowMajor, gb.Triangle.Lower, gb.Transpose.NoTrans, 8, 8, 1.0, a, 0, 8, 0.0, a, 1, 8)
    assert e.value.status == gb.StatusCode.kInsufficientMemoryC
