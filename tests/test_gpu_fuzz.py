"""Seeded random sweep over small convolution / pooling / GEMM problems against the oracle: shapes,
pads, strides, dilations, groups, storage orders and epilogue options drawn at random, so that the
corner combinations no hand-written case lists (table padding vs stage count, windows wholly in the
padding, single-row images, ...) are visited."""
import numpy as np
import pytest
import torch

import oracle
from support import max_rel, rel_fro

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
HALF_TOL = 2e-2
DTYPES = [torch.float32, torch.float16, torch.bfloat16]


def _rt(a, dt):
    return torch.from_numpy(a).to(dt).float().numpy()


def _close(got, ref, dt):
    if not np.isfinite(got).all():
        return False
    if np.abs(ref).max() == 0:
        return np.abs(got).max() == 0
    return rel_fro(got, ref) <= FP32_TOL if dt == torch.float32 else max_rel(got, ref) <= HALF_TOL


@pytest.mark.parametrize("seed", range(4))
def test_random_convolutions(seed):
    from dlf_b200 import gdnn
    rng = np.random.default_rng(100 + seed)
    for _ in range(120):
        dt = DTYPES[rng.integers(0, 3)]
        group = int(rng.choice([1, 1, 1, 2, 3, 4]))
        cg = int(rng.integers(1, 40))
        C, Co = cg * group, int(rng.integers(1, 50)) * group
        H, W = int(rng.integers(1, 30)), int(rng.integers(1, 40))
        KH, KW = int(rng.integers(1, 6)), int(rng.integers(1, 8))
        pads = tuple(int(x) for x in rng.integers(0, 4, 4))
        strides = (int(rng.integers(1, 4)), int(rng.integers(1, 5)))
        dil = (int(rng.integers(1, 3)), int(rng.integers(1, 3)))
        N = int(rng.integers(1, 5))
        relu, use_res, use_b = (bool(rng.integers(0, 2)) for _ in range(3))
        cfg = dict(N=N, C=C, H=H, W=W, Co=Co, KH=KH, KW=KW, pads=pads, strides=strides, dil=dil, group=group,
                   dt=str(dt), relu=relu, res=use_res, bias=use_b)
        X = _rt(rng.normal(size=(N, C, H, W)).astype(np.float32), dt)
        Wt = _rt((rng.normal(size=(Co, cg, KH, KW)) / np.sqrt(cg * KH * KW)).astype(np.float32), dt)
        b = _rt(rng.uniform(-0.1, 0.1, Co).astype(np.float32), dt)
        f = gdnn.Filter2D(X.shape, Wt.shape, group).pads(*pads).strides(*strides).dilations(*dil)
        R = _rt(rng.normal(size=tuple(f.output_shape())).astype(np.float32), dt)
        ref = oracle.conv2d_fused(X, Wt, residual=R if use_res else None, relu=relu, bias=b if use_b else None,
                                  group=group, pads=pads, strides=strides, dilations=dil, wide=True)
        Y = torch.full(f.output_shape(), float("nan"), dtype=dt, device="cuda")
        gdnn.conv2d_filter(torch.from_numpy(X).to(dt).cuda(), torch.from_numpy(Wt).to(dt).cuda(), Y, f,
                           bias=torch.from_numpy(b).to(dt).cuda() if use_b else None,
                           residual=torch.from_numpy(R).to(dt).cuda() if use_res else None,
                           activation="relu" if relu else None)
        assert _close(Y.float().cpu().numpy(), ref, dt), cfg


def _aligned_case(rng):
    """Shapes that reach the tensor-map-fed routes: channel counts in multiples of 8, 16-bit types,
    planes that are often multiples of 8 pixels."""
    dt = [torch.float16, torch.bfloat16][rng.integers(0, 2)]
    C = int(rng.choice([8, 16, 24, 32, 64, 64, 72, 128, 192]))
    Co = int(rng.choice([8, 16, 40, 64, 64, 72, 96, 128, 136, 256, 320]))
    k = int(rng.choice([1, 1, 3, 3, 5, 7]))
    H = int(rng.integers(max(1, k - 2), 34))
    W = int(rng.choice([4, 7, 8, 12, 14, 16, 20, 28, 30, 32, 33]))
    pad = int(rng.integers(0, k // 2 + 1))
    stride = int(rng.choice([1, 1, 1, 2]))
    if H + 2 * pad < k or W + 2 * pad < k:
        H, W = H + k, W + k
    N = int(rng.integers(1, 6))
    relu, use_res, use_b = (bool(rng.integers(0, 2)) for _ in range(3))
    return dt, N, C, H, W, Co, k, pad, stride, relu, use_res, use_b


@pytest.mark.parametrize("seed", range(3))
def test_random_aligned_convolutions_on_both_entries(seed):
    """The NCHW entry (whichever route it takes: channels-last copy + im2col-mode loads, swapped or
    pixel-per-lane, halo tiles, batched-GEMM form, residual boxes, wide boxes) and the channels-last
    entry with both output layouts, on the same random problems against the oracle."""
    from dlf_b200 import gdnn
    rng = np.random.default_rng(500 + seed)
    for _ in range(50):
        dt, N, C, H, W, Co, k, pad, stride, relu, use_res, use_b = _aligned_case(rng)
        cfg = dict(dt=str(dt), N=N, C=C, H=H, W=W, Co=Co, k=k, pad=pad, stride=stride, relu=relu, res=use_res, bias=use_b)
        X = _rt(rng.normal(size=(N, C, H, W)).astype(np.float32), dt)
        Wt = _rt((rng.normal(size=(Co, C, k, k)) / np.sqrt(C * k * k)).astype(np.float32), dt)
        b = _rt(rng.uniform(-0.1, 0.1, Co).astype(np.float32), dt)
        f = gdnn.Filter2D(X.shape, Wt.shape).pads(pad, pad).strides(stride, stride)
        osh = tuple(f.output_shape())
        R = _rt(rng.normal(size=osh).astype(np.float32), dt)
        ref = oracle.conv2d_fused(X, Wt, residual=R if use_res else None, relu=relu, bias=b if use_b else None,
                                  pads=(pad,) * 4, strides=(stride, stride), wide=True)
        dX, dW = torch.from_numpy(X).to(dt).cuda(), torch.from_numpy(Wt).to(dt).cuda()
        db = torch.from_numpy(b).to(dt).cuda() if use_b else None
        dR = torch.from_numpy(R).to(dt).cuda() if use_res else None
        act = "relu" if relu else None
        Y = torch.full(osh, float("nan"), dtype=dt, device="cuda")
        gdnn.conv2d_filter(dX, dW, Y, f, bias=db, residual=dR, activation=act)
        assert _close(Y.float().cpu().numpy(), ref, dt), ("nchw entry", cfg)
        assert gdnn.nhwc_supported(f, dt), cfg
        Xn, Wp = gdnn.nchw_to_nhwc(dX), gdnn.pack_filters_nhwc(dW)
        Yn = torch.full((osh[0], osh[2], osh[3], osh[1]), float("nan"), dtype=dt, device="cuda")
        gdnn.conv2d_nhwc(Xn, Wp, Yn, f, bias=db, residual=dR.permute(0, 2, 3, 1).contiguous() if use_res else None,
                         activation=act)
        assert _close(Yn.permute(0, 3, 1, 2).float().cpu().numpy(), ref, dt), ("channels-last entry", cfg)
        Y2 = torch.full(osh, float("nan"), dtype=dt, device="cuda")
        gdnn.conv2d_nhwc(Xn, Wp, Y2, f, bias=db, residual=dR, activation=act, y_layout=gdnn.NCHW)
        assert _close(Y2.float().cpu().numpy(), ref, dt), ("channels-last entry, NCHW output", cfg)


@pytest.mark.parametrize("seed", range(2))
def test_random_pooling(seed):
    from dlf_b200 import gdnn
    rng = np.random.default_rng(200 + seed)
    for _ in range(150):
        dt = DTYPES[rng.integers(0, 3)]
        N, C = int(rng.integers(1, 4)), int(rng.integers(1, 9))
        H, W = int(rng.integers(1, 40)), int(rng.integers(1, 60))
        KH, KW = int(rng.integers(1, min(H, 5) + 1)), int(rng.integers(1, min(W, 5) + 1))
        pads = tuple(int(x) for x in rng.integers(0, 3, 4))
        strides = (int(rng.integers(1, 4)), int(rng.integers(1, 4)))
        dil = (1, 1) if rng.integers(0, 2) else (int(rng.integers(1, 3)), int(rng.integers(1, 3)))
        mode = "max" if rng.integers(0, 2) else "avg"
        cip = bool(rng.integers(0, 2))
        cfg = dict(N=N, C=C, H=H, W=W, KH=KH, KW=KW, pads=pads, strides=strides, dil=dil, dt=str(dt), mode=mode, cip=cip)
        X = _rt(rng.normal(size=(N, C, H, W)).astype(np.float32), dt)
        f = gdnn.Filter2D(X.shape, KH, KW).pads(*pads).strides(*strides).dilations(*dil)
        ref = oracle.pool2d(X, (KH, KW), mode, pads, strides, dil, count_include_pad=cip)
        if not np.isfinite(ref).all() or (ref <= -3e38).any():
            continue  # a window wholly in the padding: lowest() / 0/0 in the reference
        Y = torch.full((N, C, f.output_h, f.output_w), float("nan"), dtype=dt, device="cuda")
        if mode == "max":
            gdnn.max_pooling(torch.from_numpy(X).to(dt).cuda(), Y, f)
            assert np.array_equal(Y.float().cpu().numpy(), ref), cfg
        else:
            gdnn.average_pooling(torch.from_numpy(X).to(dt).cuda(), Y, f, cip)
            assert _close(Y.float().cpu().numpy(), ref, dt), cfg


@pytest.mark.parametrize("seed", range(2))
def test_random_strided_batched_gemm(seed):
    from dlf_b200 import gblas
    rng = np.random.default_rng(300 + seed)
    T_, N_ = gblas.Transpose.Trans, gblas.Transpose.NoTrans
    for _ in range(120):
        dt = DTYPES[rng.integers(0, 3)]
        m, n, k = (int(x) for x in rng.integers(1, 300, 3))
        batch = int(rng.integers(1, 4))
        ta, tb = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        row = bool(rng.integers(0, 2))
        alpha, beta = float(rng.choice([1.0, 0.5, -2.0])), float(rng.choice([0.0, 0.0, 1.0, 0.5]))
        cfg = dict(m=m, n=n, k=k, batch=batch, ta=ta, tb=tb, row=row, alpha=alpha, beta=beta, dt=str(dt))
        A = _rt(rng.uniform(-1, 1, (batch, m, k)).astype(np.float32), dt)
        B = _rt(rng.uniform(-1, 1, (batch, k, n)).astype(np.float32), dt)
        Cm = _rt(rng.normal(size=(batch, m, n)).astype(np.float32), dt)
        ref = (alpha * np.einsum("bmk,bkn->bmn", A.astype(np.float64), B.astype(np.float64)) + beta * Cm).astype(np.float32)
        sa = A.transpose(0, 2, 1) if ta else A  # what a row-major caller stores
        sb = B.transpose(0, 2, 1) if tb else B
        sc = Cm
        if not row:  # a column-major caller stores the transposes
            sa, sb, sc = sa.transpose(0, 2, 1), sb.transpose(0, 2, 1), Cm.transpose(0, 2, 1)
        dA, dB, dC = (torch.from_numpy(np.ascontiguousarray(x)).to(dt).cuda().reshape(-1) for x in (sa, sb, sc))
        lda = (m if ta else k) if row else (k if ta else m)
        ldb = (k if tb else n) if row else (n if tb else k)
        ldc = n if row else m
        gblas.gemmStridedBatched(gblas.Layout.RowMajor if row else gblas.Layout.ColMajor, T_ if ta else N_,
                                 T_ if tb else N_, m, n, k, alpha, dA, 0, lda, m * k, dB, 0, ldb, k * n, beta, dC, 0,
                                 ldc, m * n, batch)
        got = dC.float().cpu().numpy().reshape(batch, *((m, n) if row else (n, m)))
        if not row:
            got = got.transpose(0, 2, 1)
        assert _close(got, ref, dt), cfg


@pytest.mark.parametrize("seed", range(2))
def test_random_aligned_batched_gemm_strided_and_through_tables(seed):
    """16-bit batched products whose bases, leading dimensions and strides are 16-byte multiples - the
    shapes that reach the tensor-map-fed kernel, its transposed form for short K, and, through
    gemmBatched with the batch entries in a shuffled order, the indexed batch coordinate."""
    from dlf_b200 import gblas as gb
    rng = np.random.default_rng(900 + seed)
    for _ in range(40):
        dt = [torch.float16, torch.bfloat16][rng.integers(0, 2)]
        m, n = int(rng.integers(1, 60)) * 8, int(rng.integers(1, 60)) * 8
        k = int(rng.choice([8, 16, 40, 64, 72, 128, 200, 256, 264, 512]))
        batch = int(rng.integers(1, 6))
        layout = [gb.Layout.RowMajor, gb.Layout.ColMajor][rng.integers(0, 2)]
        ta = [gb.Transpose.NoTrans, gb.Transpose.Trans][rng.integers(0, 2)]
        tb = [gb.Transpose.NoTrans, gb.Transpose.Trans][rng.integers(0, 2)]
        a1, a2, b1, b2, c1, c2 = gb._dims(layout, ta, tb, m, n, k)
        lda, ldb, ldc = (d + 8 * int(rng.integers(0, 2)) for d in (a1, b1, c1))
        sa = lda * a2 + 8 * int(rng.integers(0, 3))
        sb = 0 if rng.integers(0, 4) == 0 else ldb * b2 + 8 * int(rng.integers(0, 3))  # 0: one B for every product
        sc = ldc * c2 + 8 * int(rng.integers(0, 3))
        alpha, beta = float(rng.choice([1.0, 0.5, -2.0])), float(rng.choice([0.0, 0.0, 0.5]))
        tables = bool(rng.integers(0, 2))
        cfg = dict(dt=str(dt), m=m, n=n, k=k, batch=batch, layout=int(layout), ta=int(ta), tb=int(tb), lda=lda, ldb=ldb,
                   ldc=ldc, sa=sa, sb=sb, sc=sc, alpha=alpha, beta=beta, tables=tables)
        A = _rt(rng.uniform(-1, 1, sa * batch).astype(np.float32), dt)
        B = _rt(rng.uniform(-1, 1, max(sb, ldb * b2) * batch).astype(np.float32), dt)
        C = _rt(rng.normal(size=sc * batch).astype(np.float32), dt)
        ref = C.copy()
        oracle.gblas_sgemm_strided_batched(int(layout), int(ta), int(tb), m, n, k, alpha, A, 0, lda, sa, B, 0, ldb, sb,
                                           beta, ref, 0, ldc, sc, batch, wide=True)
        dA, dB, dC = (torch.from_numpy(x).to(dt).cuda() for x in (A, B, C))
        if tables:
            perm = [int(p) for p in rng.permutation(batch)]
            gb.gemmBatched(layout, ta, tb, m, n, k, [alpha] * batch, dA, [p * sa for p in perm], lda, dB,
                           [p * sb for p in perm], ldb, [beta] * batch, dC, [p * sc for p in perm], ldc, batch)
        else:
            gb.gemmStridedBatched(layout, ta, tb, m, n, k, alpha, dA, 0, lda, sa, dB, 0, ldb, sb, beta, dC, 0, ldc, sc, batch)
        assert _close(dC.float().cpu().numpy(), ref, dt), cfg
