"""GPU parity of the channels-last operators (dlf_b200_conv2d_nhwc, dlf_b200_pool_nhwc,
dlf_b200_nchw_to_nhwc, dlf_b200_pack_filters_nhwc) against the CPU oracle: the oracle computes the
reference's NCHW function, the device result is permuted back before the comparison. 16-bit
tolerance as in the parity suite: 2e-2 maximum relative error; the copies and max pooling bit for bit."""
import numpy as np
import pytest
import torch

import oracle
from support import max_rel

pytestmark = pytest.mark.gpu
HALF_TOL = 2e-2


@pytest.fixture(scope="module")
def lib():
    import dlf_b200
    return dlf_b200


@pytest.fixture(autouse=True)
def _device_status_clean(lib):
    yield
    assert lib.device_status() == 0, "a device-side bounded wait timed out"


def _round_to(a, dtype):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dtype).float().numpy()


NHWC_CASES = [
    # N, C, H, W, Cout, KH, KW, pads (t, l, b, r), strides, dilations
    (2, 64, 14, 14, 64, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1)),      # 1x1 on 196-pixel planes: no TMA-friendly NCHW form exists
    (3, 64, 7, 7, 256, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1)),       # 49-pixel planes, widening
    (2, 128, 28, 28, 128, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),    # 3x3, two channel blocks
    (2, 256, 15, 15, 72, 1, 1, (0, 0, 0, 0), (2, 2), (1, 1)),     # strided 1x1, 72 output channels: the last box is clipped
    (2, 64, 17, 13, 200, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1)),     # 3x3 stride 2, odd sizes, two tiles of output channels
    (2, 24, 9, 11, 40, 5, 3, (2, 1, 2, 1), (1, 1), (1, 1)),       # 24 channels: the 64-channel k-block is zero-filled
    (1, 72, 12, 12, 136, 3, 3, (2, 2, 2, 2), (1, 1), (2, 2)),     # dilation 2, 72 channels (Ck = 128)
    (5, 64, 5, 5, 64, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),        # tiles straddle images
    (2, 64, 20, 20, 64, 7, 7, (3, 3, 3, 3), (2, 2), (1, 1)),      # 7x7 stride 2
    (3, 512, 7, 7, 2048, 1, 1, (0, 0, 0, 0), (1, 1), (1, 1)),     # ResNet-50's last widening layer
    (3, 64, 9, 9, 96, 3, 3, (1, 1, 1, 1), (1, 1), (1, 1)),        # 96 output channels, 3x3: filter bank as operand A, bias per row, idle lanes
    (2, 128, 14, 14, 128, 3, 3, (1, 1, 1, 1), (2, 2), (1, 1)),    # the same form with stride 2
]


@pytest.mark.parametrize("y_layout", ["nhwc", "nchw"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
@pytest.mark.parametrize("case", NHWC_CASES, ids=lambda c: "x".join(map(str, c[:7])))
def test_conv2d_nhwc_fused_against_the_oracle(lib, case, dtype, y_layout):
    """Bias + residual + ReLU, channels-last input, both output layouts; a guard band around Y."""
    from dlf_b200 import gdnn
    N, C, H, W, Co, KH, KW, pads, strides, dil = case
    rng = np.random.default_rng(sum(case[:7]))
    Xh = _round_to(rng.normal(size=(N, C, H, W)), dtype)
    Wh = _round_to(np.sqrt(2.0 / (C * KH * KW)) * rng.normal(size=(Co, C, KH, KW)), dtype)
    bh = _round_to(rng.uniform(-0.1, 0.1, Co), dtype)
    f = gdnn.Filter2D(Xh.shape, Wh.shape).pads(*pads).strides(*strides).dilations(*dil)
    assert gdnn.nhwc_supported(f, dtype, gdnn.NHWC if y_layout == "nhwc" else gdnn.NCHW)
    oshape = tuple(f.output_shape())
    Rh = _round_to(rng.normal(size=oshape), dtype)
    ref = oracle.conv2d_fused(Xh, Wh, residual=Rh, relu=True, bias=bh, pads=pads, strides=strides, dilations=dil, wide=True)
    X = torch.from_numpy(Xh).to(dtype).cuda()
    Xn = gdnn.nchw_to_nhwc(X)
    assert torch.equal(Xn, X.permute(0, 2, 3, 1).contiguous())
    Wp = gdnn.pack_filters_nhwc(torch.from_numpy(Wh).to(dtype).cuda())
    b = torch.from_numpy(bh).to(dtype).cuda()
    R = torch.from_numpy(Rh).to(dtype).cuda()
    n_out = int(np.prod(oshape))
    for with_residual in (True, False):
        buf = torch.full((n_out + 64,), 3.0, dtype=dtype, device="cuda")
        Y = buf[32:32 + n_out]
        if y_layout == "nhwc":
            Rl = R.permute(0, 2, 3, 1).contiguous()
            gdnn.conv2d_nhwc(Xn, Wp, Y, f, bias=b, residual=Rl if with_residual else None, activation="relu")
            got = Y.view(oshape[0], oshape[2], oshape[3], oshape[1]).permute(0, 3, 1, 2)
        else:
            gdnn.conv2d_nhwc(Xn, Wp, Y, f, bias=b, residual=R if with_residual else None, activation="relu",
                             y_layout=gdnn.NCHW)
            got = Y.view(oshape)
        torch.cuda.synchronize()
        assert bool((buf[:32] == 3.0).all()) and bool((buf[32 + n_out:] == 3.0).all())
        want = ref if with_residual else oracle.conv2d_fused(Xh, Wh, relu=True, bias=bh, pads=pads, strides=strides,
                                                             dilations=dil, wide=True)
        assert max_rel(got.float().cpu().numpy(), want) <= HALF_TOL


def test_conv2d_nhwc_refuses_what_the_tensor_map_unit_cannot_address(lib):
    from dlf_b200 import gblas, gdnn
    X = torch.zeros((1, 8, 8, 12), dtype=torch.float16, device="cuda")   # 12 channels: pixels of 24 bytes
    W = torch.zeros(lib.lib().dlf_b200_nhwc_filter_elems(12, 16, 3, 3), dtype=torch.float16, device="cuda")
    f = gdnn.Filter2D((1, 12, 8, 8), (16, 12, 3, 3)).pads(1, 1)
    assert not gdnn.nhwc_supported(f, torch.float16)
    Y = torch.zeros((1, 8, 8, 16), dtype=torch.float16, device="cuda")
    before = lib.launch_count()
    with pytest.raises(gblas.BLASError) as e:
        gdnn.conv2d_nhwc(X, W, Y, f)
    assert e.value.status == gblas.StatusCode.kNotImplemented and lib.launch_count() == before


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
@pytest.mark.parametrize("shape", [(2, 6, 5, 7), (3, 64, 14, 14), (2, 20, 8, 8), (1, 3, 9, 9)], ids=lambda s: "x".join(map(str, s)))
def test_nchw_to_nhwc_is_the_permutation_with_zero_filled_channels(lib, shape, dtype):
    from dlf_b200 import gdnn
    X = torch.randn(shape, device="cuda").to(dtype)
    Y = gdnn.nchw_to_nhwc(X)
    cp = (shape[1] + 7) // 8 * 8
    assert tuple(Y.shape) == (shape[0], shape[2], shape[3], cp)
    assert torch.equal(Y[..., :shape[1]], X.permute(0, 2, 3, 1))
    assert bool((Y[..., shape[1]:] == 0).all())


POOL_CASES = [
    # N, C, H, W, kernel, strides, pads (t, l, b, r), average, count_include_pad
    (2, 64, 18, 18, (3, 3), (2, 2), (1, 1, 1, 1), False, False),   # the ResNet stem pool
    (3, 16, 9, 11, (2, 3), (1, 2), (0, 1, 1, 1), False, False),
    (2, 32, 8, 8, (2, 2), (2, 2), (0, 0, 0, 0), True, False),
    (2, 24, 7, 9, (3, 3), (2, 2), (1, 1, 1, 1), True, True),
    (2, 24, 7, 9, (3, 3), (2, 2), (1, 1, 1, 1), True, False),
    (4, 128, 7, 7, (7, 7), (7, 7), (0, 0, 0, 0), True, False),     # global average pool
]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16], ids=["f16", "bf16"])
@pytest.mark.parametrize("case", POOL_CASES, ids=lambda c: "x".join(map(str, c[:4])) + ("avg" if c[7] else "max"))
def test_pool_nhwc_against_the_oracle(lib, case, dtype):
    from dlf_b200 import gdnn
    N, C, H, W, kernel, strides, pads, average, cip = case
    rng = np.random.default_rng(N + C + H + W)
    Xh = _round_to(rng.normal(size=(N, C, H, W)), dtype)
    ref = oracle.pool2d(Xh, kernel, "avg" if average else "max", pads, strides, count_include_pad=cip)
    f = gdnn.Filter2D(Xh.shape, kernel[0], kernel[1]).pads(*pads).strides(*strides)
    Xn = torch.from_numpy(Xh).to(dtype).cuda().permute(0, 2, 3, 1).contiguous()
    osh = tuple(f.output_shape())
    Y = torch.empty((osh[0], osh[2], osh[3], osh[1]), dtype=dtype, device="cuda")
    gdnn.pool_nhwc(Xn, Y, f, average=average, count_include_pad=cip)
    got = Y.permute(0, 3, 1, 2).float().cpu().numpy()
    if average:
        assert max_rel(got, ref) <= HALF_TOL
    else:
        np.testing.assert_array_equal(got, ref)
