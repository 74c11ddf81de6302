"""GPU parity of the two op families beside the linear path: per-group (INT4-style) quantization of a constant and
quantized_conv.  Codes, binary64 scales, dequantized values and int32 sums must equal the CPU oracle's bit for bit
(the oracle itself is pinned against the pure-Python port and the reference's known answers on the CPU side)."""
import numpy as np
import pytest

from gpu_util import Guarded

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    import mlfw_b200
    c = mlfw_b200.Context(0)
    yield c
    c.check_status()
    c.close()


@pytest.mark.parametrize("n,G,bits", [(1 << 20, 128, 4), (4096, 32, 4), (1000, 128, 4), (777, 16, 3), (513, 64, 8), (64, 7, 2),
                                      (5, 64, 4), (1 << 16, 1, 4), (300000, 100, 4)])
def test_per_group_codes_scales_and_values(ctx, orc, n, G, bits):
    rng = np.random.default_rng(n + G)
    x = (rng.standard_normal(n) * np.exp(rng.uniform(-3, 3, n))).astype(np.float32)
    if n > 8 * G:
        x[3] = np.nan; x[G:2 * G] = 0.0; x[2 * G + 1] = np.inf; x[5 * G:6 * G] = -2.5; x[7 * G] = np.float32(1e-42)
        # exact ties of x / scale: the group's largest magnitude is `bound`, so k + 0.5 is representable
        bound = 2 ** (bits - 1) - 1
        x[3 * G:4 * G] = 0.0
        x[3 * G] = bound
        if G >= 4:
            x[3 * G + 1], x[3 * G + 2], x[3 * G + 3] = 0.5, -0.5, -1.5
    groups = (n + G - 1) // G
    dx = Guarded(ctx, (n,), np.float32, x)
    dq = Guarded(ctx, (n,), np.int8)
    ds64 = Guarded(ctx, (groups,), np.float64)
    ds32 = Guarded(ctx, (groups,), np.float32)
    ctx.quantize_per_group(dx.ptr, n, G, bits, dq.ptr, ds64.ptr, ds32.ptr)
    ctx.sync()
    s_ref = orc.per_group_scales(x, G, bits)
    q_ref = orc.quantize_per_group(x, G, s_ref, bits)
    assert (ds64.download().view(np.uint64) == s_ref.view(np.uint64)).all()
    assert (ds32.download().view(np.uint32) == s_ref.astype(np.float32).view(np.uint32)).all()
    q = dq.download()
    assert (q == q_ref).all()
    if bits == 4 and n > 8 * G and G >= 4:
        assert list(q[3 * G:3 * G + 4]) == [7, 1, 0, -1]       # Math.round: ties toward +Infinity
    dy64 = Guarded(ctx, (n,), np.float64)
    dy32 = Guarded(ctx, (n,), np.float32)
    ctx.dequantize_per_group(dq.ptr, n, G, ds64.ptr, dy64.ptr, dy32.ptr)
    ctx.sync()
    y_ref = orc.dequantize_per_group(q_ref, G, s_ref)
    y64, y32 = dy64.download(), dy32.download()
    same = lambda a, b, ui: ((a.view(ui) == b.view(ui)) | (np.isnan(a) & np.isnan(b))).all()
    assert same(y64, y_ref, np.uint64)
    with np.errstate(over="ignore"):
        assert same(y32, y_ref.astype(np.float32), np.uint32)


def test_per_group_scales_only_and_bad_arguments(ctx, orc):
    import mlfw_b200
    x = np.linspace(-3, 5, 1000, dtype=np.float32)
    dx = Guarded(ctx, (1000,), np.float32, x)
    ds64 = Guarded(ctx, (8,), np.float64)
    ctx.quantize_per_group(dx.ptr, 1000, 128, 4, None, ds64.ptr, None)
    ctx.sync()
    assert (ds64.download() == orc.per_group_scales(x, 128, 4)).all()
    with pytest.raises(mlfw_b200.B200QError):
        ctx.quantize_per_group(dx.ptr, 1000, 128, 9, None, ds64.ptr, None)
    with pytest.raises(mlfw_b200.B200QError):
        ctx.quantize_per_group(dx.ptr, 1000, 0, 4, None, ds64.ptr, None)


CONV_CASES = [
    # N, C, H, W, O, KH, KW, strides, padding, dilation, groups, zp_in, zp_ker
    (2, 4, 7, 6, 6, 3, 3, (2, 1), ((1, 0), (2, 1)), (1, 2), 2, 3, -2),
    (1, 3, 8, 8, 5, 3, 3, (1, 1), ((1, 1), (1, 1)), (1, 1), 1, 0, 0),            # 27 taps: padded to 32, tensor cores
    (2, 16, 5, 5, 8, 1, 1, (1, 1), ((0, 0), (0, 0)), (1, 1), 1, 0, 0),           # pointwise
    (1, 6, 9, 7, 6, 2, 3, (2, 2), ((0, 1), (1, 0)), (2, 1), 6, -5, 7),           # depthwise, both zero-points
    (1, 2, 4, 4, 2, 4, 4, (1, 1), ((3, 3), (3, 3)), (1, 1), 1, 127, -128),       # extreme zero-points, mostly padding
    (3, 32, 14, 14, 48, 3, 3, (1, 1), ((1, 1), (1, 1)), (1, 1), 1, 0, 0),        # 288 taps, 588 outputs per channel
    (2, 32, 15, 13, 64, 3, 3, (2, 2), ((1, 1), (1, 1)), (1, 1), 4, 0, 0),        # groups on the tensor cores
    (1, 8, 6, 6, 4, 3, 3, (1, 1), ((0, 0), (0, 0)), (1, 1), 1, 0, 9),            # one zero-point: CUDA-core contraction
    (2, 64, 9, 9, 130, 5, 5, (1, 1), ((2, 2), (2, 2)), (1, 1), 1, 0, 0),         # 1600 taps, ragged channel count
    (3, 48, 11, 7, 40, 1, 1, (1, 1), ((0, 0), (0, 0)), (1, 1), 1, 0, 0),         # pointwise: channel-last input is the row matrix itself
    (2, 32, 8, 8, 16, 1, 1, (2, 2), ((0, 0), (0, 0)), (1, 1), 1, 0, 0),          # pointwise with a stride: gathered
    (2, 32, 10, 9, 24, 3, 2, (1, 2), ((1, 2), (0, 1)), (2, 1), 2, 0, 0),         # 16 channels per group: the 16-byte gather with groups
]


@pytest.mark.parametrize("layout", ["NCHW", "NHWC"])
@pytest.mark.parametrize("case", CONV_CASES)
def test_quantized_conv_equals_oracle(ctx, orc, case, layout):
    N, C, H, W, O, KH, KW, st, pad, dil, groups, zi, zk = case
    rng = np.random.default_rng(N * 100 + C + KH)
    x = rng.integers(-128, 128, (N, C, H, W), dtype=np.int8)
    k = rng.integers(-128, 128, (O, C // groups, KH, KW), dtype=np.int8)
    if layout == "NHWC":
        x, k = np.ascontiguousarray(x.transpose(0, 2, 3, 1)), np.ascontiguousarray(k.transpose(0, 2, 3, 1))
    ref = orc.quantized_conv2d(x, k, st, pad, dil, groups, zi, zk, layout)
    dx, dk = Guarded(ctx, x.shape, np.int8, x), Guarded(ctx, k.shape, np.int8, k)
    do = Guarded(ctx, ref.shape, np.int32)
    ctx.quantized_conv2d(dx.ptr, dk.ptr, (N, C, H, W), (O, KH, KW), do.ptr, st, pad, dil, groups, zi, zk, layout)
    ctx.sync()
    assert (do.download() == ref).all()


def test_quantized_conv_resnet_sized_layer_on_tensor_cores(ctx, orc):
    """A 3x3 layer of 64 -> 128 channels on 8 images of 56x56: 25088 gathered rows of 576 taps through the tcgen05 kernel."""
    N, C, H, W, O = 8, 64, 56, 56, 128
    rng = np.random.default_rng(7)
    x = rng.integers(-127, 128, (N, H, W, C), dtype=np.int8)
    k = rng.integers(-127, 128, (O, 3, 3, C), dtype=np.int8)
    ref = orc.quantized_conv2d(x, k, (1, 1), ((1, 1), (1, 1)), (1, 1), 1, 0, 0, "NHWC")
    dx, dk = Guarded(ctx, x.shape, np.int8, x), Guarded(ctx, k.shape, np.int8, k)
    do = Guarded(ctx, ref.shape, np.int32)
    launches0 = ctx.launch_count()
    ctx.quantized_conv2d(dx.ptr, dk.ptr, (N, C, H, W), (O, 3, 3), do.ptr, (1, 1), ((1, 1), (1, 1)), (1, 1), 1, 0, 0, "NHWC")
    ctx.sync()
    assert ctx.launch_count() - launches0 == 2            # gather + contraction, result written in place
    assert (do.download() == ref).all()


def test_quantized_conv_refuses_bad_geometry(ctx):
    import mlfw_b200
    dx, dk, do = Guarded(ctx, (64,), np.int8), Guarded(ctx, (64,), np.int8), Guarded(ctx, (64,), np.int32)
    with pytest.raises(mlfw_b200.B200QError):      # groups do not divide the channels
        ctx.quantized_conv2d(dx.ptr, dk.ptr, (1, 3, 4, 4), (4, 1, 1), do.ptr, groups=2)
    with pytest.raises(mlfw_b200.B200QError):      # kernel larger than the padded input
        ctx.quantized_conv2d(dx.ptr, dk.ptr, (1, 1, 2, 2), (1, 3, 3), do.ptr)
    with pytest.raises(mlfw_b200.B200QError):
        ctx.quantized_conv2d(dx.ptr, dk.ptr, (1, 1, 4, 4), (1, 1, 1), do.ptr, strides=(0, 1))
