"""GPU parity of Conv2d forward against the float64 CPU oracle, through the C ABI."""
from pathlib import Path

import numpy as np
import pytest

from cudeep_b200 import workloads

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
TF32_TOL = 5e-3
TF32_MODEL_TOL = 2e-5


def test_reference_known_answers(dev):
    # cuDeep tests/unit/test_kernels.cu:324-425
    x = np.arange(1, 17, dtype=np.float32).reshape(1, 1, 4, 4)
    y = dev.conv2d(x, np.ones((1, 1, 1, 1), np.float32), np.zeros(1, np.float32))
    assert np.max(np.abs(y - x)) < 1e-4
    ones = np.ones((1, 1, 3, 3), np.float32)
    assert abs(dev.conv2d(ones, ones)[0, 0, 0, 0] - 9) < 1e-4
    assert abs(dev.conv2d(ones, ones, np.array([10], np.float32))[0, 0, 0, 0] - 19) < 1e-4
    y = dev.conv2d(ones, ones, None, (1, 1), (1, 1))
    assert abs(y[0, 0, 1, 1] - 9) < 1e-4 and abs(y[0, 0, 0, 0] - 4) < 1e-4 and abs(y[0, 0, 0, 1] - 6) < 1e-4


def test_reference_layer_shapes(dev):
    # cuDeep tests/unit/test_layers.py:58-75
    rng = np.random.default_rng(0)
    y = dev.conv2d(rng.standard_normal((2, 3, 8, 8), dtype=np.float32),
                   rng.standard_normal((16, 3, 3, 3), dtype=np.float32), None, (1, 1), (1, 1))
    assert y.shape == (2, 16, 8, 8) and np.isfinite(y).all()
    y = dev.conv2d(rng.standard_normal((1, 1, 8, 8), dtype=np.float32),
                   rng.standard_normal((4, 1, 3, 3), dtype=np.float32))
    assert y.shape == (1, 4, 6, 6)
    y = dev.conv2d(rng.standard_normal((1, 3, 8, 8), dtype=np.float32),
                   rng.standard_normal((8, 3, 3, 3), dtype=np.float32), None, (2, 2), (1, 1))
    assert y.shape == (1, 8, 4, 4)


def test_golden_fixtures(dev, oracle):
    g = np.load(Path(__file__).resolve().parent / "golden" / "dense_golden.npz")
    for tag in ("p1", "s2", "k1", "k5"):
        sh, sw, ph, pw = (int(v) for v in g[f"conv_{tag}_meta"])
        y = dev.conv2d(g[f"conv_{tag}_x"], g[f"conv_{tag}_w"], g[f"conv_{tag}_bias"], (sh, sw), (ph, pw), act=1)
        assert oracle.rel_frobenius(y, g[f"conv_{tag}_y"]) <= FP32_TOL     # small shapes: strict FP32 path


@pytest.mark.parametrize("shape,oc,k,stride,padding", [
    ((1, 1, 5, 5), 1, (3, 3), (1, 1), (0, 0)),
    ((2, 3, 9, 11), 8, (3, 3), (2, 2), (1, 1)),
    ((1, 16, 12, 12), 8, (5, 3), (1, 2), (2, 0)),
    ((2, 64, 14, 14), 16, (3, 3), (2, 2), (1, 1)),      # fewer than 32 output channels: direct even with many inputs
    ((2, 64, 14, 14), 64, (3, 3), (2, 2), (3, 1)),      # padding as large as the filter: direct
])
def test_direct_path_shapes(dev, oracle, shape, oc, k, stride, padding):
    rng = np.random.default_rng(sum(shape) + oc)
    x = rng.standard_normal(shape, dtype=np.float32)
    w = rng.standard_normal((oc, shape[1], *k), dtype=np.float32) * np.float32(0.2)
    bias = rng.standard_normal(oc, dtype=np.float32)
    for act in (0, 1):
        got = dev.conv2d(x, w, bias, stride, padding, act=act)
        assert oracle.rel_frobenius(got, oracle.conv2d(x, w, bias, stride, padding, act=act)) <= FP32_TOL


@pytest.mark.parametrize("shape,oc,k,padding", [
    ((2, 32, 8, 8), 128, (3, 3), (1, 1)),        # one CTA per tile, box narrower than 256 pixels
    ((1, 64, 14, 14), 64, (3, 3), (1, 1)),       # fewer output channels than a tile has rows
    ((2, 48, 9, 13), 96, (3, 3), (1, 1)),        # odd width: padded pixel box, channel count not a multiple of 32
    ((1, 32, 56, 56), 128, (1, 1), (0, 0)),      # 1x1
    ((2, 32, 8, 8), 256, (3, 3), (1, 1)),        # CTA pair
    ((1, 64, 56, 56), 256, (3, 3), (1, 1)),      # C4's image size and filter, one image
    ((2, 40, 10, 12), 200, (5, 5), (2, 2)),      # 5x5, ragged channels on both sides
    ((1, 36, 20, 20), 160, (3, 3), (0, 0)),      # no padding: output smaller than input
    ((3, 6, 16, 16), 64, (3, 3), (1, 1)),        # few input channels: each tap's K block is mostly zero padding
    ((2, 3, 32, 32), 64, (3, 3), (1, 1)),        # a first layer: three channels, the fewest this path takes
    ((1, 4, 20, 20), 32, (5, 5), (2, 2)),        # four channels, 5 x 5
    ((2, 3, 17, 33), 64, (3, 8), (1, 3)),        # row-packed K blocks: 8 taps x 4 channel slots fill a block exactly
    ((2, 8, 16, 16), 64, (3, 4), (1, 2)),        # row-packed, eight channels per tap, even filter width
    ((1, 5, 14, 18), 256, (5, 3), (2, 1)),       # row-packed, five channels in eight slots, CTA pair, odd row count
    ((1, 16, 12, 12), 32, (2, 2), (0, 0)),       # row-packed, two taps of sixteen channels
    ((4, 1, 28, 28), 32, (5, 5), (2, 2)),        # row-packed, a single input channel
    ((2, 2, 20, 24), 64, (3, 3), (1, 1)),        # row-packed, two input channels
    ((2, 3, 9, 300), 64, (1, 7), (0, 3)),        # row-packed, a single filter row, rows wider than one tile
    ((1, 32, 6, 300), 64, (3, 3), (1, 1)),       # rows wider than one tile
    ((5, 64, 7, 7), 512, (3, 3), (1, 1)),        # 7 x 7 maps: four whole images per tile, CTA pairs, the last tile has one image
    ((6, 48, 4, 4), 64, (3, 3), (1, 1)),         # 4 x 4 maps: six images fill one tile
    ((9, 32, 5, 9), 160, (3, 3), (1, 1)),        # 5 x 9 maps, ragged output channels, odd image count
    ((7, 40, 9, 9), 64, (3, 3), (0, 0)),         # 7 x 7 outputs without padding
    ((2, 32, 12, 16), 160, (3, 3), (1, 1)),      # bulk-store tiles whose rows past OC = 160 must not reach image 1
    ((3, 32, 10, 8), 96, (3, 3), (1, 1)),        # bulk-store tiles taller than the image (rows past OH clipped)
    ((6, 256, 7, 7), 512, (3, 3), (1, 1)),       # few tiles, 72 K blocks: the reduction split four ways in a cluster of 8
    ((32, 192, 7, 7), 512, (3, 3), (1, 1)),      # 16 tiles of four images, 54 K blocks split two ways (clusters of 4)
    ((7, 160, 7, 7), 96, (3, 3), (1, 1)),        # one CTA per tile, split reduction, last tile partly empty
    ((16, 288, 4, 4), 128, (3, 3), (1, 1)),      # 4 x 4 maps (an even plane size: stored from registers), split reduction
    ((9, 64, 5, 5), 256, (3, 3), (1, 1)),        # 5 x 5 maps on a pair: taps share rows of 7 pixels, 6 stages unsplit, 9 images
    ((10, 288, 3, 3), 512, (3, 3), (1, 1)),      # 3 x 3 maps: 15 of 64 operand rows per image are pixels; 27 stages, unsplit
    ((5, 32, 7, 5), 160, (3, 3), (1, 1)),        # 7 x 5 maps, 160 channels (the second CTA's rows partly past OC), 3 stages
    ((8, 128, 9, 7), 256, (5, 3), (2, 1)),       # five filter rows over 9 x 7 maps: 63 operand rows per image, the most
])
@pytest.mark.parametrize("act", [0, 1])
def test_tensor_core_path_shapes(dev, oracle, shape, oc, k, padding, act):
    rng = np.random.default_rng(sum(shape) + oc + act)
    x = rng.standard_normal(shape, dtype=np.float32)
    w = rng.standard_normal((oc, shape[1], *k), dtype=np.float32) * np.float32(0.1)
    bias = rng.standard_normal(oc, dtype=np.float32)
    got = dev.conv2d(x, w, bias, (1, 1), padding, act=act)
    assert not np.isnan(got).any()
    exact = oracle.conv2d(x, w, bias, (1, 1), padding, act=act)
    model = oracle.conv2d(x, w, bias, (1, 1), padding, act=act, input_mode=oracle.INPUT_TF32_TRUNC)
    assert got.shape == exact.shape
    assert oracle.rel_frobenius(got, exact) <= TF32_TOL
    assert oracle.rel_frobenius(got, model) <= TF32_MODEL_TOL


@pytest.mark.parametrize("shape,oc,k,padding", [
    ((2, 64, 56, 56), 256, (3, 3), (1, 1)),      # C4's rows: 2 x 58 pixels per CTA, 240 accumulator columns
    ((1, 40, 29, 28), 160, (3, 3), (1, 1)),      # 29 rows in tiles of 8: the last tile is mostly past OH; 160 channels
    ((3, 32, 12, 64), 384, (3, 3), (1, 1)),      # 64-pixel rows: one row per CTA, two loads of 32 columns per row
    ((2, 36, 30, 26), 256, (5, 3), (2, 0)),      # five filter rows, no horizontal padding: 24-pixel rows
    ((2, 64, 26, 42), 256, (3, 3), (0, 1)),      # no vertical padding: 24 output rows of 40 pixels
    ((5, 100, 32, 32), 512, (3, 3), (1, 1)),     # channels padded 100 -> 128, 512 output channels: two tile rows
    ((2, 64, 56, 56), 64, (3, 3), (1, 1)),       # one CTA per tile: 4 rows x 58 pixels, half of the 128 MMA rows are channels
    ((3, 128, 28, 28), 128, (3, 3), (1, 1)),     # one CTA: 8 rows x 30 pixels = 240 columns
    ((1, 48, 33, 32), 96, (3, 3), (1, 1)),       # one CTA, 33 rows in tiles of 7, 96 channels
])
@pytest.mark.parametrize("act", [0, 2])
def test_rows_shared_by_the_taps_of_a_filter_row(dev, oracle, shape, oc, k, padding, act):
    """Stride-1 layers with three taps per filter row and whole output rows of 24-64 pixels on CTA pairs:
    one load of the input rows serves the three taps (shifted descriptors), rows leave by 3-D bulk
    stores.  Same bars as every tensor-core convolution, plus bitwise equality with a second run."""
    rng = np.random.default_rng(sum(shape) + oc + act)
    x = rng.standard_normal(shape, dtype=np.float32)
    w = rng.standard_normal((oc, shape[1], *k), dtype=np.float32) * np.float32(0.1)
    bias = rng.standard_normal(oc, dtype=np.float32)
    got = dev.conv2d(x, w, bias, (1, 1), padding, act=act)
    assert not np.isnan(got).any()
    exact = oracle.conv2d(x, w, bias, (1, 1), padding, act=act)
    model = oracle.conv2d(x, w, bias, (1, 1), padding, act=act, input_mode=oracle.INPUT_TF32_TRUNC)
    assert got.shape == exact.shape
    assert oracle.rel_frobenius(got, exact) <= TF32_TOL
    assert oracle.rel_frobenius(got, model) <= TF32_MODEL_TOL
    assert np.array_equal(got, dev.conv2d(x, w, bias, (1, 1), padding, act=act))


@pytest.mark.parametrize("shape,oc,k,stride,padding", [
    ((2, 64, 14, 14), 64, (3, 3), (2, 2), (1, 1)),       # 7 x 7 outputs, every second pixel in both directions
    ((2, 32, 28, 28), 128, (3, 3), (2, 2), (1, 1)),      # a ResNet down-sampling layer
    ((1, 3, 64, 64), 64, (7, 7), (2, 2), (3, 3)),        # a ResNet stem: 7 x 7, stride 2, three channels
    ((2, 3, 35, 37), 96, (7, 7), (2, 3), (3, 2)),        # the same with odd sizes and different strides
    ((2, 4, 30, 30), 64, (5, 5), (3, 3), (0, 0)),        # row-packed, stride 3, no padding
    ((2, 64, 16, 16), 256, (1, 1), (2, 2), (0, 0)),      # 1 x 1 stride 2 projection, CTA pair
    ((1, 32, 20, 33), 64, (3, 3), (1, 3), (1, 1)),       # different strides per direction, width not a multiple
    ((2, 40, 39, 39), 96, (5, 5), (4, 4), (2, 2)),       # stride 4
    ((4, 32, 14, 14), 64, (3, 3), (2, 2), (1, 1)),       # 7 x 7 outputs: several whole images per tile, walked in strides
    ((6, 32, 27, 27), 64, (3, 3), (2, 2), (1, 1)),       # 14 x 14 outputs: grad_weight reads two padded rows per K block
])
@pytest.mark.parametrize("act", [0, 1])
def test_strided_tensor_core_path_shapes(dev, lib, oracle, shape, oc, k, stride, padding, act):
    """Strided convolutions: the TMA box walks the NHWC input in steps of the stride."""
    rng = np.random.default_rng(sum(shape) + oc + act)
    x = rng.standard_normal(shape, dtype=np.float32)
    w = rng.standard_normal((oc, shape[1], *k), dtype=np.float32) * np.float32(0.1)
    bias = rng.standard_normal(oc, dtype=np.float32)
    got = dev.conv2d(x, w, bias, stride, padding, act=act)
    assert not np.isnan(got).any()
    exact = oracle.conv2d(x, w, bias, stride, padding, act=act)
    model = oracle.conv2d(x, w, bias, stride, padding, act=act, input_mode=oracle.INPUT_TF32_TRUNC)
    assert got.shape == exact.shape
    assert oracle.rel_frobenius(got, exact) <= TF32_TOL
    assert oracle.rel_frobenius(got, model) <= TF32_MODEL_TOL        # so the tensor cores did run
    if act == 0:
        dy = rng.standard_normal(exact.shape, dtype=np.float32)
        dx, dw = conv_backward(dev, lib, dy, w, x, stride, padding)
        dw_ref = oracle.conv2d_backward_weight_np(dy, x, k, stride, padding)
        assert oracle.rel_frobenius(dw, dw_ref) <= TF32_TOL
        # grad_input: grad_output with zeros between its pixels through the stride-1 implicit GEMM
        # (32 or more input channels), else the direct kernel.
        dx_ref = oracle.conv2d_backward_data_np(dy, w, shape[2:], stride, padding)
        assert dx.shape == x.shape and not np.isnan(dx).any()
        assert oracle.rel_frobenius(dx, dx_ref) <= TF32_TOL
        if shape[1] >= 32:
            model = oracle.conv2d_backward_data_np(dy, w, shape[2:], stride, padding,
                                                   input_mode=oracle.INPUT_TF32_TRUNC)
            assert oracle.rel_frobenius(dx, model) <= TF32_MODEL_TOL


@pytest.mark.parametrize("shape,oc,k,stride,padding", [
    ((2, 64, 56, 56), 128, (3, 3), (2, 2), (1, 1)),      # a down-sampling layer: classes of 4, 2, 2 and 1 taps
    ((2, 32, 15, 17), 64, (3, 3), (3, 3), (1, 1)),       # stride = filter: nine classes of one tap each
    ((2, 48, 20, 20), 64, (2, 2), (2, 2), (0, 0)),       # 2 x 2 stride 2, no padding
    ((2, 64, 16, 16), 96, (1, 1), (2, 2), (0, 0)),       # filter smaller than the stride: three classes get no gradient
    ((1, 32, 22, 23), 32, (3, 3), (2, 2), (0, 0)),       # the forward pass leaves the last row unread: zeros there
    ((1, 32, 21, 21), 40, (5, 5), (2, 2), (2, 2)),       # 5 x 5: classes of 3 x 3, 3 x 2, 2 x 3, 2 x 2 taps
    ((2, 32, 18, 30), 64, (3, 5), (1, 2), (1, 2)),       # stride 1 down, 2 across
    ((3, 32, 13, 13), 64, (4, 4), (3, 2), (1, 0)),       # different strides, even filter
    ((8, 64, 14, 14), 64, (3, 3), (2, 2), (1, 1)),       # 7 x 7 classes: several whole images per tile
    ((1, 40, 40, 40), 36, (7, 7), (4, 4), (3, 3)),       # stride 4: sixteen classes; 36 channels of grad_output
])
def test_strided_grad_input_by_parity_classes(dev, lib, oracle, shape, oc, k, stride, padding):
    """grad_input of a strided layer: one stride-1 convolution of grad_output per parity class of the input
    pixels, each writing every stride-th pixel.  Every pixel of grad_input must be written (the output starts
    as NaN), pixels no tap reaches must be zero, and the values follow the truncated-operand model."""
    rng = np.random.default_rng(sum(shape) + oc + sum(k))
    x = np.zeros(shape, dtype=np.float32)
    w = rng.standard_normal((oc, shape[1], *k), dtype=np.float32) * np.float32(0.1)
    oh = (shape[2] + 2 * padding[0] - k[0]) // stride[0] + 1
    ow = (shape[3] + 2 * padding[1] - k[1]) // stride[1] + 1
    dy = rng.standard_normal((shape[0], oc, oh, ow), dtype=np.float32)
    dx, _ = conv_backward(dev, lib, dy, w, x, stride, padding)
    assert dx.shape == x.shape and not np.isnan(dx).any()
    exact = oracle.conv2d_backward_data_np(dy, w, shape[2:], stride, padding)
    model = oracle.conv2d_backward_data_np(dy, w, shape[2:], stride, padding, input_mode=oracle.INPUT_TF32_TRUNC)
    assert oracle.rel_frobenius(dx, exact) <= TF32_TOL
    assert oracle.rel_frobenius(dx, model) <= TF32_MODEL_TOL
    assert np.all(dx[exact == 0.0] == 0.0)                   # untouched pixels are exactly zero
    again, _ = conv_backward(dev, lib, dy, w, x, stride, padding)
    assert np.array_equal(dx, again)


@pytest.mark.parametrize("shape,oc,k,stride,padding", [
    ((2, 64, 28, 28), 128, 3, 1, 1),       # single-image tiles, bulk tensor stores
    ((3, 36, 19, 23), 40, 3, 1, 1),        # ragged everything; channels padded to one K block
    ((4, 128, 7, 7), 256, 3, 1, 1),        # several images per tile
    ((2, 64, 30, 30), 96, 3, 2, 1),        # strided
    ((2, 256, 14, 14), 64, 1, 1, 0),       # 1 x 1
])
@pytest.mark.parametrize("act", [0, 1])
def test_nhwc_input_matches_the_nchw_call_bit_for_bit(dev, lib, oracle, shape, oc, k, stride, padding, act):
    """The channels-last entry reads its input in place; everything after the (skipped) re-layout is the
    same kernel on the same bytes, so the result equals the NCHW call's exactly - and the oracle's."""
    rng = np.random.default_rng(sum(shape) + oc + k)
    n, c, h, w_ = shape
    x = rng.standard_normal(shape, dtype=np.float32)
    w = (rng.standard_normal((oc, c, k, k), dtype=np.float32) * np.float32(0.1))
    bias = rng.uniform(-0.5, 0.5, oc).astype(np.float32)
    want = dev.conv2d(x, w, bias, (stride, stride), (padding, padding), act=act)
    tx = dev.to_dev(np.ascontiguousarray(x.transpose(0, 2, 3, 1)))          # [N, H, W, C]
    tw, tb = dev.to_dev(w), dev.to_dev(bias)
    ty = dev.empty(want.shape)
    dev.check(lib.cudeep_b200_conv2d_forward_fused_nhwc_f32(dev.ptr(tx), dev.ptr(tw), dev.ptr(tb), dev.ptr(ty), n, c,
                                                            oc, h, w_, k, k, stride, stride, padding, padding, act,
                                                            None))
    assert dev.sync_status() == 0
    got = ty.cpu().numpy()
    assert np.array_equal(got, want)
    assert oracle.rel_frobenius(got, oracle.conv2d(x, w, bias, (stride, stride), (padding, padding), act=act)) <= 5e-3


def test_nhwc_input_refuses_what_it_cannot_read_in_place(dev, lib):
    p = dev.ptr(dev.empty((64,)))
    # 6 channels: not a multiple of 4
    rc = lib.cudeep_b200_conv2d_forward_fused_nhwc_f32(p, p, None, p, 2, 6, 64, 16, 16, 3, 3, 1, 1, 1, 1, 0, None)
    assert rc != 0 and b"NHWC input needs" in lib.cudeep_b200_last_error()
    # 8 output channels: off the tensor-core path
    rc = lib.cudeep_b200_conv2d_forward_fused_nhwc_f32(p, p, None, p, 2, 64, 8, 16, 16, 3, 3, 1, 1, 1, 1, 0, None)
    assert rc != 0 and b"NHWC input needs" in lib.cudeep_b200_last_error()


def test_no_bias_and_bias_differ_by_bias(dev):
    rng = np.random.default_rng(3)
    x = rng.standard_normal((1, 32, 8, 8), dtype=np.float32)
    w = rng.standard_normal((64, 32, 3, 3), dtype=np.float32) * np.float32(0.1)
    bias = rng.standard_normal(64, dtype=np.float32)
    y0 = dev.conv2d(x, w, None, (1, 1), (1, 1))
    y1 = dev.conv2d(x, w, bias, (1, 1), (1, 1))
    assert np.allclose(y1 - y0, bias[None, :, None, None], atol=1e-5)


def test_c4_reduced_batch(dev, oracle):
    """C4's layer (256 -> 256, 3x3, 56x56, bias + ReLU) on 2 images; the oracle checks all of it."""
    x, w, bias = workloads.c4_conv(batch=2)
    got = dev.conv2d(x, w, bias, (1, 1), (1, 1), act=1)
    exact = oracle.conv2d(x, w, bias, (1, 1), (1, 1), act=1)
    model = oracle.conv2d(x, w, bias, (1, 1), (1, 1), act=1, input_mode=oracle.INPUT_TF32_TRUNC)
    assert oracle.rel_frobenius(got, exact) <= TF32_TOL
    assert oracle.rel_frobenius(got, model) <= TF32_MODEL_TOL
    k = 256 * 9
    pre = oracle.conv2d(x, w, bias, (1, 1), (1, 1))
    got_pre = dev.conv2d(x, w, bias, (1, 1), (1, 1))
    assert np.max(np.abs(got_pre - pre)) <= oracle.tf32_elementwise_bound(x, w, k)


def test_c4_full_batch_properties(dev, oracle):
    """C4 at full size (64 images): batch independence and a sampled check against the oracle."""
    x, w, bias = workloads.c4_conv()
    got = dev.conv2d(x, w, bias, (1, 1), (1, 1), act=1)
    assert got.shape == (64, 256, 56, 56) and not np.isnan(got).any()
    # images are independent: recomputing images 17 and 63 alone gives the same bits
    for i in (17, 63):
        alone = dev.conv2d(x[i:i + 1], w, bias, (1, 1), (1, 1), act=1)
        assert np.array_equal(alone[0], got[i])
    exact = oracle.conv2d(x[40:41], w, bias, (1, 1), (1, 1), act=1)
    assert oracle.rel_frobenius(got[40:41], exact) <= TF32_TOL


# ---- backward ---------------------------------------------------------------------------------

def conv_backward(dev, lib, dy, w, x, stride, padding):
    n, c, h, wd = x.shape
    oc, _, kh, kw = w.shape
    tdy, tw, tx = dev.to_dev(dy), dev.to_dev(w), dev.to_dev(x)
    dx, dw = dev.empty(x.shape), dev.empty(w.shape)
    args = (n, c, oc, h, wd, kh, kw, stride[0], stride[1], padding[0], padding[1], None)
    dev.check(lib.cudeep_b200_conv2d_backward_data_f32(dev.ptr(tdy), dev.ptr(tw), dev.ptr(dx), *args))
    dev.check(lib.cudeep_b200_conv2d_backward_weight_f32(dev.ptr(tdy), dev.ptr(tx), dev.ptr(dw), *args))
    assert dev.sync_status() == 0
    return dx.cpu().numpy(), dw.cpu().numpy()


def test_backward_reference_known_answers(dev, lib):
    # cuDeep tests/unit/test_advanced_kernels.cu:197-241
    ones = np.ones((1, 1, 3, 3), np.float32)
    dx, dw = conv_backward(dev, lib, ones, np.full((1, 1, 1, 1), 2.0, np.float32), ones, (1, 1), (0, 0))
    assert np.max(np.abs(dx - 2.0)) < 1e-4
    assert abs(dw[0, 0, 0, 0] - 9.0) < 1e-4


@pytest.mark.parametrize("shape,oc,k,stride,padding,tensor_core", [
    ((2, 3, 9, 11), 8, (3, 3), (2, 2), (1, 1), False),      # strided: direct kernels
    ((1, 5, 8, 8), 4, (3, 2), (1, 1), (0, 1), False),       # few channels: direct kernels
    ((2, 64, 14, 14), 96, (3, 3), (1, 1), (1, 1), True),    # grad_input on the implicit-GEMM path
    ((1, 160, 12, 20), 48, (5, 5), (1, 1), (2, 2), True),   # 5x5, more input than output channels
    ((2, 32, 10, 10), 64, (3, 3), (1, 1), (0, 0), True),    # no padding: full correlation with pad 2
    ((6, 64, 7, 7), 96, (3, 3), (1, 1), (1, 1), True),      # 7 x 7 maps: grad_input on tiles of several images
])
def test_backward_against_oracle(dev, lib, oracle, shape, oc, k, stride, padding, tensor_core):
    rng = np.random.default_rng(sum(shape) + oc)
    x = rng.standard_normal(shape, dtype=np.float32)
    w = rng.standard_normal((oc, shape[1], *k), dtype=np.float32) * np.float32(0.1)
    oh = (shape[2] + 2 * padding[0] - k[0]) // stride[0] + 1
    ow = (shape[3] + 2 * padding[1] - k[1]) // stride[1] + 1
    dy = rng.standard_normal((shape[0], oc, oh, ow), dtype=np.float32)
    dx, dw = conv_backward(dev, lib, dy, w, x, stride, padding)
    dx_ref = oracle.conv2d_backward_data_np(dy, w, shape[2:], stride, padding)
    dw_ref = oracle.conv2d_backward_weight_np(dy, x, k, stride, padding)
    wgrad_on_tensor_cores = oc >= 32 and shape[0] * oh * ow >= 256       # the launcher's rule (any row length)
    assert oracle.rel_frobenius(dw, dw_ref) <= (TF32_TOL if wgrad_on_tensor_cores else FP32_TOL)
    if tensor_core:
        assert oracle.rel_frobenius(dx, dx_ref) <= TF32_TOL
        model = oracle.conv2d_backward_data_np(dy, w, shape[2:], stride, padding, input_mode=oracle.INPUT_TF32_TRUNC)
        assert oracle.rel_frobenius(dx, model) <= TF32_MODEL_TOL
    else:
        assert oracle.rel_frobenius(dx, dx_ref) <= FP32_TOL


@pytest.mark.parametrize("shape,oc,k,padding", [
    ((4, 64, 28, 28), 64, (3, 3), (1, 1)),      # one CTA per tile; 28 of the 32 pixels of a K block are real
    ((2, 256, 56, 56), 256, (3, 3), (1, 1)),    # the C4 layer: CTA pairs, two K blocks per row, 256-channel tiles
    ((3, 48, 16, 24), 160, (3, 5), (1, 2)),     # 160 output channels: the second 128-row tile is partly empty
    ((2, 320, 12, 16), 256, (3, 3), (1, 1)),    # 320 channels: two tiles of 160 columns
    ((1, 16, 20, 20), 32, (1, 1), (0, 0)),      # 1 x 1 filter, channels padded 16 -> 32
    ((5, 32, 9, 12), 40, (3, 3), (0, 0)),       # 7 x 10 outputs: rows of 10 floats, read through a padded copy
    ((4, 48, 14, 14), 64, (3, 3), (1, 1)),      # 14 x 14 feature maps
    ((8, 64, 7, 7), 128, (3, 3), (1, 1)),       # 7 x 7 feature maps: four rows padded to 8 pixels per K block
    ((16, 32, 4, 4), 32, (3, 3), (1, 1)),       # rows of 4 pixels: eight rows per K block, the image has four
    ((2, 32, 16, 16), 64, (3, 3), (1, 1)),      # rows of 16: two rows per K block, read without a padded copy
    ((8, 32, 7, 5), 32, (3, 3), (1, 1)),        # 7 rows of 5 pixels: the last K block of an image is one row short
    ((3, 40, 11, 12), 48, (3, 5), (0, 2)),      # 9 rows of 12 pixels padded to 16, no vertical padding
    ((2, 32, 24, 24), 32, (10, 10), (4, 4)),    # 10 x 10 filters: 100 tiles per channel tile
    ((2, 200, 12, 16), 40, (3, 3), (1, 1)),     # 200 channels padded to 224: one tile of 224 columns
    ((4, 3, 20, 20), 64, (3, 3), (1, 1)),       # three input channels: one tile per filter row
    ((8, 8, 12, 12), 32, (3, 4), (1, 2)),       # row-packed and short rows (13 pixels padded to 16) together
    ((2, 1, 40, 40), 160, (5, 5), (2, 2)),      # a single input channel, 160 output channels
    ((2, 16, 6, 6), 32, (3, 3), (1, 1)),        # 72 output pixels: too few, the direct kernel
    ((2, 64, 56, 56), 64, (3, 3), (1, 1)),      # the taps of a filter row share one load of 36 pixels; two boxes per row
    ((3, 128, 20, 17), 96, (3, 3), (1, 1)),     # the same with two 64-channel tiles, 96 output channels, rows of 17 (padded copy)
    ((2, 64, 18, 40), 128, (5, 3), (2, 0)),     # five filter rows, no horizontal padding: rows of 38 pixels
    ((2, 64, 24, 24), 256, (3, 3), (1, 1)),     # 64 channels on a CTA pair: four taps per tile, loaded one by one
])
def test_backward_weight_tensor_core_path(dev, lib, oracle, shape, oc, k, padding):
    """grad_weight as an implicit GEMM over output pixels (>= 32 output channels, >= 256 pixels): TF32
    bars, and FP32-accumulation agreement with the float64 sum of the TF32-truncated operands."""
    rng = np.random.default_rng(sum(shape) + oc)
    x = rng.standard_normal(shape, dtype=np.float32)
    w = np.zeros((oc, shape[1], *k), dtype=np.float32)
    oh = shape[2] + 2 * padding[0] - k[0] + 1
    ow = shape[3] + 2 * padding[1] - k[1] + 1
    dy = rng.standard_normal((shape[0], oc, oh, ow), dtype=np.float32)
    _, dw = conv_backward(dev, lib, dy, w, x, (1, 1), padding)
    _, again = conv_backward(dev, lib, dy, w, x, (1, 1), padding)
    assert np.array_equal(dw, again)                      # K ranges are added in a fixed order
    dw_ref = oracle.conv2d_backward_weight_np(dy, x, k, (1, 1), padding)
    if shape[0] * oh * ow >= 256:
        assert oracle.rel_frobenius(dw, dw_ref) <= TF32_TOL
        model = oracle.conv2d_backward_weight_np(dy, x, k, (1, 1), padding, input_mode=oracle.INPUT_TF32_TRUNC)
        pixels = shape[0] * oh * ow
        assert oracle.rel_frobenius(dw, model) <= TF32_MODEL_TOL * max(1.0, pixels / 4096.0)
    else:
        assert oracle.rel_frobenius(dw, dw_ref) <= FP32_TOL


def test_random_conv_shapes_forward_and_backward(dev, lib, oracle):
    """24 seeded layer shapes (1..3 images, 1..80 channels, 5..40 pixels a side, 1x1..5x5 filters, strides
    1..2, any valid padding): whatever path each of the three launchers picks must stay within the TF32 bar."""
    rng = np.random.default_rng(77)
    for case in range(24):
        nb = int(rng.integers(1, 4))
        c, oc = int(rng.integers(1, 81)), int(rng.integers(1, 161))
        h, wd = int(rng.integers(5, 41)), int(rng.integers(5, 41))
        kh, kw = int(rng.integers(1, 6)), int(rng.integers(1, 6))
        stride = (1, 1) if rng.random() < 0.75 else (int(rng.integers(1, 3)), int(rng.integers(1, 3)))
        ph, pw = int(rng.integers(0, kh)), int(rng.integers(0, kw))
        if h + 2 * ph < kh or wd + 2 * pw < kw:
            continue
        x = rng.standard_normal((nb, c, h, wd), dtype=np.float32)
        w = rng.standard_normal((oc, c, kh, kw), dtype=np.float32) * np.float32(0.2)
        bias = rng.standard_normal(oc, dtype=np.float32)
        y = dev.conv2d(x, w, bias, stride, (ph, pw), act=1)
        want = oracle.conv2d_np(x, w, bias, stride, (ph, pw), act=1)
        assert y.shape == want.shape, (case, x.shape, w.shape, stride, (ph, pw))
        assert oracle.rel_frobenius(y, want) <= TF32_TOL, (case, x.shape, w.shape, stride, (ph, pw))
        dy = rng.standard_normal(want.shape, dtype=np.float32)
        dx, dw = conv_backward(dev, lib, dy, w, x, stride, (ph, pw))
        assert oracle.rel_frobenius(dx, oracle.conv2d_backward_data_np(dy, w, (h, wd), stride, (ph, pw))) <= TF32_TOL, case
        assert oracle.rel_frobenius(dw, oracle.conv2d_backward_weight_np(dy, x, (kh, kw), stride, (ph, pw))) <= TF32_TOL, case


def test_conv_host_buffers(lib, cuda, oracle):
    import ctypes
    from cudeep_b200 import _lib
    x, w, bias = workloads.c4_conv(batch=1, channels=64, out_channels=128, size=28)
    y = np.full((1, 128, 28, 28), np.nan, np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    _lib.check(lib.cudeep_b200_conv2d_forward_host_f32(p(x), p(w), p(bias), p(y), 1, 64, 128, 28, 28, 3, 3,
                                                       1, 1, 1, 1, 1))
    assert _lib.device_status() == 0
    assert oracle.rel_frobenius(y, oracle.conv2d(x, w, bias, (1, 1), (1, 1), act=1)) <= TF32_TOL
