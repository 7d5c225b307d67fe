"""This library against the reference's own CUDA kernels on the same device and inputs.

oracle/_ref/libcudeep_ref.so holds cuDeep's unmodified matmul and conv sources rebuilt for
sm_100 (oracle/Makefile).  Both implementations are judged against the float64 oracle; they
are not expected to agree bit for bit (different summation order; the reference computes the
3x3 stride-1 convolution through Winograd F(4,3)).
"""
import ctypes

import numpy as np
import pytest

from cudeep_b200 import workloads

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref():
    from oracle import oracle as o
    if not o.REF_LIB_PATH.exists():
        pytest.skip("oracle/_ref/libcudeep_ref.so not built (needs the reference tree at build time)")
    return ctypes.CDLL(str(o.REF_LIB_PATH))


def ref_matmul(ref, dev, a, b, strict=False):
    ta, tb = dev.to_dev(a), dev.to_dev(b)
    m, k = a.shape
    n = b.shape[1]
    tc = dev.empty((m, n))
    fn = ref.cudeep_ref_matmul_f32_strict if strict else ref.cudeep_ref_matmul_f32
    assert fn(dev.ptr(ta), dev.ptr(tb), dev.ptr(tc), m, n, k, None) == 0
    dev.torch.cuda.synchronize()
    return tc.cpu().numpy()


@pytest.mark.parametrize("n", [512, 1024, 2048, 4096])
def test_tf32_matmul_both_within_bounds(ref, dev, oracle, n):
    a, b = workloads.c2_gemm(n)
    ours = dev.matmul(a, b)
    theirs = ref_matmul(ref, dev, a, b)
    # whole product, whatever the size; FP32 accumulation error grows with K (both sides carry it)
    assert oracle.rel_frobenius(ours, theirs) <= 2e-5 * max(1.0, n / 2048)
    if n > 2048:   # the float64 oracle on 128 sampled rows (all columns)
        rows = np.sort(np.random.default_rng(n).choice(n, size=128, replace=False))
        a, ours, theirs = a[rows], ours[rows], theirs[rows]
    exact = oracle.gemm(a, b)
    assert oracle.rel_frobenius(theirs, exact) <= 5e-3        # the oracle describes the reference
    assert oracle.rel_frobenius(ours, exact) <= 5e-3
    # same operand truncation, different summation order: they agree to accumulation error,
    # and both follow the truncated-operand model
    model = oracle.gemm(a, b, input_mode=oracle.INPUT_TF32_TRUNC)
    assert oracle.rel_frobenius(theirs, model) <= 2e-5 * max(1.0, n / 2048)
    assert oracle.rel_frobenius(ours, model) <= 2e-5 * max(1.0, n / 2048)


def test_fp32_matmul_c1(ref, dev, oracle):
    a, b = workloads.c1_sgemm()
    exact = oracle.gemm(a, b)
    ours = dev.matmul(a, b, strict=True)
    theirs = ref_matmul(ref, dev, a, b, strict=True)
    assert oracle.rel_frobenius(theirs, exact) <= 1e-5
    assert oracle.rel_frobenius(ours, exact) <= 1e-5


def test_reference_known_answers_on_reference(ref, dev):
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[5, 6], [7, 8]], np.float32)
    assert np.allclose(ref_matmul(ref, dev, a, b), [[19, 22], [43, 50]], atol=1e-5)


def test_conv_3x3_both_within_bounds(ref, dev, oracle):
    x, w, bias = workloads.c4_conv(batch=2, channels=64, out_channels=128, size=28)
    exact = oracle.conv2d(x, w, bias, (1, 1), (1, 1))
    ours = dev.conv2d(x, w, bias, (1, 1), (1, 1))
    tx, tw, tb = dev.to_dev(x), dev.to_dev(w), dev.to_dev(bias)
    ty = dev.empty(exact.shape)
    assert ref.cudeep_ref_conv2d_forward_f32(dev.ptr(tx), dev.ptr(tw), dev.ptr(tb), dev.ptr(ty), 2, 64, 128, 28,
                                             28, 3, 3, 1, 1, 1, 1, None) == 0
    dev.torch.cuda.synchronize()
    theirs = ty.cpu().numpy()
    err_ours = oracle.rel_frobenius(ours, exact)
    err_theirs = oracle.rel_frobenius(theirs, exact)
    assert err_ours <= 5e-3
    # Winograd in FP32 followed by TF32 GEMMs amplifies the error; the reference stays
    # within a looser bound, and the direct implicit GEMM is at least as accurate.
    assert err_theirs <= 5e-2
    assert err_ours <= err_theirs * 1.5


# ---- the reference's fused-activation GEMM (sgemm_tc_fused_kernel, src/kernels/matmul_kernel.cu:1543-1735;
# fast_gelu_ptx / fast_silu_ptx / fast_sigmoid_ptx, include/cudeep/ptx_intrinsics.cuh:531-554) --------------

@pytest.mark.parametrize("act", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("m,n,k", [(512, 512, 256), (1024, 1024, 512)])
def test_fused_activation_matches_the_reference_kernel(ref, dev, oracle, lib, act, m, n, k):
    """Shapes are multiples of the reference's 128 x 128 x 32 tile (the fused kernel is its unguarded
    aligned one) with N / 128 a multiple of 4: its tile raster walks columns in groups of 4
    (matmul_kernel.cu:1565-1576) and covers C only then."""
    rng = np.random.default_rng(100 * act + m)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = (rng.standard_normal((k, n), dtype=np.float32) * np.float32(4.0 / np.sqrt(k)))   # pre-activations ~ N(0, 4)
    ta, tb = dev.to_dev(a), dev.to_dev(b)
    ours_t, theirs_t = dev.empty((m, n)), dev.empty((m, n))
    dev.check(lib.cudeep_b200_matmul_fused_act(dev.ptr(ta), dev.ptr(tb), dev.ptr(ours_t), m, n, k, act, None))
    assert ref.cudeep_ref_matmul_fused_act(dev.ptr(ta), dev.ptr(tb), dev.ptr(theirs_t), m, n, k, act, None) == 0
    assert dev.sync_status() == 0
    ours, theirs = ours_t.cpu().numpy(), theirs_t.cpu().numpy()
    model = oracle.gemm(a, b, act=act, input_mode=oracle.INPUT_TF32_TRUNC)
    # both follow "float64 activation of the truncated-operand product" to SFU accuracy, and each other
    assert oracle.rel_frobenius(theirs, model) <= 2e-5
    assert oracle.rel_frobenius(ours, model) <= 2e-5
    assert oracle.rel_frobenius(ours, theirs) <= 2e-5
    assert np.max(np.abs(ours - theirs)) <= 2e-5 * max(1.0, float(np.max(np.abs(theirs))))


# ---- the reference's im2col + TF32 GEMM convolution branch (src/kernels/conv_kernel.cu:242-334: taken when
# the filter is not 3x3 stride 1, C*KH*KW >= 9 and the im2col matrix is at most 4 MiB) ------------------------

@pytest.mark.parametrize("geom", [
    # batch, C, OC, H, W, KH, KW, stride, pad    -> GEMM [OC, C*KH*KW] x [C*KH*KW, batch*OH*OW]
    (2, 32, 128, 16, 16, 5, 5, 1, 2),            # 128 x 800 x 512, im2col matrix 1.6 MB
    (2, 64, 256, 32, 32, 3, 3, 2, 1),            # 256 x 576 x 512, 1.2 MB (stride 2)
    (1, 32, 128, 16, 32, 5, 5, 1, 2),            # one image: the reference writes NCHW straight from the GEMM
])
def test_conv_im2col_branch_of_the_reference_pins_the_oracle(ref, dev, oracle, geom):
    batch, c, oc, h, w_, kh, kw, stride, pad = geom
    rng = np.random.default_rng(sum(geom))
    x = rng.standard_normal((batch, c, h, w_), dtype=np.float32)
    w = (rng.standard_normal((oc, c, kh, kw), dtype=np.float32) * np.float32(np.sqrt(2.0 / (c * kh * kw))))
    bias = rng.uniform(-0.1, 0.1, oc).astype(np.float32)
    oh, ow = (h + 2 * pad - kh) // stride + 1, (w_ + 2 * pad - kw) // stride + 1
    assert c * kh * kw * batch * oh * ow * 4 <= 4 << 20 and not (kh == 3 and stride == 1)
    ours = dev.conv2d(x, w, bias, (stride, stride), (pad, pad))
    tx, tw, tb = dev.to_dev(x), dev.to_dev(w), dev.to_dev(bias)
    ty = dev.empty((batch, oc, oh, ow))
    assert ref.cudeep_ref_conv2d_forward_f32(dev.ptr(tx), dev.ptr(tw), dev.ptr(tb), dev.ptr(ty), batch, c, oc, h, w_,
                                             kh, kw, stride, stride, pad, pad, None) == 0
    dev.torch.cuda.synchronize()
    theirs = ty.cpu().numpy()
    exact = oracle.conv2d(x, w, bias, (stride, stride), (pad, pad))
    model = oracle.conv2d(x, w, bias, (stride, stride), (pad, pad), input_mode=oracle.INPUT_TF32_TRUNC)
    assert oracle.rel_frobenius(theirs, exact) <= 5e-3
    assert oracle.rel_frobenius(ours, exact) <= 5e-3
    # on this branch the reference is a plain TF32 GEMM over gathered operands: it agrees with the
    # truncated-operand convolution oracle, and with this library, to FP32-accumulation error
    assert oracle.rel_frobenius(theirs, model) <= 2e-5
    assert oracle.rel_frobenius(ours, model) <= 2e-5
    assert oracle.rel_frobenius(ours, theirs) <= 2e-5
