"""Pins the CPU oracle (CPU only).

1. The reference's own known-answer tests for this path, replayed against the
   oracle: tests/unit/test_matmul.cu:13-68, tests/unit/test_tensor.cu:189-248 and
   :368-381, tests/unit/test_kernels.cu:324-425, tests/unit/test_tensor_ops.py:210-262,
   tests/unit/test_nn.py:50-76 (paths in the cuDeep tree).
2. The C oracle against its independent NumPy restatement.
3. The committed golden fixtures (tests/golden/dense_golden.npz).
"""
from pathlib import Path

import numpy as np
import pytest

GOLDEN = Path(__file__).resolve().parent / "golden" / "dense_golden.npz"


# ---- 1. reference known answers ---------------------------------------------------------

def test_ref_matmul_diag_times_identity(oracle):
    # test_matmul.cu:13-40: diag(1..4) * I == diag(1..4), tolerance 1e-5
    a = np.diag(np.arange(1, 5)).astype(np.float32)
    c = oracle.gemm(a, np.eye(4, dtype=np.float32))
    assert np.max(np.abs(c - a)) < 1e-5


def test_ref_matmul_2x2(oracle):
    # test_matmul.cu:42-66 and test_tensor_ops.py:211-218: {1,2,3,4}*{5,6,7,8} = {19,22,43,50}
    a = np.array([[1, 2], [3, 4]], dtype=np.float32)
    b = np.array([[5, 6], [7, 8]], dtype=np.float32)
    assert np.allclose(oracle.gemm(a, b), [[19, 22], [43, 50]], atol=1e-5)
    # the TF32 datapath is exact on small integers, which is why the reference's
    # tensor-core kernel passes this test (operands have <= 10 mantissa bits)
    assert np.array_equal(oracle.gemm(a, b, input_mode=oracle.INPUT_TF32_TRUNC), oracle.gemm(a, b))


def test_ref_tensor_matmul_partial_identity(oracle):
    # test_tensor.cu:205-228: [2,3] x [3,4] with B = [I3 | 0] copies A into the first 3 columns
    a = np.arange(1, 7, dtype=np.float32).reshape(2, 3)
    b = np.zeros((3, 4), dtype=np.float32)
    b[:, :3] = np.eye(3)
    c = oracle.gemm(a, b)
    assert np.allclose(c[:, :3], a) and np.all(c[:, 3] == 0)


def test_ref_tensor_matmul_8x8_identity(oracle):
    # test_tensor.cu:230-248 (tol 0.01) and test_tensor_ops.py:220-227 (rtol 1e-5): A*I == A
    rng = np.random.default_rng(0)
    a = rng.standard_normal((8, 8), dtype=np.float32)
    assert np.allclose(oracle.gemm(a, np.eye(8, dtype=np.float32)), a, rtol=1e-5)


def test_ref_matmul_f64_2x2(oracle):
    # test_tensor.cu:368-381, test_tensor_ops.py:247-254: double 2x2, tolerance 1e-10
    a = np.array([[1.5, 2.5], [3.5, 4.5]])
    b = np.array([[0.5, 1.5], [2.5, 3.5]])
    assert np.max(np.abs(oracle.gemm_f64_inputs(a, b) - a @ b)) < 1e-10


def test_ref_linear_known_weights(oracle):
    # test_nn.py:50-62: W = [[1,0,0],[0,1,0]], no bias: y = first two features of x
    w = np.array([[1, 0, 0], [0, 1, 0]], dtype=np.float32)
    x = np.array([[1, 2, 3], [4, 5, 6]], dtype=np.float32)
    assert np.allclose(oracle.linear(x, w), [[1, 2], [4, 5]], rtol=1e-5)
    # test_nn.py:64-76: identity weight plus bias {100, 200}
    y = oracle.linear(np.array([[1, 2]], dtype=np.float32), np.eye(2, dtype=np.float32),
                      np.array([100, 200], dtype=np.float32))
    assert np.allclose(y, [[101, 202]], rtol=1e-5)


def test_ref_conv_1x1_identity(oracle):
    # test_kernels.cu:324-351: 1x1 kernel of weight 1 on a 4x4 iota image returns the image
    x = np.arange(1, 17, dtype=np.float32).reshape(1, 1, 4, 4)
    y = oracle.conv2d(x, np.ones((1, 1, 1, 1), np.float32), np.zeros(1, np.float32))
    assert np.max(np.abs(y - x)) < 1e-4


def test_ref_conv_3x3_ones(oracle):
    # test_kernels.cu:353-374: all-ones 3x3 image and kernel, no padding -> 9
    x = np.ones((1, 1, 3, 3), np.float32)
    w = np.ones((1, 1, 3, 3), np.float32)
    assert abs(oracle.conv2d(x, w)[0, 0, 0, 0] - 9.0) < 1e-4
    # :376-398 with bias 10 -> 19
    assert abs(oracle.conv2d(x, w, np.array([10], np.float32))[0, 0, 0, 0] - 19.0) < 1e-4


def test_ref_conv_3x3_padding(oracle):
    # test_kernels.cu:400-425: pad 1 -> centre 9, corner 4, edge 6
    x = np.ones((1, 1, 3, 3), np.float32)
    y = oracle.conv2d(x, np.ones((1, 1, 3, 3), np.float32), None, (1, 1), (1, 1))
    assert y.shape == (1, 1, 3, 3)
    assert abs(y[0, 0, 1, 1] - 9) < 1e-4 and abs(y[0, 0, 0, 0] - 4) < 1e-4 and abs(y[0, 0, 0, 1] - 6) < 1e-4


def test_ref_conv_layer_shapes(oracle):
    # tests/unit/test_layers.py:58-75: output shapes of Conv2d(3->16, 3x3, pad 1) on 2x3x8x8,
    # Conv2d(1->4, 3x3) on 1x1x8x8 and a stride-2 layer
    assert oracle.conv2d(np.zeros((2, 3, 8, 8), np.float32), np.zeros((16, 3, 3, 3), np.float32),
                         None, (1, 1), (1, 1)).shape == (2, 16, 8, 8)
    assert oracle.conv2d(np.zeros((1, 1, 8, 8), np.float32), np.zeros((4, 1, 3, 3), np.float32)).shape == (1, 4, 6, 6)
    assert oracle.conv2d(np.zeros((1, 3, 8, 8), np.float32), np.zeros((8, 3, 3, 3), np.float32),
                         None, (2, 2), (1, 1)).shape == (1, 8, 4, 4)


def test_ref_conv_backward_known_answers(oracle):
    # tests/unit/test_advanced_kernels.cu:197-219: 1x1 kernel of weight 2, grad_output all ones -> grad_input all 2
    dy = np.ones((1, 1, 3, 3), np.float32)
    dx = oracle.conv2d_backward_data_np(dy, np.full((1, 1, 1, 1), 2.0, np.float32), (3, 3))
    assert np.max(np.abs(dx - 2.0)) < 1e-4
    # :221-241: input all ones, grad_output all ones -> grad_weight = 9
    dw = oracle.conv2d_backward_weight_np(dy, np.ones((1, 1, 3, 3), np.float32), (1, 1))
    assert abs(dw[0, 0, 0, 0] - 9.0) < 1e-4


def test_conv_backward_is_the_adjoint_of_forward(oracle):
    """<conv(x, w), dy> == <x, dgrad(dy, w)> == <w, wgrad(dy, x)> for random data, strides and paddings."""
    rng = np.random.default_rng(31)
    for (shape, oc, k, stride, padding) in [((2, 3, 7, 8), 4, (3, 3), (1, 1), (1, 1)),
                                            ((1, 2, 9, 9), 3, (3, 2), (2, 1), (0, 1)),
                                            ((2, 4, 6, 6), 2, (1, 1), (1, 1), (0, 0))]:
        x = rng.standard_normal(shape, dtype=np.float32)
        w = rng.standard_normal((oc, shape[1], *k), dtype=np.float32)
        y = oracle.conv2d(x, w, None, stride, padding)
        dy = rng.standard_normal(y.shape).astype(np.float32)
        lhs = float(np.sum(y * dy))
        dx = oracle.conv2d_backward_data_np(dy, w, shape[2:], stride, padding)
        dw = oracle.conv2d_backward_weight_np(dy, x, k, stride, padding)
        assert abs(lhs - float(np.sum(x.astype(np.float64) * dx))) <= 1e-9 * abs(lhs) + 1e-9
        assert abs(lhs - float(np.sum(w.astype(np.float64) * dw))) <= 1e-9 * abs(lhs) + 1e-9


# ---- 2. C oracle vs NumPy restatement ---------------------------------------------------

@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 3, 7), (64, 48, 80), (33, 129, 17)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_c_gemm_matches_numpy(oracle, m, n, k, mode):
    rng = np.random.default_rng(m * 1000 + n * 10 + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    assert oracle.rel_frobenius(oracle.gemm(a, b, input_mode=mode), oracle.gemm_np(a, b, input_mode=mode)) < 1e-14
    w = np.ascontiguousarray(b.T)
    bias = rng.standard_normal(n, dtype=np.float32)
    for act in range(5):
        got = oracle.linear(a, w, bias, act=act, input_mode=mode)
        want = oracle.gemm_np(a, w, b_is_nk=True, bias=bias, act=act, input_mode=mode)
        assert oracle.rel_frobenius(got, want) < 1e-13


@pytest.mark.parametrize("shape,oc,k,stride,padding", [
    ((1, 1, 5, 5), 1, (3, 3), (1, 1), (0, 0)),
    ((2, 3, 8, 9), 4, (3, 3), (1, 1), (1, 1)),
    ((1, 5, 10, 7), 2, (5, 3), (2, 1), (2, 0)),
    ((3, 2, 6, 6), 7, (1, 1), (1, 1), (0, 0)),
])
def test_c_conv_matches_numpy(oracle, shape, oc, k, stride, padding):
    rng = np.random.default_rng(sum(shape) + oc)
    x = rng.standard_normal(shape, dtype=np.float32)
    w = rng.standard_normal((oc, shape[1], *k), dtype=np.float32)
    bias = rng.standard_normal(oc, dtype=np.float32)
    for act in (0, 1, 2):
        got = oracle.conv2d(x, w, bias, stride, padding, act=act)
        want = oracle.conv2d_np(x, w, bias, stride, padding, act=act)
        assert got.shape == want.shape
        assert oracle.rel_frobenius(got, want) < 1e-13


def test_tf32_truncation_model(oracle):
    x = np.array([1.0, 1.0 + 2.0 ** -10, 1.0 + 2.0 ** -11, -(1.0 + 2.0 ** -11 + 2.0 ** -12), 3.14159274], np.float32)
    t = oracle.tf32_truncate(x)
    assert t[0] == 1.0 and t[1] == x[1] and t[2] == 1.0 and t[3] == -1.0
    assert np.all(np.abs(t) <= np.abs(x)) and np.all(np.abs(x - t) <= np.abs(x) * 2.0 ** -10)
    r = oracle.tf32_round(x)
    assert r[2] == 1.0 and r[3] == np.float32(-(1.0 + 2.0 ** -10))
    assert np.all(np.abs(x - r) <= np.abs(x) * 2.0 ** -11)
    out = np.empty_like(x)
    import ctypes
    oracle.lib().oracle_tf32_truncate(x.ctypes.data_as(ctypes.c_void_p), out.ctypes.data_as(ctypes.c_void_p),
                                      ctypes.c_size_t(x.size))
    assert np.array_equal(out, t)


def test_activations_match_definitions(oracle):
    x = np.linspace(-6, 6, 97)
    assert np.allclose(oracle.activation(x, oracle.EPI_SIGMOID), 1 / (1 + np.exp(-x)))
    assert np.allclose(oracle.activation(x, oracle.EPI_SILU), x / (1 + np.exp(-x)))
    assert np.array_equal(oracle.activation(x, oracle.EPI_RELU), np.maximum(x, 0))
    # tanh-form GELU (ptx_intrinsics.cuh:545-549), close to but not equal to the erf form
    from math import erf
    g = oracle.activation(x, oracle.EPI_GELU)
    erf_form = np.array([0.5 * v * (1 + erf(v / np.sqrt(2))) for v in x])
    assert np.max(np.abs(g - erf_form)) < 2e-3 and np.max(np.abs(g - erf_form)) > 1e-5
    c = [oracle.lib().oracle_activation(float(v), oracle.EPI_GELU) for v in x]
    assert np.allclose(c, g, rtol=1e-14, atol=1e-15)


def test_sgemm_f32_baseline_kernel(oracle):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((130, 300), dtype=np.float32)
    b = rng.standard_normal((300, 70), dtype=np.float32)
    assert oracle.rel_frobenius(oracle.sgemm_f32(a, b), oracle.gemm(a, b)) < 1e-5


# ---- 3. golden fixtures -----------------------------------------------------------------

def test_golden_gemm_and_linear(oracle):
    g = np.load(GOLDEN)
    for tag in ("aligned", "ragged"):
        a, b, w, bias = (g[f"gemm_{tag}_{s}"] for s in ("a", "b", "w", "bias"))
        assert oracle.rel_frobenius(oracle.gemm(a, b), g[f"gemm_{tag}_c"]) < 1e-15
        assert oracle.rel_frobenius(oracle.gemm(a, b, input_mode=1), g[f"gemm_{tag}_c_tf32"]) < 1e-15
        for act in range(5):
            assert oracle.rel_frobenius(oracle.linear(a, w, bias, act=act), g[f"linear_{tag}_act{act}"]) < 1e-15


def test_golden_conv(oracle):
    g = np.load(GOLDEN)
    for tag in ("p1", "s2", "k1", "k5"):
        sh, sw, ph, pw = (int(v) for v in g[f"conv_{tag}_meta"])
        y = oracle.conv2d(g[f"conv_{tag}_x"], g[f"conv_{tag}_w"], g[f"conv_{tag}_bias"], (sh, sw), (ph, pw),
                          act=oracle.EPI_RELU)
        assert y.shape == g[f"conv_{tag}_y"].shape
        assert oracle.rel_frobenius(y, g[f"conv_{tag}_y"]) < 1e-15
