"""_cudeep_core, the pybind11 extension cuDeep's Python layer imports
(python/cuDeep/_core.py:3-34 in the reference), built on libcudeep_b200.so.

CPU: the module builds, imports without a GPU, exposes every name _core.py imports, and refuses
both off-path operators and device work on a machine with no GPU.
GPU: the reference's own call chains (tests/python/test_matmul.py, test_conv.py style:
Tensor.from_numpy(...).matmul(...).numpy(), conv2d_forward, broadcast_add) against the oracle."""
import importlib
import sys

import numpy as np
import pytest

# python/cuDeep/_core.py:3-34
CORE_NAMES = [
    "Tensor", "DType", "Layout", "Stream", "Event", "MemoryPool", "relu", "sigmoid", "tanh_act", "gelu", "silu",
    "leaky_relu", "broadcast_add", "scalar_mul", "div_op", "neg", "exp_op", "log_op", "sqrt_op", "pow_op", "abs_op",
    "clamp_op", "gt_mask", "sum", "mean", "max", "min", "sum_reduce_rows", "softmax", "mse_loss",
    "cross_entropy_loss", "conv2d_forward", "conv2d_backward_data", "conv2d_backward_weight", "max_pool2d",
    "avg_pool2d", "batchnorm_forward", "layernorm_forward", "activation_backward", "sgd_update", "adam_update",
    "adamw_update", "device_info",
]
ON_PATH = {"Tensor", "DType", "Layout", "Stream", "Event", "MemoryPool", "relu", "sigmoid", "gelu", "silu",
           "broadcast_add", "conv2d_forward", "conv2d_backward_data", "conv2d_backward_weight", "device_info"}


@pytest.fixture(scope="session")
def core(lib):
    from cudeep_b200 import build
    path = build.build_bindings()
    if str(path.parent) not in sys.path:
        sys.path.insert(0, str(path.parent))
    return importlib.import_module("_cudeep_core")


def test_core_exposes_every_name_the_reference_imports(core):
    missing = [n for n in CORE_NAMES if not hasattr(core, n)]
    assert not missing
    for extra in ("linear_forward", "matmul_nt", "matmul_tn"):
        assert hasattr(core, extra)
    assert {m for m in ("float16", "float32", "float64")} <= set(core.DType.__members__)
    assert set(core.Layout.__members__) == {"NCHW", "NHWC"}


def test_off_path_names_raise(core):
    for name in CORE_NAMES:
        if name in ON_PATH:
            continue
        with pytest.raises(RuntimeError, match="outside the dense-contraction path"):
            getattr(core, name)(1, 2)


def test_no_gpu_means_error_not_fallback(core):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="CUDA"):
        core.Tensor([2, 2])


# ---------------------------------------------------------------- GPU: through the reference's calls

def _rel(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


@pytest.mark.gpu
def test_tensor_roundtrip_and_repr(core, cuda):
    a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
    t = core.Tensor.from_numpy(a)
    assert t.shape() == [2, 3, 4] and t.numel() == 24 and t.dtype() == core.DType.float32
    np.testing.assert_array_equal(t.numpy(), a)
    np.testing.assert_array_equal(t.transpose(0, 2).contiguous().numpy(), a.transpose(2, 1, 0))
    assert "shape=[2, 3, 4]" in repr(t) and "float32" in repr(t)
    d = core.Tensor.from_numpy(a.astype(np.float64))
    assert d.dtype() == core.DType.float64 and d.numpy().dtype == np.float64


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(2, 2, 3), (33, 17, 9), (64, 64, 64), (256, 512, 128), (1024, 1024, 1024)])
def test_matmul_chain(core, cuda, oracle, m, n, k):
    rng = np.random.default_rng(m * 7 + n)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    got = core.Tensor.from_numpy(a).matmul(core.Tensor.from_numpy(b)).numpy()
    want = oracle.gemm_f64_inputs(a, b)
    tensor_core = m >= 64 and n >= 64 and k >= 32
    assert _rel(got, want) <= (5e-3 if tensor_core else 1e-5)   # TF32 / FP32 tolerances of the path


@pytest.mark.gpu
def test_matmul_float64_and_mismatch(core, cuda):
    rng = np.random.default_rng(3)
    a = rng.standard_normal((40, 24))
    b = rng.standard_normal((24, 56))
    got = core.Tensor.from_numpy(a).matmul(core.Tensor.from_numpy(b)).numpy()
    np.testing.assert_allclose(got, a @ b, rtol=1e-12, atol=1e-12)
    with pytest.raises(RuntimeError):
        core.Tensor.from_numpy(a).matmul(core.Tensor.from_numpy(a))


@pytest.mark.gpu
def test_linear_as_the_reference_builds_it(core, cuda, oracle):
    """nn.Linear.forward (python/cuDeep/nn.py:110-115): x.matmul(w.transpose(0,1)) + broadcast_add,
    where the Python matmul wrapper makes the transposed view contiguous first
    (python/cuDeep/tensor.py:334-335) because Tensor::matmul refuses views (src/tensor.cu:391-392);
    and the fused addition linear_forward. Both agree with the oracle and with each other."""
    rng = np.random.default_rng(11)
    x = rng.standard_normal((96, 160), dtype=np.float32)
    w = rng.standard_normal((224, 160), dtype=np.float32)
    bias = rng.standard_normal(224, dtype=np.float32)
    tx, tw, tb = (core.Tensor.from_numpy(v) for v in (x, w, bias))
    wt = tw.transpose(0, 1)
    assert not wt.is_contiguous()
    with pytest.raises(RuntimeError, match="contiguous"):
        tx.matmul(wt)
    composed = core.broadcast_add(tx.matmul(wt.contiguous()), tb).numpy()
    fused = core.linear_forward(tx, tw, tb).numpy()
    want = oracle.linear(x.astype(np.float64), w.astype(np.float64), bias.astype(np.float64))
    assert _rel(composed, want) <= 5e-3 and _rel(fused, want) <= 5e-3
    assert _rel(fused, composed.astype(np.float64)) <= 1e-6
    relu = core.linear_forward(tx, tw, tb, 1).numpy()
    np.testing.assert_array_equal(relu, np.maximum(fused, 0))
    np.testing.assert_array_equal(core.relu(core.Tensor.from_numpy(fused)).numpy(), np.maximum(fused, 0))


@pytest.mark.gpu
def test_matmul_nt_tn(core, cuda, oracle):
    rng = np.random.default_rng(5)
    a = rng.standard_normal((128, 96), dtype=np.float32)
    b = rng.standard_normal((160, 96), dtype=np.float32)
    got = core.matmul_nt(core.Tensor.from_numpy(a), core.Tensor.from_numpy(b)).numpy()
    assert _rel(got, a.astype(np.float64) @ b.astype(np.float64).T) <= 5e-3
    at = rng.standard_normal((96, 128), dtype=np.float32)
    bt = rng.standard_normal((96, 160), dtype=np.float32)
    got = core.matmul_tn(core.Tensor.from_numpy(at), core.Tensor.from_numpy(bt)).numpy()
    assert _rel(got, at.astype(np.float64).T @ bt.astype(np.float64)) <= 5e-3


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [
    (1, 1, 5, 5, 1, 3, 1, 0),       # single channel, the reference's smallest case
    (2, 3, 8, 8, 4, 3, 1, 1),
    (2, 3, 9, 9, 5, 3, 2, 1),
    (4, 64, 28, 28, 64, 3, 1, 1),   # tensor-core implicit GEMM
])
def test_conv2d_forward_and_backward(core, cuda, oracle, shape):
    b, ic, ih, iw, oc, ks, s, p = shape
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal((b, ic, ih, iw), dtype=np.float32)
    w = rng.standard_normal((oc, ic, ks, ks), dtype=np.float32)
    bias = rng.standard_normal(oc, dtype=np.float32)
    tx, tw, tb = (core.Tensor.from_numpy(v) for v in (x, w, bias))
    y = core.conv2d_forward(tx, tw, tb, [s, s], [p, p])
    want = oracle.conv2d_np(x.astype(np.float64), w.astype(np.float64), bias.astype(np.float64), (s, s), (p, p))
    assert y.shape() == list(want.shape)
    assert _rel(y.numpy(), want) <= 5e-3
    no_bias = core.conv2d_forward(tx, tw, None, [s, s], [p, p]).numpy()
    assert _rel(no_bias, want - bias.astype(np.float64)[None, :, None, None]) <= 5e-3

    dy = rng.standard_normal(want.shape, dtype=np.float32)
    tdy = core.Tensor.from_numpy(dy)
    gi = core.conv2d_backward_data(tdy, tw, [b, ic, ih, iw], [s, s], [p, p]).numpy()
    gw = core.conv2d_backward_weight(tdy, tx, [oc, ic, ks, ks], [s, s], [p, p]).numpy()
    want_gi = oracle.conv2d_backward_data_np(dy.astype(np.float64), w.astype(np.float64), (ih, iw), (s, s), (p, p))
    want_gw = oracle.conv2d_backward_weight_np(dy.astype(np.float64), x.astype(np.float64), (ks, ks), (s, s), (p, p))
    assert _rel(gi, want_gi) <= 5e-3
    assert _rel(gw, want_gw) <= 5e-3      # tensor cores (TF32) where the shape allows, else strict FP32


@pytest.mark.gpu
def test_conv_bindings_reject_mismatched_operands_before_any_launch(core, cuda):
    """Every extent the kernels and their tensor maps assume is checked against the operands:
    a mismatch is a RuntimeError, not a read past the smaller buffer."""
    T = core.Tensor
    f32 = lambda *shape: T.from_numpy(np.zeros(shape, np.float32))
    f64 = lambda *shape: T.from_numpy(np.zeros(shape, np.float64))
    x, w, b = f32(2, 8, 10, 10), f32(16, 8, 3, 3), f32(16)
    core.conv2d_forward(x, w, b, [1, 1], [1, 1])                       # the well-formed call works
    with pytest.raises(RuntimeError, match="input channels"):
        core.conv2d_forward(x, f32(16, 4, 3, 3), b, [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="dtype"):
        core.conv2d_forward(x, f64(16, 8, 3, 3), None, [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="dtype"):
        core.conv2d_forward(x, w, f64(16), [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="out_channels"):
        core.conv2d_forward(x, w, f32(8), [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="kernel larger"):
        core.conv2d_forward(f32(1, 8, 2, 2), w, None, [1, 1], [0, 0])
    with pytest.raises(RuntimeError, match="stride"):
        core.conv2d_forward(x, w, None, [0, 1], [1, 1])
    with pytest.raises(RuntimeError, match="padding"):
        core.conv2d_forward(x, w, None, [1, 1], [-1, 1])
    with pytest.raises(RuntimeError, match="4-D"):
        core.conv2d_forward(f32(8, 10, 10), w, None, [1, 1], [1, 1])
    go = f32(2, 16, 10, 10)
    core.conv2d_backward_data(go, w, [2, 8, 10, 10], [1, 1], [1, 1])
    core.conv2d_backward_weight(go, x, [16, 8, 3, 3], [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="grad_output must be"):
        core.conv2d_backward_data(f32(2, 16, 9, 10), w, [2, 8, 10, 10], [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="grad_output must be"):
        core.conv2d_backward_data(go, w, [2, 8, 20, 20], [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="dtype"):
        core.conv2d_backward_data(go, f64(16, 8, 3, 3), [2, 8, 10, 10], [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="input channels"):
        core.conv2d_backward_data(go, w, [2, 4, 10, 10], [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="grad_output must be"):
        core.conv2d_backward_weight(f32(2, 8, 10, 10), x, [16, 8, 3, 3], [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="dtype"):
        core.conv2d_backward_weight(go, f64(2, 8, 10, 10), [16, 8, 3, 3], [1, 1], [1, 1])
    with pytest.raises(RuntimeError, match="input channels"):
        core.conv2d_backward_weight(go, x, [16, 4, 3, 3], [1, 1], [1, 1])


@pytest.mark.gpu
def test_broadcast_add_rejects_bad_shapes(core, cuda):
    m = core.Tensor.from_numpy(np.ones((4, 6), dtype=np.float32))
    with pytest.raises(RuntimeError, match="broadcast_add"):
        core.broadcast_add(m, core.Tensor.from_numpy(np.ones(5, dtype=np.float32)))


@pytest.mark.gpu
def test_stream_event_pool_device_info(core, cuda):
    info = core.device_info()
    assert info["multiprocessors"] > 0 and "." in info["compute_capability"]
    pool = core.MemoryPool.instance()
    before = pool.allocated_bytes
    t = core.Tensor([1024, 1024])
    assert pool.allocated_bytes >= before + 4 * 1024 * 1024
    del t
    assert pool.allocated_bytes == before
    pool.release_cached()
    assert pool.cached_bytes == 0
    s = core.Stream()
    e0, e1 = core.Event(), core.Event()
    e0.record(s)
    a = core.Tensor.from_numpy(np.eye(96, dtype=np.float32))
    a.set_stream(s)                      # addition: the product and its storage belong to stream s
    prod = a.matmul(a)
    e1.record(s)
    s.synchronize()
    np.testing.assert_array_equal(prod.numpy(), np.eye(96, dtype=np.float32))
    e1.synchronize()
    assert e1.elapsed_ms(e0) >= 0.0
