"""Host-side logic that needs no GPU: tensor metadata and views over a fake storage, argument
checks that must fire before any device call, Sequential's fusion plan, workload generators."""
import numpy as np
import pytest


@pytest.fixture()
def cd(monkeypatch):
    import cudeep_b200
    from cudeep_b200 import tensor

    class FakeStorage:
        def __init__(self, nbytes):
            self.ptr = None
            self.nbytes = nbytes

    monkeypatch.setattr(tensor, "_Storage", FakeStorage)
    return cudeep_b200


def test_strides_views_and_reshape(cd):
    t = cd.Tensor([2, 3, 4])
    assert t.strides() == [12, 4, 1] and t.numel() == 24 and t.nbytes() == 96 and t.is_contiguous()
    tt = t.transpose(0, 2)
    assert tt.shape() == [4, 3, 2] and tt.strides() == [1, 4, 12] and not tt.is_contiguous()
    assert tt._storage is t._storage                       # a view, as in the reference (tensor.cu:239-254)
    assert t.transpose(-1, -2).shape() == [2, 4, 3]
    r = t.reshape([6, -1])
    assert r.shape() == [6, 4] and r._storage is t._storage
    with pytest.raises(RuntimeError):
        t.reshape([5, 5])
    with pytest.raises(RuntimeError):
        t.transpose(0, 3)
    assert cd.Tensor([3], cd.DType.float64).nbytes() == 24
    with pytest.raises(RuntimeError):
        cd.Tensor([2], cd.DType.float16)


def test_matmul_argument_checks_fire_before_any_device_call(cd):
    a = cd.Tensor([4, 6])
    with pytest.raises(RuntimeError, match="inner"):
        a.matmul(cd.Tensor([5, 3]))
    with pytest.raises(RuntimeError, match="dtype"):
        a.matmul(cd.Tensor([6, 3], cd.DType.float64))
    with pytest.raises(RuntimeError, match="contiguous"):
        a.matmul(cd.Tensor([3, 6]).transpose(0, 1))
    with pytest.raises(RuntimeError, match="2-D"):
        cd.Tensor([2, 3, 4]).matmul(a)


def test_linear_and_conv_argument_checks(cd):
    with pytest.raises(RuntimeError):
        cd.linear(cd.Tensor([4, 6]), cd.Tensor([3, 5]))
    with pytest.raises(RuntimeError):
        cd.linear(cd.Tensor([4, 6]), cd.Tensor([3, 6]), cd.Tensor([4]))
    with pytest.raises(RuntimeError, match="unknown activation"):
        cd.linear(cd.Tensor([4, 6]), cd.Tensor([3, 6]), None, "tanh")
    with pytest.raises(RuntimeError, match="channel"):
        cd.conv2d(cd.Tensor([1, 3, 8, 8]), cd.Tensor([4, 2, 3, 3]))
    with pytest.raises(RuntimeError, match="kernel larger"):
        cd.conv2d(cd.Tensor([1, 3, 2, 2]), cd.Tensor([4, 3, 3, 3]))
    with pytest.raises(RuntimeError):
        cd.conv2d(cd.Tensor([1, 3, 8, 8]), cd.Tensor([4, 3, 3, 3]), cd.Tensor([5]))


def test_sequential_fusion_plan(cd, monkeypatch):
    calls = []

    class L(cd.nn.Linear):
        def __init__(self):
            cd.nn.Module.__init__(self)

        def forward(self, x, activation=None):
            calls.append(("linear", activation))
            return x

    class A(cd.nn.GELU):
        def forward(self, x):
            calls.append(("gelu", None))
            return x

    x = cd.Tensor([2, 2])
    cd.nn.Sequential(L(), A(), L(), L(), A(), A())(x)
    assert calls == [("linear", "gelu"), ("linear", None), ("linear", "gelu"), ("gelu", None)]
    calls.clear()
    cd.nn.Sequential(L(), A(), fuse=False)(x)
    assert calls == [("linear", None), ("gelu", None)]


def test_workload_generators_are_seeded_and_shaped():
    from cudeep_b200 import workloads as w
    a, b = w.c1_sgemm()
    assert a.shape == b.shape == (512, 512) and a.dtype == np.float32 and np.abs(a).max() <= 1.0
    a2, _ = w.c1_sgemm()
    assert np.array_equal(a, a2)
    x, w1, b1, w2, b2 = w.c3_linear_stack(batch=4, d_in=64, d_hidden=128, d_out=32)
    assert w1.shape == (128, 64) and w2.shape == (32, 128) and x.shape == (4, 64)
    assert np.abs(w1).max() <= np.sqrt(6 / 64) and np.abs(b1).max() <= 0.01 and np.abs(b2).max() <= 0.01
    xc, wc, bc = w.c4_conv(batch=1, channels=8, size=6, out_channels=4)
    assert xc.shape == (1, 8, 6, 6) and wc.shape == (4, 8, 3, 3) and bc.shape == (4,)
    assert abs(float(wc.std()) - np.sqrt(2 / 72)) < 0.05
    band = w.c5_a_band(3, 64)
    assert band.shape == (w.C5_BAND_ROWS, 64)
    rows = w.c5_a_rows(2 * w.C5_BAND_ROWS, 2 * w.C5_BAND_ROWS, 64)
    assert np.array_equal(rows[w.C5_BAND_ROWS:], band)
    assert w.gemm_flops(2, 3, 4) == 48 and w.conv_flops(64, 256, 256, 56, 56, 3, 3) == pytest.approx(236.76e9, rel=1e-4)


# ---- the launcher's tile choice (host arithmetic of cudeep_b200/csrc/gemm_tf32.cu) -----------------

def _plan(lib, m, n, k, act=0, sms=148):
    import ctypes
    from cudeep_b200 import _lib
    ctas, bn, split, katoms = (ctypes.c_int() for _ in range(4))
    est = ctypes.c_double()
    _lib.check(lib.cudeep_b200_gemm_tf32_plan(m, n, k, act, sms, ctypes.byref(ctas), ctypes.byref(bn),
                                              ctypes.byref(split), ctypes.byref(katoms), ctypes.byref(est)))
    return ctas.value, bn.value, split.value, katoms.value, est.value


def test_plan_fills_the_machine_with_wide_pair_tiles(lib):
    for shape in [(8192, 8192, 8192), (4096, 4096, 4096), (2048, 2048, 2048), (8192, 16384, 4096)]:
        ctas, bn, split, katoms, est = _plan(lib, *shape)
        assert (ctas, bn, split, katoms) == (2, 256, 1, 2), shape
        assert est > 0.0


def test_plan_narrows_tiles_for_small_problems(lib):
    # Small cubes: narrow tiles, and the reduction split two ways inside a cluster so that both more SMs
    # work and each takes in half the operand bytes (the exchange costs less than that saves).
    assert _plan(lib, 1024, 1024, 1024)[:3] == (1, 128, 2)      # 64 tiles of 128 x 128, two CTAs each
    assert _plan(lib, 512, 512, 512)[:3] == (1, 64, 2)          # 32 tiles of 128 x 64, two CTAs each
    assert _plan(lib, 256, 256, 256)[:3] == (1, 64, 2)
    assert _plan(lib, 128, 128, 64)[:3] == (1, 64, 1)           # two K blocks: nothing to split
    ctas, bn, split, _, _ = _plan(lib, 1536, 1536, 1536)
    assert (ctas, bn, split) == (2, 128, 1)                     # 72 CTA pairs of 256 x 128


def test_plan_splits_k_inside_a_cluster_for_few_tiles_and_long_k(lib):
    for shape in [(512, 512, 4096), (128, 4096, 4096), (256, 1024, 8192), (1024, 1024, 4096)]:
        ctas, bn, split, katoms, _ = _plan(lib, *shape)
        assert split in (2, 4) and bn <= 128 and ctas * split <= 8, (shape, ctas, bn, split)
    # the clusters of one launch must fit the machine at once
    ctas, bn, split, _, _ = _plan(lib, 1024, 1024, 4096)
    tiles = -(-1024 // (128 * ctas)) * -(-1024 // bn)
    assert tiles * split * ctas <= 148


def test_plan_follows_the_sm_count_and_rejects_nonsense(lib):
    from cudeep_b200 import _lib
    few = _plan(lib, 1024, 1024, 1024, sms=16)
    many = _plan(lib, 1024, 1024, 1024, sms=148)
    assert few[1] > many[1]                                     # 16 SMs are full with wide tiles already
    assert lib.cudeep_b200_gemm_tf32_plan(0, 8, 8, 0, 148, None, None, None, None, None) != 0
    assert "positive" in lib.cudeep_b200_last_error().decode()
    assert _plan(lib, 4096, 4096, 4096, act=2)[:2] == (2, 256)  # an activation rules out the split last wave only
