"""The Python host layer (cudeep_b200.Tensor / nn) on a GPU.

The cases follow the reference's own Python tests for this path so that a cuDeep user finds the
same behaviour: tests/unit/test_tensor_ops.py:210-262 (TestMatmul), tests/unit/test_nn.py:29-118
(TestLinear, TestSequential), tests/unit/test_layers.py:58-75 (TestConv2dLayer),
tests/performance/test_perf.py:126-142 (pool leak check); plus parity of the fused paths against
the CPU oracle.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cd(lib, cuda):
    import cudeep_b200
    return cudeep_b200


class TestMatmul:
    def test_matmul_2x2(self, cd):
        a = np.array([[1, 2], [3, 4]], dtype=np.float32)
        b = np.array([[5, 6], [7, 8]], dtype=np.float32)
        c = cd.Tensor.from_numpy(a).matmul(cd.Tensor.from_numpy(b))
        np.testing.assert_allclose(c.numpy(), a @ b, rtol=1e-5)

    def test_matmul_identity(self, cd):
        a = np.random.default_rng(0).standard_normal((8, 8)).astype(np.float32)
        c = cd.Tensor.from_numpy(a).matmul(cd.Tensor.from_numpy(np.eye(8, dtype=np.float32)))
        np.testing.assert_allclose(c.numpy(), a, rtol=1e-5)

    def test_matmul_nonsquare(self, cd):
        rng = np.random.default_rng(1)
        a = rng.standard_normal((3, 5)).astype(np.float32)
        b = rng.standard_normal((5, 7)).astype(np.float32)
        c = cd.Tensor.from_numpy(a) @ cd.Tensor.from_numpy(b)
        assert c.shape() == [3, 7]
        np.testing.assert_allclose(c.numpy(), a @ b, rtol=1e-4, atol=1e-6)

    def test_matmul_large(self, cd):
        rng = np.random.default_rng(2)
        a = rng.standard_normal((64, 128)).astype(np.float32)
        b = rng.standard_normal((128, 32)).astype(np.float32)
        c = cd.Tensor.from_numpy(a).matmul(cd.Tensor.from_numpy(b))
        assert c.shape() == [64, 32]
        np.testing.assert_allclose(c.numpy(), a @ b, rtol=1e-3, atol=1e-3)

    def test_matmul_f64(self, cd):
        a = np.array([[1, 2], [3, 4]], dtype=np.float64)
        b = np.array([[5, 6], [7, 8]], dtype=np.float64)
        c = cd.Tensor.from_numpy(a).matmul(cd.Tensor.from_numpy(b))
        np.testing.assert_allclose(c.numpy(), a @ b)

    def test_matmul_output_shape(self, cd):
        assert cd.Tensor.randn([10, 20]).matmul(cd.Tensor.randn([20, 30])).shape() == [10, 30]

    def test_matmul_perf_sizes_vs_numpy(self, cd):
        # tests/performance/test_perf.py:34-49: 256, 512, 1024 square vs NumPy, rtol 1e-2 / atol 1e-1
        rng = np.random.default_rng(3)
        for n in (256, 512, 1024):
            a = rng.standard_normal((n, n)).astype(np.float32)
            b = rng.standard_normal((n, n)).astype(np.float32)
            c = cd.Tensor.from_numpy(a).matmul(cd.Tensor.from_numpy(b)).numpy()
            np.testing.assert_allclose(c, a @ b, rtol=1e-2, atol=1e-1)

    def test_matmul_rejects_what_the_reference_rejects(self, cd):
        t = cd.Tensor.randn([4, 6])
        with pytest.raises(RuntimeError):
            t.matmul(cd.Tensor.randn([5, 3]))                         # inner extents
        with pytest.raises(RuntimeError):
            t.matmul(cd.Tensor.randn([6, 3], cd.DType.float64))       # dtype
        with pytest.raises(RuntimeError):
            t.matmul(cd.Tensor.randn([3, 6]).transpose(0, 1))         # not contiguous
        with pytest.raises(RuntimeError):
            cd.Tensor.randn([2, 3, 4]).matmul(t)                      # not 2-D

    def test_matmul_backward(self, cd, oracle):
        rng = np.random.default_rng(12)
        a = rng.standard_normal((256, 128)).astype(np.float32)
        b = rng.standard_normal((128, 192)).astype(np.float32)
        g = rng.standard_normal((256, 192)).astype(np.float32)
        ga, gb = cd.matmul_backward(cd.Tensor.from_numpy(a), cd.Tensor.from_numpy(b), cd.Tensor.from_numpy(g))
        assert ga.shape() == [256, 128] and gb.shape() == [128, 192]
        assert oracle.rel_frobenius(ga.numpy(), g.astype(np.float64) @ b.T.astype(np.float64)) <= 5e-3
        assert oracle.rel_frobenius(gb.numpy(), a.T.astype(np.float64) @ g.astype(np.float64)) <= 5e-3

    def test_strict_fp32_option(self, cd, oracle):
        rng = np.random.default_rng(4)
        a = rng.standard_normal((256, 256)).astype(np.float32)
        b = rng.standard_normal((256, 256)).astype(np.float32)
        ta, tb = cd.Tensor.from_numpy(a), cd.Tensor.from_numpy(b)
        assert oracle.rel_frobenius(ta.matmul(tb, strict_fp32=True).numpy(), oracle.gemm(a, b)) <= 1e-5
        assert 1e-5 < oracle.rel_frobenius(ta.matmul(tb).numpy(), oracle.gemm(a, b)) <= 5e-3


class TestTensorPlumbing:
    def test_roundtrip_and_metadata(self, cd):
        a = np.arange(24, dtype=np.float32).reshape(2, 3, 4)
        t = cd.Tensor.from_numpy(a)
        assert t.shape() == [2, 3, 4] and t.strides() == [12, 4, 1] and t.ndim() == 3
        assert t.numel() == 24 and t.nbytes() == 96 and t.dtype() == cd.DType.float32 and t.is_contiguous()
        np.testing.assert_array_equal(t.numpy(), a)
        assert "shape=[2, 3, 4]" in repr(t)

    def test_transpose_contiguous_reshape(self, cd):
        a = np.random.default_rng(5).standard_normal((37, 53)).astype(np.float32)
        t = cd.Tensor.from_numpy(a).transpose(0, 1)
        assert t.shape() == [53, 37] and not t.is_contiguous()
        c = t.contiguous()
        assert c.is_contiguous()
        np.testing.assert_array_equal(c.numpy(), a.T)
        np.testing.assert_array_equal(t.numpy(), a.T)
        np.testing.assert_array_equal(cd.Tensor.from_numpy(a).reshape([53, 37]).numpy(), a.reshape(53, 37))
        b = np.random.default_rng(6).standard_normal((3, 4, 5)).astype(np.float64)
        np.testing.assert_array_equal(cd.Tensor.from_numpy(b).transpose(0, 2).contiguous().numpy(),
                                      b.transpose(2, 1, 0))

    def test_fill_zeros_ones(self, cd):
        np.testing.assert_array_equal(cd.Tensor.zeros([3, 5]).numpy(), np.zeros((3, 5), np.float32))
        np.testing.assert_array_equal(cd.Tensor.ones([4], cd.DType.float64).numpy(), np.ones(4))
        np.testing.assert_array_equal(cd.Tensor([2, 2]).fill_(7.5).numpy(), np.full((2, 2), 7.5, np.float32))

    def test_broadcast_add(self, cd):
        m = np.arange(12, dtype=np.float32).reshape(3, 4)
        r = np.array([10, 20, 30, 40], dtype=np.float32)
        out = cd.broadcast_add(cd.Tensor.from_numpy(m), cd.Tensor.from_numpy(r))
        np.testing.assert_array_equal(out.numpy(), m + r)

    def test_pool_reuses_blocks(self, cd):
        # tests/performance/test_perf.py:126-142
        pool = cd.MemoryPool.instance()
        before = pool.allocated_bytes()
        for _ in range(50):
            cd.Tensor.zeros([256, 256])
        import gc
        gc.collect()
        assert pool.allocated_bytes() == before
        assert pool.cached_bytes() >= 256 * 256 * 4
        pool.release_cached()
        assert pool.cached_bytes() == 0

    def test_events_and_streams(self, cd):
        s = cd.Stream()
        e0, e1 = cd.Event(), cd.Event()
        a = cd.Tensor.randn([512, 512])
        a.stream = s.handle
        e0.record(s)
        b = a.matmul(a)
        e1.record(s)
        e1.synchronize()
        assert e1.elapsed_ms(e0) >= 0.0
        s.synchronize()
        assert b.shape() == [512, 512]
        info = cd.device_info()
        assert info["sm_count"] > 0 and info["compute_capability"][0] == 10


class TestLinear:
    def test_creation(self, cd):
        layer = cd.nn.Linear(10, 5)
        assert len(layer.parameters()) == 2
        assert layer._parameters["weight"].shape() == [5, 10]
        assert layer._parameters["bias"].shape() == [5]
        assert len(cd.nn.Linear(10, 5, bias=False).parameters()) == 1

    def test_forward_shape(self, cd):
        assert cd.nn.Linear(8, 4)(cd.Tensor.randn([2, 8])).shape() == [2, 4]

    def test_forward_deterministic(self, cd):
        layer = cd.nn.Linear(3, 2, bias=False)
        w = np.array([[1, 0, 0], [0, 1, 0]], dtype=np.float32)
        layer._parameters["weight"] = cd.Tensor.from_numpy(w)
        x = np.array([[10, 20, 30], [40, 50, 60]], dtype=np.float32)
        np.testing.assert_allclose(layer(cd.Tensor.from_numpy(x)).numpy(), x @ w.T, rtol=1e-5)

    def test_forward_with_bias(self, cd):
        layer = cd.nn.Linear(2, 2)
        w, b = np.eye(2, dtype=np.float32), np.array([100, 200], dtype=np.float32)
        layer._parameters["weight"] = cd.Tensor.from_numpy(w)
        layer._parameters["bias"] = cd.Tensor.from_numpy(b)
        x = np.array([[1, 2]], dtype=np.float32)
        np.testing.assert_allclose(layer(cd.Tensor.from_numpy(x)).numpy(), x @ w.T + b, rtol=1e-5)

    def test_f64(self, cd):
        layer = cd.nn.Linear(4, 3, dtype=cd.DType.float64)
        x = np.random.default_rng(7).standard_normal((1, 4))
        out = layer(cd.Tensor.from_numpy(x))
        assert out.shape() == [1, 3]
        sd = layer.state_dict()
        np.testing.assert_allclose(out.numpy(), x @ sd["weight"].T + sd["bias"], rtol=1e-12)

    def test_fused_equals_reference_sequence(self, cd, oracle):
        """One fused kernel against the reference's three steps (transpose copy, matmul, broadcast_add)
        run through this library, and against the oracle."""
        rng = np.random.default_rng(8)
        x = rng.standard_normal((256, 192)).astype(np.float32)
        layer = cd.nn.Linear(192, 320)
        layer._parameters["bias"] = cd.Tensor.from_numpy(rng.standard_normal(320).astype(np.float32))
        tx = cd.Tensor.from_numpy(x)
        fused = layer(tx).numpy()
        w = layer._parameters["weight"]
        stepwise = cd.broadcast_add(tx.matmul(w.transpose(0, 1).contiguous()), layer._parameters["bias"]).numpy()
        assert oracle.rel_frobenius(fused, stepwise) <= 2e-5
        sd = layer.state_dict()
        assert oracle.rel_frobenius(fused, oracle.linear(x, sd["weight"], sd["bias"])) <= 5e-3


class TestSequential:
    def test_creation_and_shapes(self, cd):
        model = cd.nn.Sequential(cd.nn.Linear(10, 5), cd.nn.Linear(5, 2))
        assert len(model.parameters()) == 4 and len(model) == 2
        assert model(cd.Tensor.randn([4, 10])).shape() == [4, 2]

    def test_train_eval_propagates(self, cd):
        l1, l2 = cd.nn.Linear(10, 5), cd.nn.Linear(5, 2)
        model = cd.nn.Sequential(l1, l2)
        model.eval()
        assert l1._training is False and l2._training is False
        model.train()
        assert l1._training is True and l2._training is True

    def test_deeper_model(self, cd):
        model = cd.nn.Sequential(cd.nn.Linear(784, 256), cd.nn.Linear(256, 128), cd.nn.Linear(128, 10))
        assert model(cd.Tensor.randn([8, 784])).shape() == [8, 10]
        assert len(model.parameters()) == 6

    def test_activation_fusion_matches_unfused(self, cd, oracle):
        rng = np.random.default_rng(9)
        x = rng.standard_normal((128, 256)).astype(np.float32)
        layers = [cd.nn.Linear(256, 512), cd.nn.GELU(), cd.nn.Linear(512, 128), cd.nn.ReLU()]
        for layer, scale in ((layers[0], 0.05), (layers[2], 0.05)):
            shape = layer._parameters["weight"].shape()
            layer._parameters["weight"] = cd.Tensor.from_numpy((rng.standard_normal(shape) * scale).astype(np.float32))
        fused = cd.nn.Sequential(*layers)(cd.Tensor.from_numpy(x)).numpy()
        unfused = cd.nn.Sequential(*layers, fuse=False)(cd.Tensor.from_numpy(x)).numpy()
        assert oracle.rel_frobenius(fused, unfused) <= 1e-6
        sd = cd.nn.Sequential(*layers).state_dict()
        h = oracle.linear(x, sd["0.weight"], sd["0.bias"], act=oracle.EPI_GELU)
        y = oracle.linear(h.astype(np.float32), sd["2.weight"], sd["2.bias"], act=oracle.EPI_RELU)
        assert oracle.rel_frobenius(fused, y) <= 5e-3

    def test_state_dict_roundtrip(self, cd):
        a = cd.nn.Sequential(cd.nn.Linear(6, 4), cd.nn.ReLU(), cd.nn.Linear(4, 3))
        b = cd.nn.Sequential(cd.nn.Linear(6, 4), cd.nn.ReLU(), cd.nn.Linear(4, 3))
        b.load_state_dict(a.state_dict())
        x = cd.Tensor.randn([5, 6], seed=1)
        np.testing.assert_array_equal(a(x).numpy(), b(x).numpy())
        assert sorted(a.state_dict()) == ["0.bias", "0.weight", "2.bias", "2.weight"]


class TestConv2dLayer:
    def test_shapes(self, cd):
        assert cd.nn.Conv2d(3, 16, 3, padding=1)(cd.Tensor.randn([2, 3, 8, 8])).shape() == [2, 16, 8, 8]
        assert cd.nn.Conv2d(1, 4, 3)(cd.Tensor.randn([1, 1, 8, 8])).shape() == [1, 4, 6, 6]
        assert cd.nn.Conv2d(3, 8, 3, stride=2, padding=1)(cd.Tensor.randn([1, 3, 8, 8])).shape() == [1, 8, 4, 4]

    def test_values_and_fused_relu(self, cd, oracle):
        rng = np.random.default_rng(10)
        conv = cd.nn.Conv2d(32, 64, 3, padding=1)
        w = (rng.standard_normal((64, 32, 3, 3)) * 0.1).astype(np.float32)
        b = rng.standard_normal(64).astype(np.float32)
        conv.load_state_dict({"weight": w, "bias": b})
        x = rng.standard_normal((2, 32, 12, 12)).astype(np.float32)
        y = cd.nn.Sequential(conv, cd.nn.ReLU())(cd.Tensor.from_numpy(x)).numpy()
        assert oracle.rel_frobenius(y, oracle.conv2d(x, w, b, (1, 1), (1, 1), act=oracle.EPI_RELU)) <= 5e-3
        y64 = cd.conv2d(cd.Tensor.from_numpy(x.astype(np.float64)), cd.Tensor.from_numpy(w.astype(np.float64)),
                        cd.Tensor.from_numpy(b.astype(np.float64)), padding=1).numpy()
        assert oracle.rel_frobenius(y64, oracle.conv2d(x, w, b, (1, 1), (1, 1))) <= 1e-12


def test_pool_is_stream_aware(lib, cuda):
    """A block freed on a stream serves that stream again at once, but another stream only after
    the work queued before the free has drained (include/cudeep/memory.cuh)."""
    import ctypes
    from cudeep_b200 import _lib
    torch = cuda
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    p1, p2 = ctypes.c_void_p(s1.cuda_stream), ctypes.c_void_p(s2.cuda_stream)
    nbytes = (8 << 20) + 4096          # a size class of its own

    def alloc(stream):
        out = ctypes.c_void_p()
        _lib.check(lib.cudeep_b200_pool_alloc_on_stream(nbytes, stream, ctypes.byref(out)))
        return out.value

    def free(ptr, stream):
        _lib.check(lib.cudeep_b200_pool_free_on_stream(ctypes.c_void_p(ptr), stream))

    _lib.check(lib.cudeep_b200_pool_release_cached())
    block = alloc(p1)
    # About 10 ms of work on stream 1, then the block is released behind it.
    n = 8192
    a = torch.randn((n, n), device="cuda")
    c = torch.empty((n, n), device="cuda")
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    torch.cuda.synchronize()
    for _ in range(8):
        _lib.check(lib.cudeep_b200_matmul_f32(ptr(a), ptr(a), ptr(c), n, n, n, p1))
    free(block, p1)
    same_stream = alloc(p1)
    assert same_stream == block                      # ordered behind the pending work by the stream itself
    free(same_stream, p1)
    other_stream = alloc(p2)
    still_busy = not s1.query()
    if still_busy:
        assert other_stream != block                 # stream 1 has not drained: a fresh block instead
    torch.cuda.synchronize()
    free(other_stream, p2)
    later = alloc(p2)
    assert later in (block, other_stream)            # everything has drained: cached blocks serve any stream
    free(later, p2)
    assert _lib.device_status() == 0
    _lib.check(lib.cudeep_b200_pool_release_cached())


def test_entry_points_can_be_captured_in_a_cuda_graph(lib, cuda, oracle):
    """Launch-bound chains are meant to be replayed from CUDA graphs: GEMM, fused Linear, conv forward
    (with its stream-ordered scratch) and conv grad_weight are captured once on a side stream and
    replayed on new inputs."""
    import ctypes
    from cudeep_b200 import _lib
    torch = cuda
    rng = np.random.default_rng(31)
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    x = torch.zeros((128, 256), device="cuda")
    w = torch.from_numpy(rng.standard_normal((512, 256), dtype=np.float32) * np.float32(0.1)).cuda()
    b = torch.from_numpy(rng.standard_normal(512, dtype=np.float32)).cuda()
    h = torch.empty((128, 512), device="cuda")
    w2 = torch.from_numpy(rng.standard_normal((512, 64), dtype=np.float32) * np.float32(0.1)).cuda()
    y = torch.empty((128, 64), device="cuda")
    img = torch.zeros((2, 32, 16, 16), device="cuda")
    filt = torch.from_numpy(rng.standard_normal((64, 32, 3, 3), dtype=np.float32) * np.float32(0.1)).cuda()
    out = torch.empty((2, 64, 16, 16), device="cuda")
    dw = torch.empty_like(filt)
    side = torch.cuda.Stream()
    sp = ctypes.c_void_p(side.cuda_stream)

    def chain():
        _lib.check(lib.cudeep_b200_linear_forward_f32(ptr(x), ptr(w), ptr(b), ptr(h), 128, 512, 256, 1, sp))
        _lib.check(lib.cudeep_b200_matmul_f32(ptr(h), ptr(w2), ptr(y), 128, 64, 512, sp))
        _lib.check(lib.cudeep_b200_conv2d_forward_f32(ptr(img), ptr(filt), None, ptr(out), 2, 32, 64, 16, 16, 3, 3,
                                                      1, 1, 1, 1, sp))
        _lib.check(lib.cudeep_b200_conv2d_backward_weight_f32(ptr(out), ptr(img), ptr(dw), 2, 32, 64, 16, 16, 3, 3,
                                                              1, 1, 1, 1, sp))

    with torch.cuda.stream(side):
        chain()                                    # first use outside the capture (attributes, pools)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            chain()
        for seed in (1, 2):
            xr = np.random.default_rng(seed).standard_normal((128, 256), dtype=np.float32)
            ir = np.random.default_rng(seed + 10).standard_normal((2, 32, 16, 16), dtype=np.float32)
            x.copy_(torch.from_numpy(xr))
            img.copy_(torch.from_numpy(ir))
            graph.replay()
            torch.cuda.synchronize()
            hidden = oracle.linear(xr, w.cpu().numpy(), b.cpu().numpy(), act=oracle.EPI_RELU)
            assert oracle.rel_frobenius(h.cpu().numpy(), hidden) <= 5e-3
            assert oracle.rel_frobenius(y.cpu().numpy(), oracle.gemm(h.cpu().numpy(), w2.cpu().numpy())) <= 5e-3
            conv = oracle.conv2d_np(ir, filt.cpu().numpy(), None, (1, 1), (1, 1))
            assert oracle.rel_frobenius(out.cpu().numpy(), conv) <= 5e-3
            grad = oracle.conv2d_backward_weight_np(out.cpu().numpy(), ir, (3, 3), (1, 1), (1, 1))
            assert oracle.rel_frobenius(dw.cpu().numpy(), grad) <= 5e-3
    assert _lib.device_status() == 0
