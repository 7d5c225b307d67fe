"""GPU parity of the matmul / Linear path against the float64 CPU oracle, through the C ABI.

Bars (from the benchmark specification):
  strict FP32 path  : relative Frobenius error <= 1e-5
  TF32 path         : relative Frobenius error <= 5e-3 and every element within
                      2^-9 * K * max|a| * max|b| of the float64 product
and, stronger, the TF32 path must agree with the float64 product of the
TF32-truncated inputs to FP32-accumulation accuracy (<= 2e-5 relative up to K = 4096,
growing in proportion to K beyond), which pins the operand handling to the reference's
(raw FP32 words into the TF32 MMA).
"""
import numpy as np
import pytest

from cudeep_b200 import workloads

pytestmark = pytest.mark.gpu

FP32_TOL = 1e-5
TF32_TOL = 5e-3
TF32_MODEL_TOL = 2e-5


def check_tf32(oracle, got, a, b, k, *, b_is_nk=False, bias=None, act=0, rows=None):
    sel = slice(None) if rows is None else rows
    exact = oracle.gemm(a[sel], b, b_is_nk=b_is_nk, bias=bias, act=act)
    model = oracle.gemm(a[sel], b, b_is_nk=b_is_nk, bias=bias, act=act, input_mode=oracle.INPUT_TF32_TRUNC)
    g = got[sel]
    assert not np.isnan(g).any()
    assert oracle.rel_frobenius(g, exact) <= TF32_TOL
    # The tensor core's FP32 accumulation adds an error that grows linearly with K (about
    # 2.4e-9 * K relative: 1.2e-6 at K = 512, 3.8e-5 at K = 16384), so the bound widens past K = 4096.
    assert oracle.rel_frobenius(g, model) <= TF32_MODEL_TOL * max(1.0, k / 4096.0)
    if act == 0:
        assert np.max(np.abs(g - exact)) <= oracle.tf32_elementwise_bound(a, b, k)


# ---- reference known-answer cases through the library -------------------------------------

def test_known_answers(dev, oracle):
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[5, 6], [7, 8]], np.float32)
    assert np.allclose(dev.matmul(a, b), [[19, 22], [43, 50]], atol=1e-5)      # test_matmul.cu:42-66
    d = np.diag(np.arange(1, 5)).astype(np.float32)
    assert np.allclose(dev.matmul(d, np.eye(4, dtype=np.float32)), d, atol=1e-5)  # test_matmul.cu:13-40
    rng = np.random.default_rng(0)
    r = rng.standard_normal((8, 8), dtype=np.float32)
    assert np.allclose(dev.matmul(r, np.eye(8, dtype=np.float32)), r, rtol=1e-5)  # test_tensor_ops.py:220-227
    a35, b57 = rng.standard_normal((3, 5), dtype=np.float32), rng.standard_normal((5, 7), dtype=np.float32)
    assert np.allclose(dev.matmul(a35, b57), a35 @ b57, rtol=1e-4, atol=1e-6)     # test_tensor_ops.py:229-237
    a1, b1 = rng.standard_normal((64, 128), dtype=np.float32), rng.standard_normal((128, 32), dtype=np.float32)
    assert np.allclose(dev.matmul(a1, b1), a1 @ b1, rtol=1e-3, atol=1e-3)         # test_tensor_ops.py:239-245


def test_known_answers_f64(dev, lib):
    import torch
    a = np.array([[1.5, 2.5], [3.5, 4.5]])
    b = np.array([[0.5, 1.5], [2.5, 3.5]])
    ta, tb = dev.to_dev(a), dev.to_dev(b)
    tc = dev.empty((2, 2), dtype=torch.float64)
    dev.check(lib.cudeep_b200_matmul_f64(dev.ptr(ta), dev.ptr(tb), dev.ptr(tc), 2, 2, 2, None))
    assert dev.sync_status() == 0
    assert np.max(np.abs(tc.cpu().numpy() - a @ b)) < 1e-10                    # test_tensor.cu:368-381


# ---- C1: strict FP32 ---------------------------------------------------------------------

def test_c1_fp32_512(dev, oracle):
    a, b = workloads.c1_sgemm()
    got = dev.matmul(a, b, strict=True)
    assert oracle.rel_frobenius(got, oracle.gemm(a, b)) <= FP32_TOL


@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (2, 2, 2), (3, 7, 5), (70, 33, 45), (129, 257, 65), (300, 130, 1000)])
def test_fp32_shapes(dev, oracle, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    assert oracle.rel_frobenius(dev.matmul(a, b, strict=True), oracle.gemm(a, b)) <= FP32_TOL


def test_small_and_unaligned_dispatch_is_fp32_exact(dev, oracle):
    """Shapes the tensor-core path does not take must come out at FP32 accuracy."""
    rng = np.random.default_rng(11)
    for m, n, k in [(8, 8, 8), (63, 200, 64), (200, 63, 64), (128, 130, 64), (128, 128, 30)]:
        a = rng.standard_normal((m, k), dtype=np.float32)
        b = rng.standard_normal((k, n), dtype=np.float32)
        assert oracle.rel_frobenius(dev.matmul(a, b), oracle.gemm(a, b)) <= FP32_TOL


def test_golden_fixtures_fp32(dev, oracle):
    from pathlib import Path
    g = np.load(Path(__file__).resolve().parent / "golden" / "dense_golden.npz")
    for tag in ("aligned", "ragged"):
        a, b, w, bias = (g[f"gemm_{tag}_{s}"] for s in ("a", "b", "w", "bias"))
        assert oracle.rel_frobenius(dev.matmul(a, b, strict=True), g[f"gemm_{tag}_c"]) <= FP32_TOL
        for act in range(5):
            got = dev.linear(a, w, bias, act=act)
            assert oracle.rel_frobenius(got, g[f"linear_{tag}_act{act}"]) <= 2e-5   # SFU-approximate activations


# ---- C2: TF32 tensor-core GEMM, B as [K, N] --------------------------------------------------

@pytest.mark.parametrize("n", [1024, 2048])
def test_c2_tf32_full(dev, oracle, n):
    a, b = workloads.c2_gemm(n)
    got = dev.matmul(a, b)
    check_tf32(oracle, got, a, b, n)


@pytest.mark.parametrize("n", [4096, 8192])
def test_c2_tf32_sampled_rows(dev, oracle, n):
    """Full-size products; the float64 oracle checks 96 random rows (all columns) of each."""
    a, b = workloads.c2_gemm(n)
    got = dev.matmul(a, b)
    rows = np.sort(np.random.default_rng(n).choice(n, size=96, replace=False))
    check_tf32(oracle, got, a, b, n, rows=rows)
    # every tile took part: no row of the output is left poisoned, and a column checksum of
    # the whole product matches the one formed from the operands (sum_i C[i,:] = (sum_i A[i,:]) B)
    assert not np.isnan(got).any()
    colsum = got.sum(axis=0, dtype=np.float64)
    want = a.sum(axis=0, dtype=np.float64) @ b.astype(np.float64)
    assert np.linalg.norm(colsum - want) / np.linalg.norm(want) <= TF32_TOL


def test_c5_shapes_single_shard(dev, oracle):
    """The sharded configurations as one GPU sees them: an 8192-row shard of 65536 x 8192 x 8192
    (rows 3*8192.. of A, generated band by band as every rank would) and a 2048-row shard of
    16384^3; the float64 oracle checks 64 sampled rows of each."""
    b = workloads.c5_b(8192, 8192)
    a = workloads.c5_a_rows(3 * 8192, 8192, 8192)
    got = dev.matmul(a, b)
    rows = np.sort(np.random.default_rng(5).choice(8192, size=64, replace=False))
    check_tf32(oracle, got, a, b, 8192, rows=rows)
    del got
    b2 = workloads.c5_b(16384, 16384)
    a2 = workloads.c5_a_rows(7 * 2048, 2048, 16384)
    got2 = dev.matmul(a2, b2)
    assert got2.shape == (2048, 16384) and not np.isnan(got2).any()
    rows = np.sort(np.random.default_rng(6).choice(2048, size=64, replace=False))
    check_tf32(oracle, got2, a2, b2, 16384, rows=rows)


@pytest.mark.parametrize("ctas,bn,katoms", [(1, 256, 1), (1, 128, 1), (1, 128, 2), (1, 64, 1), (1, 64, 2),
                                            (2, 256, 1), (2, 256, 2), (2, 128, 1), (2, 128, 2)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_tf32_every_tile_configuration(dev, oracle, ctas, bn, katoms, b_is_nk):
    rng = np.random.default_rng(ctas * 1000 + bn + int(b_is_nk))
    m, n, k = 640, 768, 416          # several tiles per CTA; 13 K blocks: odd, last one partial
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((n, k) if b_is_nk else (k, n), dtype=np.float32)
    got = dev.gemm_tuned(a, b, b_is_nk, ctas=ctas, bn=bn, katoms=katoms, max_ctas=8)   # 8 CTAs walk many tiles each
    check_tf32(oracle, got, a, b, k, b_is_nk=b_is_nk)


def test_tf32_b_loaded_as_separate_boxes(dev, oracle):
    """B[K,N] with N a multiple of 32 normally takes one chunked TMA box; the per-chunk path must agree."""
    rng = np.random.default_rng(77)
    a = rng.standard_normal((384, 160), dtype=np.float32)
    b = rng.standard_normal((160, 512), dtype=np.float32)
    one = dev.gemm_tuned(a, b, False, ctas=2, bn=256)
    many = dev.gemm_tuned(a, b, False, ctas=2, bn=256, unchunked=True)
    assert np.array_equal(one, many)
    check_tf32(oracle, one, a, b, 160)


@pytest.mark.parametrize("m,n,k", [(64, 64, 32), (100, 260, 36), (129, 132, 200), (1000, 72, 64), (257, 1028, 516)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_tf32_ragged_shapes(dev, oracle, m, n, k, b_is_nk):
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((n, k) if b_is_nk else (k, n), dtype=np.float32)
    got = dev.gemm_tuned(a, b, b_is_nk)
    check_tf32(oracle, got, a, b, k, b_is_nk=b_is_nk)


@pytest.mark.parametrize("ctas,bn,max_ctas,split_k", [
    (2, 256, 0, 0),      # 12 tiles on 74 CTA pairs: no full wave, so the launcher does not split
    (2, 256, 0, 4),      # forced four ranges
    (1, 256, 0, 3),      # one CTA per tile, three ranges (1024 K blocks do not divide evenly)
    (2, 256, 10, 2),     # 5 pairs, 12 tiles: 10 whole tiles, 2 tail tiles split in two
    (1, 128, 6, 2),      # narrow tiles, whole tiles and split tiles mixed
    (2, 256, 0, 1),      # splitting switched off
])
@pytest.mark.parametrize("b_is_nk,bias", [(False, False), (True, True)])
def test_tf32_split_k(dev, oracle, ctas, bn, max_ctas, split_k, b_is_nk, bias):
    rng = np.random.default_rng(ctas * 100 + bn + split_k)
    m, n, k = 520, 1500, 2080          # ragged rows and columns: scalar and vector partial-sum paths
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((n, k) if b_is_nk else (k, n), dtype=np.float32)
    bv = rng.standard_normal(n, dtype=np.float32) if bias else None
    got = dev.gemm_tuned(a, b, b_is_nk, bias=bv, ctas=ctas, bn=bn, max_ctas=max_ctas, split_k=split_k)
    check_tf32(oracle, got, a, b, k, b_is_nk=b_is_nk, bias=bv)


def test_tf32_split_k_chosen_by_the_launcher(dev, lib, oracle):
    """4096 x 4096 x 512: 256 tiles on 74 CTA pairs leave a 34-tile last wave, which the launcher
    splits in two K ranges that accumulate into C - so it must first clear what the caller left there."""
    rng = np.random.default_rng(123)
    a = rng.standard_normal((4096, 512), dtype=np.float32)
    b = rng.standard_normal((512, 4096), dtype=np.float32)
    ta, tb = dev.to_dev(a), dev.to_dev(b)
    tc = dev.torch.full((4096, 4096), 1.0e6, device=dev.dev)
    dev.check(lib.cudeep_b200_matmul_f32(dev.ptr(ta), dev.ptr(tb), dev.ptr(tc), 4096, 4096, 512, None))
    assert dev.sync_status() == 0
    got = tc.cpu().numpy()
    rows = np.sort(rng.choice(4096, size=128, replace=False))
    check_tf32(oracle, got, a, b, 512, rows=rows)
    colsum = got.sum(axis=0, dtype=np.float64)
    want = a.sum(axis=0, dtype=np.float64) @ b.astype(np.float64)
    assert np.linalg.norm(colsum - want) / np.linalg.norm(want) <= TF32_TOL
    again = dev.matmul(a, b)
    assert np.array_equal(got, again)          # two K ranges: order-independent, bitwise reproducible


# ---- split-K inside a thread-block cluster (partial sums exchanged through distributed shared memory)

@pytest.mark.parametrize("ctas,bn,cluster_split,katoms", [
    (1, 64, 2, 0), (1, 128, 2, 0), (1, 128, 4, 0), (1, 128, 4, 1), (2, 128, 2, 0), (2, 128, 4, 0),
    (1, 256, 2, 0), (1, 256, 4, 0), (1, 256, 8, 0), (2, 256, 2, 0), (2, 256, 4, 0),
])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_tf32_cluster_split_k(dev, oracle, ctas, bn, cluster_split, katoms, b_is_nk):
    """Every cluster shape; ragged M and N, bias and ReLU fused after the reduction; 33 K blocks, so
    the last K range is shorter than the others and ends in a partial block."""
    rng = np.random.default_rng(ctas * 1000 + bn + cluster_split)
    m, n, k = 300, 520, 1044
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((n, k) if b_is_nk else (k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    got = dev.gemm_tuned(a, b, b_is_nk, bias=bias, act=1, ctas=ctas, bn=bn, katoms=katoms,
                         cluster_split=cluster_split)
    check_tf32(oracle, got, a, b, k, b_is_nk=b_is_nk, bias=bias, act=1)
    again = dev.gemm_tuned(a, b, b_is_nk, bias=bias, act=1, ctas=ctas, bn=bn, katoms=katoms,
                           cluster_split=cluster_split)
    assert np.array_equal(got, again)          # partial sums are added in a fixed order


def test_tf32_cluster_split_k_falls_back_when_k_is_short(dev, oracle):
    """64 floats of K are two blocks: a request for four ranges runs as two, one block each."""
    rng = np.random.default_rng(9)
    a = rng.standard_normal((256, 64), dtype=np.float32)
    b = rng.standard_normal((64, 256), dtype=np.float32)
    got = dev.gemm_tuned(a, b, False, ctas=1, bn=128, cluster_split=4)
    check_tf32(oracle, got, a, b, 64)
    one = rng.standard_normal((256, 32), dtype=np.float32)        # a single block cannot be split at all
    got = dev.gemm_tuned(one, b[:32].copy(), False, ctas=1, bn=128, cluster_split=2)
    check_tf32(oracle, got, one, b[:32].copy(), 32)


@pytest.mark.parametrize("m,n,k", [(512, 512, 4096), (128, 4096, 4096), (256, 1024, 8192), (1024, 1024, 4096)])
def test_tf32_cluster_split_k_chosen_by_the_launcher(dev, lib, oracle, m, n, k):
    """Few tiles and a long K: the plain entry points spread each tile's K over a cluster.  The result
    must not depend on what the caller left in C."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    ta, tb = dev.to_dev(a), dev.to_dev(b)
    tc = dev.torch.full((m, n), 1.0e6, device=dev.dev)
    dev.check(lib.cudeep_b200_matmul_f32(dev.ptr(ta), dev.ptr(tb), dev.ptr(tc), m, n, k, None))
    assert dev.sync_status() == 0
    got = tc.cpu().numpy()
    check_tf32(oracle, got, a, b, k)
    w = np.ascontiguousarray(b.T)
    bias = rng.standard_normal(n, dtype=np.float32)
    y = dev.linear(a, w, bias, act=2)
    check_tf32(oracle, y, a, w, k, b_is_nk=True, bias=bias, act=2)


# ---- the two ways of writing C ------------------------------------------------------------------

@pytest.mark.parametrize("m,n,k", [(640, 768, 416), (300, 520, 100), (129, 132, 64), (2048, 2048, 64)])
@pytest.mark.parametrize("b_is_nk", [False, True])
def test_tf32_bulk_store_matches_register_store(dev, oracle, m, n, k, b_is_nk):
    """C goes out through shared memory and bulk tensor stores when its rows are 16-byte multiples,
    else straight from registers; both must give the same bits (edge tiles are clipped by the store)."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((n, k) if b_is_nk else (k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    for ctas, bn in [(2, 256), (1, 256), (1, 64), (2, 128)]:
        bulk = dev.gemm_tuned(a, b, b_is_nk, bias=bias, act=3, ctas=ctas, bn=bn)
        regs = dev.gemm_tuned(a, b, b_is_nk, bias=bias, act=3, ctas=ctas, bn=bn, register_store=True)
        assert np.array_equal(bulk, regs)
    check_tf32(oracle, bulk, a, b, k, b_is_nk=b_is_nk, bias=bias, act=3)


@pytest.mark.parametrize("ctas,bn,max_ctas", [(2, 256, 0), (1, 256, 0), (1, 64, 0), (2, 256, 4), (1, 128, 6)])
def test_tf32_last_tile_staged_in_the_stage_ring(dev, oracle, ctas, bn, max_ctas):
    """A CTA's last tile may stage its results in the idle operand ring instead of the two small
    staging blocks; with few CTAs (max_ctas) the earlier tiles of each CTA take the normal path.
    Both ways must give the same bits."""
    rng = np.random.default_rng(ctas * 10 + bn + max_ctas)
    m, n, k = 900, 1100, 288
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    bias = rng.standard_normal(n, dtype=np.float32)
    ring = dev.gemm_tuned(a, b, False, bias=bias, act=1, ctas=ctas, bn=bn, max_ctas=max_ctas)
    plain = dev.gemm_tuned(a, b, False, bias=bias, act=1, ctas=ctas, bn=bn, max_ctas=max_ctas, flip_ring_staging=True)
    assert np.array_equal(ring, plain)
    check_tf32(oracle, ring, a, b, k, bias=bias, act=1)


def test_tf32_store_does_not_touch_memory_behind_c(dev, lib, oracle):
    """Tiles hang over the edge of C (M = 130, N = 36): rows behind the last one stay as they were."""
    rng = np.random.default_rng(2)
    m, n, k = 130, 36, 64
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    ta, tb = dev.to_dev(a), dev.to_dev(b)
    tc = dev.torch.full((m + 4, n), 7.0, device=dev.dev)
    dev.check(lib.cudeep_b200_gemm_tf32_tuned(dev.ptr(ta), dev.ptr(tb), 0, dev.ptr(tc), m, n, k, None, 0, 0,
                                              0, 0, 0, 0, 0, 0, None))
    assert dev.sync_status() == 0
    got = tc.cpu().numpy()
    assert np.all(got[m:] == 7.0)
    check_tf32(oracle, got[:m], a, b, k)


def test_tf32_is_deterministic(dev):
    a, b = workloads.c2_gemm(1024)
    assert np.array_equal(dev.matmul(a, b), dev.matmul(a, b))


def test_tf32_linearity(dev, oracle):
    """(2A)B == 2(AB) exactly: scaling by a power of two commutes with truncation and rounding."""
    a, b = workloads.c2_gemm(1024)
    assert np.array_equal(dev.matmul(2 * a, b), 2 * dev.matmul(a, b))


# ---- seeded random shapes through the plain entry points (whatever path the launcher picks) ----------

def test_random_shapes_through_the_launchers(dev, oracle):
    """60 seeded shapes, extents 1..900 with a bias towards multiples of 4 and long K: every dispatch
    outcome (SIMT, each tile shape, cluster split, bulk and register stores, ragged edges) must stay
    within the TF32 bar, and within the FP32 bar when the shape cannot take the tensor cores."""
    rng = np.random.default_rng(2024)
    for case in range(60):
        m, n = (int(rng.integers(1, 900)) for _ in range(2))
        k = int(rng.integers(1, 900)) if case % 3 else int(rng.integers(900, 5000))
        if rng.random() < 0.7:
            n, k = max(4, n // 4 * 4), max(4, k // 4 * 4)
        a = rng.standard_normal((m, k), dtype=np.float32)
        if case % 2 == 0:
            b = rng.standard_normal((k, n), dtype=np.float32)
            got = dev.matmul(a, b)
            want = oracle.gemm(a, b)
            tensor_core = m >= 64 and n >= 64 and k >= 32 and k % 4 == 0 and n % 4 == 0
        else:
            w = rng.standard_normal((n, k), dtype=np.float32)
            bias = rng.standard_normal(n, dtype=np.float32)
            act = int(rng.integers(0, 5))
            got = dev.linear(a, w, bias, act=act)
            want = oracle.linear(a, w, bias, act=act)
            tensor_core = m >= 64 and n >= 64 and k >= 32 and k % 4 == 0
        assert got.shape == want.shape and not np.isnan(got).any(), (case, m, n, k)
        err = oracle.rel_frobenius(got, want)
        assert err <= (TF32_TOL if tensor_core else 2e-5), (case, m, n, k, err)


# ---- FP16 operands, FP32 result (launch_matmul_kernel_fp16, matmul.cuh:27-30) -----------------------

@pytest.mark.parametrize("m,n,k,ctas", [
    (256, 256, 64, 1), (256, 256, 64, 2),          # one K block
    (640, 768, 416, 1), (640, 768, 416, 2),        # several tiles, 6.5 K blocks
    (300, 520, 1000, 2),                           # ragged M, N a multiple of 8 but not of 64: B loaded chunk by chunk
    (130, 72, 64, 1),                              # barely more than one tile row
    (2048, 2048, 2048, 2),
])
def test_fp16_tensor_core_gemm(dev, oracle, m, n, k, ctas):
    """FP16 x FP16 products are exact in FP32, so only the FP32 accumulation separates the result from
    the float64 product: the strict-FP32 bar applies, scaled like the accumulation error with K."""
    rng = np.random.default_rng(m + n + k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    b = rng.standard_normal((k, n)).astype(np.float16)
    got = dev.matmul_f16(a, b, ctas=ctas)
    want = oracle.gemm(a.astype(np.float32), b.astype(np.float32))
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, want) <= FP32_TOL * max(1.0, k / 4096.0)


@pytest.mark.parametrize("m,n,k", [(2, 2, 3), (33, 17, 20), (64, 64, 60), (100, 260, 36), (512, 512, 512)])
def test_fp16_launcher_any_shape(dev, oracle, m, n, k):
    """The launcher takes every shape: tensor cores where aligned and large enough, SIMT otherwise."""
    rng = np.random.default_rng(m * 3 + n * 5 + k)
    a = rng.standard_normal((m, k)).astype(np.float16)
    b = rng.standard_normal((k, n)).astype(np.float16)
    got = dev.matmul_f16(a, b)
    want = oracle.gemm(a.astype(np.float32), b.astype(np.float32))
    assert oracle.rel_frobenius(got, want) <= FP32_TOL


@pytest.mark.parametrize("m,n,k", [
    (256, 256, 64), (640, 768, 416), (300, 520, 1000), (2048, 2048, 2048),      # tensor cores: one CTA and CTA pairs
    (2, 2, 3), (33, 17, 20), (100, 260, 36),                                      # SIMT: small or unaligned
])
def test_bf16_launcher(dev, lib, oracle, m, n, k):
    """BF16 operands on the FP16 mainloop (the MMA's operand-format bits are the only difference).  BF16
    products are exact in FP32, so the result is the float64 product of the BF16 values up to FP32
    accumulation - the strict bar; a kernel that read the bits as FP16 would miss it by orders of magnitude."""
    import torch
    rng = np.random.default_rng(m * 7 + n + k)
    ta = torch.from_numpy(rng.standard_normal((m, k), dtype=np.float32)).to(torch.bfloat16).to(dev.dev)
    tb = torch.from_numpy(rng.standard_normal((k, n), dtype=np.float32)).to(torch.bfloat16).to(dev.dev)
    tc = dev.empty((m, n))
    dev.check(lib.cudeep_b200_matmul_bf16(dev.ptr(ta), dev.ptr(tb), dev.ptr(tc), m, n, k, None))
    assert dev.sync_status() == 0
    got = tc.cpu().numpy()
    want = oracle.gemm(ta.float().cpu().numpy(), tb.float().cpu().numpy())
    assert not np.isnan(got).any()
    assert oracle.rel_frobenius(got, want) <= FP32_TOL * max(1.0, k / 4096.0)


# ---- transposed operands (the products of matmul's backward pass) ---------------------------------

@pytest.mark.parametrize("m,n,k", [
    (512, 512, 256),      # CTA pair, chunked A and B loads
    (384, 260, 200),      # N not a multiple of 32: B loaded chunk by chunk
    (132, 512, 96),       # M not a multiple of 32: A loaded chunk by chunk
    (1024, 2048, 520),    # several tiles, odd number of K blocks with a partial last one
    (66, 70, 50),         # extents not multiples of 4: strict FP32 path
    (8, 6, 4),
])
def test_matmul_tn(dev, lib, oracle, m, n, k):
    rng = np.random.default_rng(m + n + k)
    a_km = rng.standard_normal((k, m), dtype=np.float32)          # A stored transposed
    b = rng.standard_normal((k, n), dtype=np.float32)
    ta, tb = dev.to_dev(a_km), dev.to_dev(b)
    tc = dev.empty((m, n))
    dev.check(lib.cudeep_b200_matmul_tn_f32(dev.ptr(ta), dev.ptr(tb), dev.ptr(tc), m, n, k, None))
    assert dev.sync_status() == 0
    got = tc.cpu().numpy()
    a = np.ascontiguousarray(a_km.T)
    if m >= 64 and n >= 64 and k >= 32 and m % 4 == 0 and n % 4 == 0:
        check_tf32(oracle, got, a, b, k)
    else:
        assert oracle.rel_frobenius(got, oracle.gemm(a, b)) <= FP32_TOL


@pytest.mark.parametrize("m,n,k", [(512, 768, 256), (130, 100, 72), (8, 10, 6)])
def test_matmul_nt(dev, lib, oracle, m, n, k):
    rng = np.random.default_rng(m * 3 + n + k)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b_nk = rng.standard_normal((n, k), dtype=np.float32)
    ta, tb = dev.to_dev(a), dev.to_dev(b_nk)
    tc = dev.empty((m, n))
    dev.check(lib.cudeep_b200_matmul_nt_f32(dev.ptr(ta), dev.ptr(tb), dev.ptr(tc), m, n, k, None))
    assert dev.sync_status() == 0
    got = tc.cpu().numpy()
    if m >= 64 and n >= 64 and k >= 32 and k % 4 == 0:
        check_tf32(oracle, got, a, b_nk, k, b_is_nk=True)
    else:
        assert oracle.rel_frobenius(got, oracle.gemm(a, b_nk, b_is_nk=True)) <= FP32_TOL


def test_matmul_backward_products_match_transposed_copies(dev, lib, oracle):
    """grad_a = grad b^T and grad_b = a^T grad against the reference's way of computing them
    (explicit transposed copies, then a plain matmul), both through this library."""
    rng = np.random.default_rng(99)
    a = rng.standard_normal((640, 384), dtype=np.float32)
    b = rng.standard_normal((384, 512), dtype=np.float32)
    grad = rng.standard_normal((640, 512), dtype=np.float32)
    ta, tb, tg = dev.to_dev(a), dev.to_dev(b), dev.to_dev(grad)
    ga, gb = dev.empty((640, 384)), dev.empty((384, 512))
    dev.check(lib.cudeep_b200_matmul_nt_f32(dev.ptr(tg), dev.ptr(tb), dev.ptr(ga), 640, 384, 512, None))
    dev.check(lib.cudeep_b200_matmul_tn_f32(dev.ptr(ta), dev.ptr(tg), dev.ptr(gb), 384, 512, 640, None))
    assert dev.sync_status() == 0
    ga_ref = dev.matmul(grad, np.ascontiguousarray(b.T))
    gb_ref = dev.matmul(np.ascontiguousarray(a.T), grad)
    assert oracle.rel_frobenius(ga.cpu().numpy(), ga_ref) <= TF32_MODEL_TOL
    assert oracle.rel_frobenius(gb.cpu().numpy(), gb_ref) <= TF32_MODEL_TOL
    assert oracle.rel_frobenius(gb.cpu().numpy(), oracle.gemm(np.ascontiguousarray(a.T), grad)) <= TF32_TOL


# ---- fused epilogues and Linear -----------------------------------------------------------

@pytest.mark.parametrize("act", [0, 1, 2, 3, 4])
def test_fused_activation(dev, lib, oracle, act):
    rng = np.random.default_rng(act)
    m, n, k = 256, 512, 128
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32) * np.float32(0.2)
    ta, tb = dev.to_dev(a), dev.to_dev(b)
    tc = dev.empty((m, n))
    dev.check(lib.cudeep_b200_matmul_fused_act(dev.ptr(ta), dev.ptr(tb), dev.ptr(tc), m, n, k, act, None))
    assert dev.sync_status() == 0
    check_tf32(oracle, tc.cpu().numpy(), a, b, k, act=act)


@pytest.mark.parametrize("m,n,k", [(256, 512, 128), (130, 100, 72), (8, 10, 6)])
@pytest.mark.parametrize("act", [0, 2])
def test_linear_forward(dev, oracle, m, n, k, act):
    rng = np.random.default_rng(m + act)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.uniform(-0.3, 0.3, (n, k)).astype(np.float32)
    bias = rng.uniform(-0.5, 0.5, n).astype(np.float32)
    got = dev.linear(x, w, bias, act=act)
    if m >= 64 and n >= 64 and k >= 32 and k % 4 == 0:
        check_tf32(oracle, got, x, w, k, b_is_nk=True, bias=bias, act=act)
    else:
        assert oracle.rel_frobenius(got, oracle.linear(x, w, bias, act=act)) <= 2e-5


def test_linear_known_weights(dev):
    w = np.array([[1, 0, 0], [0, 1, 0]], np.float32)
    x = np.array([[1, 2, 3], [4, 5, 6]], np.float32)
    assert np.allclose(dev.linear(x, w), [[1, 2], [4, 5]], rtol=1e-5)               # test_nn.py:50-62
    y = dev.linear(np.array([[1, 2]], np.float32), np.eye(2, dtype=np.float32), np.array([100, 200], np.float32))
    assert np.allclose(y, [[101, 202]], rtol=1e-5)                                   # test_nn.py:64-76


def test_c3_linear_stack_reduced_batch(dev, oracle):
    """C3's layer widths and initialisation at batch 256 (the oracle finishes in seconds)."""
    x, w1, b1, w2, b2 = workloads.c3_linear_stack(batch=256)
    h = dev.linear(x, w1, b1, act=2)
    y = dev.linear(h, w2, b2)
    h_ref = oracle.linear(x, w1, b1, act=2)
    assert oracle.rel_frobenius(h, h_ref) <= TF32_TOL
    y_ref = oracle.linear(h_ref.astype(np.float32), w2, b2)
    assert oracle.rel_frobenius(y, y_ref) <= TF32_TOL


def test_c3_linear_stack_full_batch_sampled_rows(dev, oracle):
    """C3 as specified: X[8192, 4096] -> Linear(4096 -> 16384, bias, GELU) -> Linear(16384 -> 4096, bias),
    both layers through the fused launch the benchmark times.  The float64 oracle checks 64 sampled rows
    (all columns) of the hidden activation and of the output; column checksums cover every tile."""
    x, w1, b1, w2, b2 = workloads.c3_linear_stack()
    m = x.shape[0]
    h = dev.linear(x, w1, b1, act=2)
    y = dev.linear(h, w2, b2)
    assert h.shape == (8192, 16384) and y.shape == (8192, 4096)
    assert not np.isnan(h).any() and not np.isnan(y).any()
    rows = np.sort(np.random.default_rng(33).choice(m, size=64, replace=False))
    check_tf32(oracle, h, x, w1, 4096, b_is_nk=True, bias=b1, act=2, rows=rows)
    # layer 2 on the hidden rows the GPU produced (isolates the second launch) ...
    check_tf32(oracle, y, h, w2, 16384, b_is_nk=True, bias=b2, rows=rows)
    # ... and the whole stack against float64 from the inputs
    h_ref = oracle.linear(x[rows], w1, b1, act=2)
    y_ref = oracle.linear(h_ref.astype(np.float32), w2, b2)
    assert oracle.rel_frobenius(y[rows], y_ref) <= TF32_TOL
    # column checksums over all 8192 rows: sum_i (H W2^T + b2)[i, :] = (sum_i H[i, :]) W2^T + m b2,
    # and the same identity for layer 1 launched without its activation
    want = h.sum(axis=0, dtype=np.float64) @ w2.astype(np.float64).T + m * b2.astype(np.float64)
    got = y.sum(axis=0, dtype=np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= TF32_TOL
    del y
    pre = dev.linear(x, w1, b1, act=0)
    want = x.sum(axis=0, dtype=np.float64) @ w1.astype(np.float64).T + m * b1.astype(np.float64)
    got = pre.sum(axis=0, dtype=np.float64)
    assert np.linalg.norm(got - want) / np.linalg.norm(want) <= TF32_TOL
    # GELU applied where it should be: the fused output equals the oracle's activation of the
    # pre-activation values this library produced (sampled rows)
    sample = pre[rows[:4]]
    assert np.max(np.abs(h[rows[:4]] - oracle.activation(sample, 2))) <= 2e-5 * max(1.0, float(np.max(np.abs(sample))))


# ---- host-buffer entry point ---------------------------------------------------------------

def test_matmul_host_buffers(lib, cuda, oracle):
    import ctypes
    from cudeep_b200 import _lib
    a, b = workloads.c2_gemm(1024)
    c = np.full((1024, 1024), np.nan, np.float32)
    p = lambda x: x.ctypes.data_as(ctypes.c_void_p)
    _lib.check(lib.cudeep_b200_matmul_host_f32(p(a), p(b), p(c), 1024, 1024, 1024, 0))
    assert _lib.device_status() == 0
    assert oracle.rel_frobenius(c, oracle.gemm(a, b)) <= TF32_TOL
    c2 = np.empty_like(c)
    _lib.check(lib.cudeep_b200_matmul_host_f32(p(a), p(b), p(c2), 1024, 1024, 1024, 1))
    assert oracle.rel_frobenius(c2, oracle.gemm(a, b)) <= FP32_TOL


# ---- bounded waits: a wait that cannot complete ends the kernel with a status, not a hang -----------

@pytest.mark.parametrize("ctas,bn", [(1, 64), (1, 256), (2, 256)])
def test_a_wait_that_runs_out_reports_a_status_and_leaves_the_device_usable(dev, lib, oracle, ctas, bn):
    """Diagnostic mode: the producer loads nothing, so the MMA issuer's wait for operands reaches its
    limit (set to 40 ms here).  The kernel must return, the status word must name the role that gave
    up (2 = MMA issuer waiting for operands, or 4 = an epilogue of the pair's second CTA waiting for
    the accumulator), and the next launch must work."""
    import time
    from cudeep_b200 import _lib
    rng = np.random.default_rng(8)
    a = rng.standard_normal((256, 128), dtype=np.float32)
    b = rng.standard_normal((128, 512), dtype=np.float32)
    ta, tb = dev.to_dev(a), dev.to_dev(b)
    tc = dev.empty((256, 512))
    starve, limit_ms = 1 << 31, 40
    t0 = time.time()
    dev.check(lib.cudeep_b200_gemm_tf32_tuned(dev.ptr(ta), dev.ptr(tb), 0, dev.ptr(tc), 256, 512, 128, None, 0, 0,
                                              ctas, bn, 0, 0, 0, starve | (limit_ms << 16), None))
    status = dev.sync_status()                 # synchronises, reads and clears the status word
    elapsed = time.time() - t0
    assert status in (2, 4), status
    assert 0.03 <= elapsed < 5.0               # it waited for the limit, and only about that long
    assert _lib.device_status() == 0           # cleared
    got = dev.gemm_tuned(a, b, False, ctas=ctas, bn=bn)     # the device and the library still work
    check_tf32(oracle, got, a, b, 128)
