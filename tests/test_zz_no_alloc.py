"""The allocation-free convolution entry point against the regular one (GPU).

cudeep_b200_conv2d_forward_noalloc_f32 serves callers that run with a fixed device-memory
plan (their own allocator owns the free memory, or an allocation's synchronisation or failure
cannot be tolerated mid-step): its scratch is an array built into the library.  The test calls
it twice in a row with different inputs - the array keeps the first call's contents, so the
second call would expose anything that relied on stale or pre-cleared scratch - and compares
each result with cudeep_b200_conv2d_forward_fused_f32 on the same inputs.

This file sorts last so that a run stopping at the first failure has already run every other test.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL = 2e-5   # the parity tests' bound for "same arithmetic, possibly different summation order"


def conv_both(dev, lib, x, w, bias, padding, act):
    from cudeep_b200 import _lib
    n, c, h, wd = x.shape
    oc, _, kh, kw = w.shape
    oh, ow = h + 2 * padding[0] - kh + 1, wd + 2 * padding[1] - kw + 1
    tx, tw, tb = dev.to_dev(x), dev.to_dev(w), dev.to_dev(bias)
    regular = dev.empty((n, oc, oh, ow))
    fixed = dev.empty((n, oc, oh, ow))
    args = (n, c, oc, h, wd, kh, kw, 1, 1, padding[0], padding[1], act, None)
    _lib.check(lib.cudeep_b200_conv2d_forward_fused_f32(dev.ptr(tx), dev.ptr(tw), dev.ptr(tb), dev.ptr(regular), *args))
    _lib.check(lib.cudeep_b200_conv2d_forward_noalloc_f32(dev.ptr(tx), dev.ptr(tw), dev.ptr(tb), dev.ptr(fixed), *args))
    assert dev.sync_status() == 0
    return regular.cpu().numpy(), fixed.cpu().numpy()


def test_noalloc_matches_regular_on_two_calls_in_a_row(dev, lib, oracle):
    rng = np.random.default_rng(2024)
    # first call: larger scratch footprint (48 channels pad to 64 in the packed filters)
    x1 = rng.standard_normal((3, 48, 20, 24), dtype=np.float32)
    w1 = rng.standard_normal((160, 48, 3, 3), dtype=np.float32) * np.float32(0.1)
    b1 = rng.standard_normal(160, dtype=np.float32)
    regular, fixed = conv_both(dev, lib, x1, w1, b1, (1, 1), 1)
    assert not np.isnan(fixed).any()
    assert oracle.rel_frobenius(fixed, regular) <= TOL
    assert oracle.rel_frobenius(fixed, oracle.conv2d(x1, w1, b1, (1, 1), (1, 1), act=1)) <= 5e-3
    # second call: different shape and data, smaller footprint inside the same array
    x2 = rng.standard_normal((2, 32, 14, 14), dtype=np.float32)
    w2 = rng.standard_normal((64, 32, 5, 5), dtype=np.float32) * np.float32(0.1)
    b2 = rng.standard_normal(64, dtype=np.float32)
    regular, fixed = conv_both(dev, lib, x2, w2, b2, (2, 2), 2)
    assert not np.isnan(fixed).any()
    assert oracle.rel_frobenius(fixed, regular) <= TOL
    assert oracle.rel_frobenius(fixed, oracle.conv2d(x2, w2, b2, (1, 1), (2, 2), act=2)) <= 5e-3
    # and the first problem again: the array now holds the second call's leftovers
    regular, fixed = conv_both(dev, lib, x1, w1, b1, (1, 1), 1)
    assert oracle.rel_frobenius(fixed, regular) <= TOL


def test_noalloc_takes_no_device_memory_once_a_shape_class_is_warm(dev, lib):
    """The array and the kernels of a shape class are loaded at their first use; from then on a call
    leaves the device's free memory exactly where it was."""
    from cudeep_b200 import _lib
    rng = np.random.default_rng(3)
    x = rng.standard_normal((2, 32, 14, 14), dtype=np.float32)
    w = rng.standard_normal((64, 32, 3, 3), dtype=np.float32)
    tx, tw = dev.to_dev(x), dev.to_dev(w)
    ty = dev.empty((2, 64, 14, 14))
    args = (2, 32, 64, 14, 14, 3, 3, 1, 1, 1, 1, 0, None)
    assert lib.cudeep_b200_conv2d_noalloc_capacity() == 32 << 20          # resolves the array on this device
    _lib.check(lib.cudeep_b200_conv2d_forward_noalloc_f32(dev.ptr(tx), dev.ptr(tw), None, dev.ptr(ty), *args))
    dev.torch.cuda.synchronize()
    free_before, _ = dev.torch.cuda.mem_get_info()
    for _ in range(3):
        _lib.check(lib.cudeep_b200_conv2d_forward_noalloc_f32(dev.ptr(tx), dev.ptr(tw), None, dev.ptr(ty), *args))
    dev.torch.cuda.synchronize()
    free_after, _ = dev.torch.cuda.mem_get_info()
    assert free_after == free_before


def test_noalloc_refuses_shapes_beyond_its_scratch(dev, lib):
    cap = lib.cudeep_b200_conv2d_noalloc_capacity()
    assert cap == 32 << 20
    # 16 x 256 x 56 x 56 floats = 51 MB of NHWC scratch: too large; nothing is launched
    p = ctypes.c_void_p(dev.torch.empty(1, device=dev.dev).data_ptr())
    rc = lib.cudeep_b200_conv2d_forward_noalloc_f32(p, p, None, p, 16, 256, 256, 56, 56, 3, 3, 1, 1, 1, 1, 0, None)
    assert rc != 0
    msg = lib.cudeep_b200_last_error().decode()
    assert "built-in scratch" in msg and str(cap) in msg


def test_noalloc_runs_direct_kernel_for_shapes_off_the_tensor_core_path(dev, lib, oracle):
    """Six output channels: under the 32 the implicit GEMM needs, so the direct kernel runs (no scratch)."""
    from cudeep_b200 import _lib
    rng = np.random.default_rng(5)
    x = rng.standard_normal((2, 8, 12, 12), dtype=np.float32)
    w = rng.standard_normal((6, 8, 3, 3), dtype=np.float32)
    b = rng.standard_normal(6, dtype=np.float32)
    tx, tw, tb = dev.to_dev(x), dev.to_dev(w), dev.to_dev(b)
    ty = dev.empty((2, 6, 6, 6))
    _lib.check(lib.cudeep_b200_conv2d_forward_noalloc_f32(dev.ptr(tx), dev.ptr(tw), dev.ptr(tb), dev.ptr(ty),
                                                          2, 8, 6, 12, 12, 3, 3, 2, 2, 1, 1, 0, None))
    assert dev.sync_status() == 0
    assert oracle.rel_frobenius(ty.cpu().numpy(), oracle.conv2d(x, w, b, (2, 2), (1, 1))) <= 1e-5
