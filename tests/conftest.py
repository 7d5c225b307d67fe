import ctypes
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def lib():
    """The C-ABI library; building it needs nvcc only."""
    from cudeep_b200 import _lib
    if not _lib.LIB_PATH.exists():
        from cudeep_b200 import build
        build.build()
    return _lib.load()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.lib()
    return o


@pytest.fixture(scope="session")
def cuda():
    """torch on cuda:0 — used only to hold device buffers for the C-ABI calls."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


class DeviceOps:
    """Thin helpers around the C ABI working on torch-held device buffers."""

    def __init__(self, lib, torch):
        self.lib = lib
        self.torch = torch
        self.dev = torch.device("cuda:0")

    def to_dev(self, a):
        return self.torch.from_numpy(np.ascontiguousarray(a)).to(self.dev)

    @staticmethod
    def ptr(t):
        return None if t is None else ctypes.c_void_p(t.data_ptr())

    def check(self, rc):
        from cudeep_b200 import _lib
        _lib.check(rc)

    def sync_status(self):
        from cudeep_b200 import _lib
        self.torch.cuda.synchronize()
        return _lib.device_status(True)

    def empty(self, shape, dtype=None, poison=True):
        t = self.torch.empty(shape, device=self.dev, dtype=dtype or self.torch.float32)
        if poison:
            t.fill_(float("nan"))
        return t

    def matmul(self, a, b, strict=False):
        ta, tb = self.to_dev(a), self.to_dev(b)
        m, k = a.shape
        n = b.shape[1]
        tc = self.empty((m, n))
        fn = self.lib.cudeep_b200_matmul_f32_strict if strict else self.lib.cudeep_b200_matmul_f32
        self.check(fn(self.ptr(ta), self.ptr(tb), self.ptr(tc), m, n, k, None))
        assert self.sync_status() == 0
        return tc.cpu().numpy()

    def gemm_tuned(self, a, b, b_is_nk, bias=None, bias_per_row=False, act=0, ctas=0, bn=0, raster=0,
                   max_ctas=0, katoms=0, unchunked=False, split_k=0, cluster_split=0, register_store=False,
                   flip_ring_staging=False):
        ta, tb = self.to_dev(a), self.to_dev(b)
        m, k = a.shape
        n = b.shape[0] if b_is_nk else b.shape[1]
        tbias = self.to_dev(bias) if bias is not None else None
        tc = self.empty((m, n))
        self.check(self.lib.cudeep_b200_gemm_tf32_tuned(
            self.ptr(ta), self.ptr(tb), int(b_is_nk), self.ptr(tc), m, n, k, self.ptr(tbias),
            int(bias_per_row), act, ctas, bn, raster,
            max_ctas | (int(unchunked) << 28) | (katoms << 29),
            (split_k << 16) | (cluster_split << 24) | (int(register_store) << 28) | (int(flip_ring_staging) << 31),
            0, None))
        assert self.sync_status() == 0
        return tc.cpu().numpy()

    def matmul_f16(self, a, b, ctas=None):
        """a, b: float16 arrays; returns float32.  ctas None: the launcher's own choice of path."""
        ta, tb = self.to_dev(a), self.to_dev(b)
        m, k = a.shape
        n = b.shape[1]
        tc = self.empty((m, n))
        if ctas is None:
            self.check(self.lib.cudeep_b200_matmul_f16(self.ptr(ta), self.ptr(tb), self.ptr(tc), m, n, k, None))
        else:
            self.check(self.lib.cudeep_b200_matmul_f16_tuned(self.ptr(ta), self.ptr(tb), self.ptr(tc), m, n, k,
                                                             ctas, 0, 0, None))
        assert self.sync_status() == 0
        return tc.cpu().numpy()

    def linear(self, x, w, bias=None, act=0):
        tx, tw = self.to_dev(x), self.to_dev(w)
        tb = self.to_dev(bias) if bias is not None else None
        m, k = x.shape
        n = w.shape[0]
        ty = self.empty((m, n))
        self.check(self.lib.cudeep_b200_linear_forward_f32(self.ptr(tx), self.ptr(tw), self.ptr(tb),
                                                           self.ptr(ty), m, n, k, act, None))
        assert self.sync_status() == 0
        return ty.cpu().numpy()

    def conv2d(self, x, w, bias=None, stride=(1, 1), padding=(0, 0), act=0):
        tx, tw = self.to_dev(x), self.to_dev(w)
        tb = self.to_dev(bias) if bias is not None else None
        n, c, h, wd = x.shape
        oc, _, kh, kw = w.shape
        oh = (h + 2 * padding[0] - kh) // stride[0] + 1
        ow = (wd + 2 * padding[1] - kw) // stride[1] + 1
        ty = self.empty((n, oc, oh, ow))
        self.check(self.lib.cudeep_b200_conv2d_forward_fused_f32(
            self.ptr(tx), self.ptr(tw), self.ptr(tb), self.ptr(ty), n, c, oc, h, wd, kh, kw,
            stride[0], stride[1], padding[0], padding[1], act, None))
        assert self.sync_status() == 0
        return ty.cpu().numpy()


@pytest.fixture(scope="session")
def dev(lib, cuda):
    return DeviceOps(lib, cuda)
