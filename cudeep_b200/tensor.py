"""Device tensor and the functional ops of the dense-contraction path.

Mirrors what the reference exposes for this path: the `_cudeep_core.Tensor` class
(src/bindings/module.cpp:91-162: shape / strides / ndim / numel / nbytes / dtype /
is_contiguous / reshape / transpose / contiguous / fill_ / zero_ / matmul / numpy and the
statics zeros / ones / randn / from_numpy), `conv2d_forward` (module.cpp:326-381) and
`broadcast_add` (module.cpp:664-694), plus `linear` for the fused Linear path.  Forward only:
the autograd tape of python/cuDeep/autograd.py is outside this library's scope.

Every operation goes through the C ABI of libcudeep_b200.so; there is no NumPy fallback.
Errors surface as RuntimeError (CudeepError), as they do in the reference.
"""
from __future__ import annotations

import ctypes
import enum
from typing import Optional, Sequence

import numpy as np

from . import _lib


class DType(enum.Enum):
    """Element types (include/cudeep/common.cuh:10-14)."""
    float16 = 0
    float32 = 1
    float64 = 2


_NP = {DType.float32: np.float32, DType.float64: np.float64}
EPILOGUE = {None: 0, "none": 0, "relu": 1, "gelu": 2, "silu": 3, "sigmoid": 4}


def _epilogue_code(act) -> int:
    if isinstance(act, int):
        if not 0 <= act <= 4:
            raise RuntimeError("unknown epilogue code")
        return act
    try:
        return EPILOGUE[act]
    except KeyError:
        raise RuntimeError(f"unknown activation {act!r}") from None


def _contiguous_strides(shape: Sequence[int]) -> list[int]:
    strides, acc = [], 1
    for s in reversed(shape):
        strides.append(acc)
        acc *= s
    return list(reversed(strides))


class _Storage:
    """A pool block, returned to the pool when the last view of it goes away.  `stream` is the
    stream its tensor last worked on: the pool lets other streams have the block only after
    that stream has drained."""

    def __init__(self, nbytes: int, stream=None):
        self.ptr = ctypes.c_void_p()
        self.stream = stream
        _lib.check(_lib.load().cudeep_b200_pool_alloc_on_stream(max(int(nbytes), 1), stream,
                                                                ctypes.byref(self.ptr)))

    def __del__(self):
        try:
            if self.ptr:
                _lib.load().cudeep_b200_pool_free_on_stream(self.ptr, self.stream)
        except Exception:
            pass


class Tensor:
    def __init__(self, shape: Sequence[int], dtype: DType = DType.float32, *, _storage=None, _strides=None):
        self._shape = [int(s) for s in shape]
        if any(s < 0 for s in self._shape):
            raise RuntimeError("Tensor: negative extent")
        if dtype not in _NP:
            raise RuntimeError("Tensor: only float32 and float64 are supported on this path")
        self._dtype = dtype
        self._strides = list(_strides) if _strides is not None else _contiguous_strides(self._shape)
        self._storage = _storage if _storage is not None else _Storage(self.nbytes())
        self._stream = getattr(self._storage, "stream", None)

    @property
    def stream(self):
        """cudaStream_t (int / c_void_p) this tensor's operations are queued on; None = legacy default."""
        return self._stream

    @stream.setter
    def stream(self, value):
        self._stream = value
        self._storage.stream = value

    def set_stream(self, stream) -> None:
        """Accepts a Stream object or a raw handle (Tensor::set_stream, include/cudeep/tensor.cuh).
        A Stream object is kept alive for as long as the storage that was used on it."""
        self.stream = getattr(stream, "handle", stream)
        self._storage.stream_owner = stream

    # ---- metadata ------------------------------------------------------------------------
    def shape(self) -> list[int]:
        return list(self._shape)

    def strides(self) -> list[int]:
        return list(self._strides)

    def ndim(self) -> int:
        return len(self._shape)

    def numel(self) -> int:
        n = 1
        for s in self._shape:
            n *= s
        return n

    def itemsize(self) -> int:
        return 4 if self._dtype == DType.float32 else 8

    def nbytes(self) -> int:
        return self.numel() * self.itemsize()

    def dtype(self) -> DType:
        return self._dtype

    def is_contiguous(self) -> bool:
        return self._strides == _contiguous_strides(self._shape)

    def data_ptr(self) -> int:
        return int(self._storage.ptr.value or 0)

    def __repr__(self) -> str:
        return f"cuDeep.Tensor(shape={self._shape}, dtype={self._dtype.name})"

    # ---- factories -----------------------------------------------------------------------
    @staticmethod
    def zeros(shape, dtype: DType = DType.float32) -> "Tensor":
        return Tensor(shape, dtype).fill_(0.0)

    @staticmethod
    def ones(shape, dtype: DType = DType.float32) -> "Tensor":
        return Tensor(shape, dtype).fill_(1.0)

    @staticmethod
    def randn(shape, dtype: DType = DType.float32, seed: Optional[int] = None) -> "Tensor":
        """Standard-normal values.  The reference draws them with a time-seeded cuRAND generator
        (src/tensor.cu:158-206); here they come from NumPy so that a seed reproduces them."""
        rng = np.random.default_rng(seed)
        return Tensor.from_numpy(rng.standard_normal(tuple(shape)).astype(_NP[dtype]))

    @staticmethod
    def from_numpy(arr) -> "Tensor":
        arr = np.asarray(arr)
        if arr.dtype == np.float32:
            dtype = DType.float32
        elif arr.dtype == np.float64:
            dtype = DType.float64
        else:
            raise RuntimeError("Unsupported numpy dtype")
        arr = np.ascontiguousarray(arr)
        t = Tensor(arr.shape, dtype)
        if arr.nbytes:
            _lib.check(_lib.load().cudeep_b200_memcpy_h2d(t._storage.ptr, arr.ctypes.data_as(ctypes.c_void_p),
                                                          arr.nbytes, None))
        return t

    def numpy(self) -> np.ndarray:
        src = self if self.is_contiguous() else self.contiguous()
        out = np.empty(tuple(self._shape), dtype=_NP[self._dtype])
        if out.nbytes:
            lib = _lib.load()
            if self.stream is not None:
                _lib.check(lib.cudeep_b200_stream_synchronize(self.stream))
            _lib.check(lib.cudeep_b200_memcpy_d2h(out.ctypes.data_as(ctypes.c_void_p), src._storage.ptr,
                                                  out.nbytes, None))
        return out

    # ---- views and copies ----------------------------------------------------------------
    def reshape(self, new_shape) -> "Tensor":
        new_shape = [int(s) for s in new_shape]
        if -1 in new_shape:
            known = 1
            for s in new_shape:
                if s != -1:
                    known *= s
            new_shape[new_shape.index(-1)] = self.numel() // max(known, 1)
        n = 1
        for s in new_shape:
            n *= s
        if n != self.numel():
            raise RuntimeError("reshape: element count mismatch")
        base = self if self.is_contiguous() else self.contiguous()
        out = Tensor(new_shape, self._dtype, _storage=base._storage)
        out.stream = self.stream
        return out

    def transpose(self, dim0: int, dim1: int) -> "Tensor":
        nd = self.ndim()
        if not (-nd <= dim0 < nd and -nd <= dim1 < nd):
            raise RuntimeError("transpose: dimension out of range")
        dim0 %= nd
        dim1 %= nd
        shape, strides = self.shape(), self.strides()
        shape[dim0], shape[dim1] = shape[dim1], shape[dim0]
        strides[dim0], strides[dim1] = strides[dim1], strides[dim0]
        out = Tensor(shape, self._dtype, _storage=self._storage, _strides=strides)
        out.stream = self.stream
        return out

    def contiguous(self) -> "Tensor":
        if self.is_contiguous():
            return self
        out = Tensor(self._shape, self._dtype)
        out.stream = self.stream
        nd = self.ndim()
        shape = (ctypes.c_longlong * nd)(*self._shape)
        strides = (ctypes.c_longlong * nd)(*self._strides)
        _lib.check(_lib.load().cudeep_b200_strided_copy(self._storage.ptr, out._storage.ptr, nd, shape, strides,
                                                        self.itemsize(), self.stream))
        return out

    def fill_(self, value: float) -> "Tensor":
        if not self.is_contiguous():
            raise RuntimeError("fill_: tensor must be contiguous")
        lib = _lib.load()
        fn = lib.cudeep_b200_fill_f32 if self._dtype == DType.float32 else lib.cudeep_b200_fill_f64
        _lib.check(fn(self._storage.ptr, float(value), self.numel(), self.stream))
        return self

    def zero_(self) -> "Tensor":
        return self.fill_(0.0)

    # ---- the hot path --------------------------------------------------------------------
    def matmul(self, other: "Tensor", *, strict_fp32: bool = False) -> "Tensor":
        """2-D product.  Same checks as Tensor::matmul (src/tensor.cu:384-420): both operands 2-D,
        same dtype, inner extents equal, contiguous.  float32 uses TF32 tensor cores for large
        aligned shapes unless strict_fp32 is set; float64 is computed in FP64."""
        if not isinstance(other, Tensor):
            raise RuntimeError("matmul: operand must be a Tensor")
        if self.ndim() != 2 or other.ndim() != 2:
            raise RuntimeError("matmul requires 2-D tensors")
        if self._dtype != other._dtype:
            raise RuntimeError("matmul: dtype mismatch")
        if self._shape[1] != other._shape[0]:
            raise RuntimeError("matmul: inner dimensions do not match")
        if not (self.is_contiguous() and other.is_contiguous()):
            raise RuntimeError("matmul requires contiguous tensors")
        m, k = self._shape
        n = other._shape[1]
        out = Tensor([m, n], self._dtype)
        out.stream = self.stream
        lib = _lib.load()
        if self._dtype == DType.float64:
            fn = lib.cudeep_b200_matmul_f64
        else:
            fn = lib.cudeep_b200_matmul_f32_strict if strict_fp32 else lib.cudeep_b200_matmul_f32
        _lib.check(fn(self._storage.ptr, other._storage.ptr, out._storage.ptr, m, n, k, self.stream))
        return out

    __matmul__ = matmul

    def _matmul_variant(self, other: "Tensor", which: str) -> "Tensor":
        if self.ndim() != 2 or other.ndim() != 2 or self._dtype != DType.float32 or other._dtype != DType.float32:
            raise RuntimeError(f"matmul_{which}: 2-D float32 tensors expected")
        if not (self.is_contiguous() and other.is_contiguous()):
            raise RuntimeError(f"matmul_{which} requires contiguous tensors")
        lib = _lib.load()
        if which == "nt":            # self [M,K] x other[N,K]^T
            (m, k), (n, k2) = self._shape, other._shape
            fn = lib.cudeep_b200_matmul_nt_f32
        else:                        # self[K,M]^T x other[K,N]
            (k, m), (k2, n) = self._shape, other._shape
            fn = lib.cudeep_b200_matmul_tn_f32
        if k != k2:
            raise RuntimeError(f"matmul_{which}: inner dimensions do not match")
        out = Tensor([m, n], self._dtype)
        out.stream = self.stream
        _lib.check(fn(self._storage.ptr, other._storage.ptr, out._storage.ptr, m, n, k, self.stream))
        return out

    def matmul_nt(self, other: "Tensor") -> "Tensor":
        """self @ other^T without materialising the transpose (other is [N, K])."""
        return self._matmul_variant(other, "nt")

    def matmul_tn(self, other: "Tensor") -> "Tensor":
        """self^T @ other without materialising the transpose (self is [K, M])."""
        return self._matmul_variant(other, "tn")

    def _activation(self, act: int) -> "Tensor":
        if self._dtype != DType.float32:
            raise RuntimeError("activations are float32 only")
        src = self if self.is_contiguous() else self.contiguous()
        out = Tensor(self._shape, self._dtype)
        out.stream = self.stream
        _lib.check(_lib.load().cudeep_b200_activation_f32(src._storage.ptr, out._storage.ptr, self.numel(), act,
                                                          self.stream))
        return out

    def relu(self):
        return self._activation(1)

    def gelu(self):
        return self._activation(2)

    def silu(self):
        return self._activation(3)

    def sigmoid(self):
        return self._activation(4)


# ---- functional ops ------------------------------------------------------------------------

def broadcast_add(matrix: Tensor, row: Tensor) -> Tensor:
    """out[i, j] = matrix[i, j] + row[j]  (module.cpp:664-694)."""
    if matrix.ndim() != 2 or row.numel() != matrix.shape()[1] or matrix.dtype() != row.dtype():
        raise RuntimeError("broadcast_add: expected [rows, cols] + [cols] of one dtype")
    m = matrix if matrix.is_contiguous() else matrix.contiguous()
    r = row if row.is_contiguous() else row.contiguous()
    out = Tensor(matrix.shape(), matrix.dtype())
    out.stream = matrix.stream
    lib = _lib.load()
    fn = lib.cudeep_b200_broadcast_add_f32 if matrix.dtype() == DType.float32 else lib.cudeep_b200_broadcast_add_f64
    _lib.check(fn(m._storage.ptr, r._storage.ptr, out._storage.ptr, matrix.shape()[0], matrix.shape()[1],
                  matrix.stream))
    return out


def matmul_backward(a: Tensor, b: Tensor, grad: Tensor):
    """Gradients of c = a @ b: (grad @ b^T, a^T @ grad), the two products of MatMulOp.backward
    (python/cuDeep/tensor.py:430-443) without its transposed copies."""
    return grad.matmul_nt(b), a.matmul_tn(grad)


def linear(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, activation=None) -> Tensor:
    """act(x @ weight^T + bias) in one kernel; weight is [out_features, in_features] as nn.Linear
    stores it (python/cuDeep/nn.py:104-115).  Leading dimensions of x are flattened."""
    if weight.ndim() != 2 or x.ndim() < 1 or x.shape()[-1] != weight.shape()[1]:
        raise RuntimeError("linear: x[..., in_features] and weight[out_features, in_features] expected")
    if x.dtype() != weight.dtype() or (bias is not None and bias.dtype() != x.dtype()):
        raise RuntimeError("linear: dtype mismatch")
    if bias is not None and bias.numel() != weight.shape()[0]:
        raise RuntimeError("linear: bias must have out_features elements")
    act = _epilogue_code(activation)
    xc = x if x.is_contiguous() else x.contiguous()
    wc = weight if weight.is_contiguous() else weight.contiguous()
    bc = None if bias is None else (bias if bias.is_contiguous() else bias.contiguous())
    k = weight.shape()[1]
    n = weight.shape()[0]
    m = xc.numel() // k
    out = Tensor(x.shape()[:-1] + [n], x.dtype())
    out.stream = x.stream
    lib = _lib.load()
    fn = lib.cudeep_b200_linear_forward_f32 if x.dtype() == DType.float32 else lib.cudeep_b200_linear_forward_f64
    _lib.check(fn(xc._storage.ptr, wc._storage.ptr, None if bc is None else bc._storage.ptr, out._storage.ptr,
                  m, n, k, act, x.stream))
    return out


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def conv2d(x: Tensor, weight: Tensor, bias: Optional[Tensor] = None, stride=(1, 1), padding=(0, 0),
           activation=None) -> Tensor:
    """NCHW x OIHW cross-correlation with zero padding (module.cpp:326-381); `activation` is fused
    into the epilogue."""
    if x.ndim() != 4 or weight.ndim() != 4:
        raise RuntimeError("conv2d: input [N,C,H,W] and weight [OC,C,KH,KW] expected")
    if x.shape()[1] != weight.shape()[1]:
        raise RuntimeError("conv2d: channel mismatch")
    if x.dtype() != weight.dtype() or (bias is not None and bias.dtype() != x.dtype()):
        raise RuntimeError("conv2d: dtype mismatch")
    (sh, sw), (ph, pw) = _pair(stride), _pair(padding)
    n, c, h, w = x.shape()
    oc, _, kh, kw = weight.shape()
    if bias is not None and bias.numel() != oc:
        raise RuntimeError("conv2d: bias must have out_channels elements")
    act = _epilogue_code(activation)
    if sh <= 0 or sw <= 0 or h + 2 * ph < kh or w + 2 * pw < kw:
        raise RuntimeError("conv2d: bad stride or kernel larger than the padded input")
    oh, ow = (h + 2 * ph - kh) // sh + 1, (w + 2 * pw - kw) // sw + 1
    xc = x if x.is_contiguous() else x.contiguous()
    wc = weight if weight.is_contiguous() else weight.contiguous()
    bc = None if bias is None else (bias if bias.is_contiguous() else bias.contiguous())
    out = Tensor([n, oc, oh, ow], x.dtype())
    out.stream = x.stream
    lib = _lib.load()
    bptr = None if bc is None else bc._storage.ptr
    if x.dtype() == DType.float32:
        _lib.check(lib.cudeep_b200_conv2d_forward_fused_f32(xc._storage.ptr, wc._storage.ptr, bptr, out._storage.ptr,
                                                            n, c, oc, h, w, kh, kw, sh, sw, ph, pw, act, x.stream))
    else:
        if act != 0:
            raise RuntimeError("conv2d: fused activations are float32 only")
        _lib.check(lib.cudeep_b200_conv2d_forward_f64(xc._storage.ptr, wc._storage.ptr, bptr, out._storage.ptr,
                                                      n, c, oc, h, w, kh, kw, sh, sw, ph, pw, x.stream))
    return out


def relu(x: Tensor) -> Tensor:
    return x.relu()


def gelu(x: Tensor) -> Tensor:
    return x.gelu()


def silu(x: Tensor) -> Tensor:
    return x.silu()


def sigmoid(x: Tensor) -> Tensor:
    return x.sigmoid()


class MemoryPool:
    """cudeep::MemoryPool of the current device (include/cudeep/memory.cuh:13-46)."""

    @staticmethod
    def instance() -> "MemoryPool":
        return MemoryPool()

    @staticmethod
    def _stats():
        a, c = ctypes.c_size_t(0), ctypes.c_size_t(0)
        _lib.check(_lib.load().cudeep_b200_pool_stats(ctypes.byref(a), ctypes.byref(c)))
        return a.value, c.value

    def allocated_bytes(self) -> int:
        return self._stats()[0]

    def cached_bytes(self) -> int:
        return self._stats()[1]

    def release_cached(self) -> None:
        _lib.check(_lib.load().cudeep_b200_pool_release_cached())


class Stream:
    """RAII stream (include/cudeep/stream.cuh:8-24)."""

    def __init__(self):
        self.handle = ctypes.c_void_p()
        _lib.check(_lib.load().cudeep_b200_stream_create(ctypes.byref(self.handle)))

    def synchronize(self) -> None:
        _lib.check(_lib.load().cudeep_b200_stream_synchronize(self.handle))

    def __del__(self):
        try:
            if self.handle:
                _lib.load().cudeep_b200_stream_destroy(self.handle)
        except Exception:
            pass


class Event:
    """RAII event with record / synchronize / elapsed_ms (include/cudeep/stream.cuh:26-44)."""

    def __init__(self):
        self.handle = ctypes.c_void_p()
        _lib.check(_lib.load().cudeep_b200_event_create(ctypes.byref(self.handle)))

    def record(self, stream: Optional[Stream] = None) -> None:
        _lib.check(_lib.load().cudeep_b200_event_record(self.handle, None if stream is None else stream.handle))

    def synchronize(self) -> None:
        _lib.check(_lib.load().cudeep_b200_event_synchronize(self.handle))

    def elapsed_ms(self, start: "Event") -> float:
        ms = ctypes.c_float(0.0)
        _lib.check(_lib.load().cudeep_b200_event_elapsed_ms(start.handle, self.handle, ctypes.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            if self.handle:
                _lib.load().cudeep_b200_event_destroy(self.handle)
        except Exception:
            pass


def device_info() -> dict:
    """module.cpp:642-658."""
    dev, sms, major, minor = (ctypes.c_int(0) for _ in range(4))
    total = ctypes.c_size_t(0)
    _lib.check(_lib.load().cudeep_b200_device_info(ctypes.byref(dev), ctypes.byref(sms), ctypes.byref(major),
                                                   ctypes.byref(minor), ctypes.byref(total)))
    return {"device": dev.value, "sm_count": sms.value, "compute_capability": (major.value, minor.value),
            "total_memory": total.value}
