"""TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Python face of the CPU oracle (oracle/dense_oracle.c) plus pure-NumPy
restatements of the same functions for cross-checking.  Only tests/, the smoke
test and bench.py's CPU-baseline legs import this module; the library itself
never does.

What each function restates in the reference (KevinWeiss1995/cuDeep):
  gemm / gemm_np      Tensor::matmul, src/tensor.cu:384-420
  linear              nn.Linear.forward, python/cuDeep/nn.py:110-115
  conv2d / conv2d_np  conv2d_forward_naive_kernel, src/kernels/conv_kernel.cu:113-159
  activation          include/cudeep/ptx_intrinsics.cuh:531-554 (tanh-form GELU)
  tf32_truncate       operand handling of the TF32 MMA, src/kernels/matmul_kernel.cu:186-201

Parity pin: tests/test_oracle_pins.py replays the reference's own known-answer
tests against these functions.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_build" / "liboracle.so"
REF_LIB_PATH = HERE / "_ref" / "libcudeep_ref.so"
DROPIN_DIR = HERE / "_ref" / "dropin"

EPI_NONE, EPI_RELU, EPI_GELU, EPI_SILU, EPI_SIGMOID = range(5)
INPUT_EXACT, INPUT_TF32_TRUNC, INPUT_TF32_ROUND = range(3)

_lib = None


def reference_dir() -> Path | None:
    """Root of a cuDeep checkout: $CUDEEP_REFERENCE_DIR, else a directory named `reference`
    beside this repository; None when neither holds the reference's sources."""
    import os
    candidates = [os.environ.get("CUDEEP_REFERENCE_DIR"), HERE.parent.parent / "reference"]
    for c in candidates:
        if c and (Path(c) / "src" / "kernels" / "matmul_kernel.cu").exists():
            return Path(c)
    return None


def build(ref: bool = False, dropin: bool = False) -> None:
    """Compile the C oracle.  With ref / dropin and a cuDeep checkout at hand (reference_dir()),
    also the reference's kernels as a checker library, and the drop-in proof (the reference's
    binding module, remaining kernels and C++ tests built on this repository's headers and
    library; see oracle/Makefile)."""
    subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    where = reference_dir()
    targets = (["ref"] if ref else []) + (["dropin"] if dropin else [])
    if targets and where is not None:
        subprocess.run(["make", "-s", "-C", str(HERE), *targets, f"REFERENCE={where}"], check=True)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        _lib = ctypes.CDLL(str(LIB_PATH))
        _lib.oracle_activation.restype = ctypes.c_double
        _lib.oracle_activation.argtypes = [ctypes.c_double, ctypes.c_int]
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def tf32_truncate(x) -> np.ndarray:
    """FP32 values as the TF32 datapath sees them: low 13 mantissa bits dropped."""
    x = _f32(x)
    return (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def tf32_round(x) -> np.ndarray:
    """FP32 values rounded to nearest-even at 10 mantissa bits."""
    x = _f32(x)
    u = x.view(np.uint32).astype(np.uint64)
    finite = (u & 0x7F800000) != 0x7F800000
    r = (u + 0xFFF + ((u >> 13) & 1)) & 0xFFFFE000
    return np.where(finite, r, u).astype(np.uint32).view(np.float32)


def activation(x, act: int) -> np.ndarray:
    x = np.asarray(x, dtype=np.float64)
    if act == EPI_RELU:
        return np.maximum(x, 0.0)
    if act == EPI_GELU:
        return 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    if act == EPI_SILU:
        return x / (1.0 + np.exp(-x))
    if act == EPI_SIGMOID:
        return 1.0 / (1.0 + np.exp(-x))
    return x


def gemm(a, b, *, b_is_nk: bool = False, bias=None, bias_per_row: bool = False, act: int = EPI_NONE,
         input_mode: int = INPUT_EXACT) -> np.ndarray:
    """float64 act(A @ B + bias) from float32 inputs, by the C oracle."""
    a, b = _f32(a), _f32(b)
    m, k = a.shape
    n = b.shape[0] if b_is_nk else b.shape[1]
    assert (b.shape[1] if b_is_nk else b.shape[0]) == k
    bias32 = None if bias is None else _f32(bias)
    c = np.empty((m, n), dtype=np.float64)
    lib().oracle_gemm_f64(_ptr(a), _ptr(b), int(b_is_nk), _ptr(c), m, n, k, _ptr(bias32),
                          int(bias_per_row), int(act), int(input_mode))
    return c


def gemm_np(a, b, *, b_is_nk: bool = False, bias=None, act: int = EPI_NONE,
            input_mode: int = INPUT_EXACT) -> np.ndarray:
    """Same as gemm(), in NumPy float64 (independent of the C code)."""
    a, b = _f32(a), _f32(b)
    if input_mode == INPUT_TF32_TRUNC:
        a, b = tf32_truncate(a), tf32_truncate(b)
    elif input_mode == INPUT_TF32_ROUND:
        a, b = tf32_round(a), tf32_round(b)
    a64, b64 = a.astype(np.float64), b.astype(np.float64)
    c = a64 @ (b64.T if b_is_nk else b64)
    if bias is not None:
        c = c + np.asarray(bias, dtype=np.float64)[None, :]
    return activation(c, act)


def gemm_f64_inputs(a, b, *, b_is_nk: bool = False, bias=None, act: int = EPI_NONE) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float64)
    b = np.ascontiguousarray(b, dtype=np.float64)
    m, k = a.shape
    n = b.shape[0] if b_is_nk else b.shape[1]
    bias64 = None if bias is None else np.ascontiguousarray(bias, dtype=np.float64)
    c = np.empty((m, n), dtype=np.float64)
    lib().oracle_gemm_f64_in64(_ptr(a), _ptr(b), int(b_is_nk), _ptr(c), m, n, k, _ptr(bias64), int(act))
    return c


def linear(x, w, bias=None, act: int = EPI_NONE, input_mode: int = INPUT_EXACT) -> np.ndarray:
    """y = act(x @ W^T + b) with W stored [out_features, in_features]."""
    return gemm(x, w, b_is_nk=True, bias=bias, act=act, input_mode=input_mode)


def conv_out_size(size: int, k: int, s: int, p: int) -> int:
    return (size + 2 * p - k) // s + 1


def conv2d(x, w, bias=None, stride=(1, 1), padding=(0, 0), act: int = EPI_NONE,
           input_mode: int = INPUT_EXACT) -> np.ndarray:
    """float64 NCHW x OIHW cross-correlation by the C oracle."""
    x, w = _f32(x), _f32(w)
    n, c, h, wd = x.shape
    oc, c2, kh, kw = w.shape
    assert c == c2
    oh = conv_out_size(h, kh, stride[0], padding[0])
    ow = conv_out_size(wd, kw, stride[1], padding[1])
    bias32 = None if bias is None else _f32(bias)
    out = np.empty((n, oc, oh, ow), dtype=np.float64)
    lib().oracle_conv2d_f64(_ptr(x), _ptr(w), _ptr(bias32), _ptr(out), n, c, oc, h, wd, kh, kw,
                            stride[0], stride[1], padding[0], padding[1], int(act), int(input_mode))
    return out


def conv2d_np(x, w, bias=None, stride=(1, 1), padding=(0, 0), act: int = EPI_NONE) -> np.ndarray:
    """Same as conv2d(), in NumPy float64 (tap-by-tap accumulation)."""
    x = np.asarray(x, dtype=np.float64)
    w = np.asarray(w, dtype=np.float64)
    n, c, h, wd = x.shape
    oc, _, kh, kw = w.shape
    sh, sw = stride
    ph, pw = padding
    oh = conv_out_size(h, kh, sh, ph)
    ow = conv_out_size(wd, kw, sw, pw)
    xp = np.zeros((n, c, h + 2 * ph, wd + 2 * pw), dtype=np.float64)
    xp[:, :, ph:ph + h, pw:pw + wd] = x
    out = np.zeros((n, oc, oh, ow), dtype=np.float64)
    for r in range(kh):
        for s in range(kw):
            patch = xp[:, :, r:r + sh * (oh - 1) + 1:sh, s:s + sw * (ow - 1) + 1:sw]
            out += np.einsum("nchw,oc->nohw", patch, w[:, :, r, s])
    if bias is not None:
        out += np.asarray(bias, dtype=np.float64)[None, :, None, None]
    return activation(out, act)


def conv2d_backward_data_np(dy, w, in_hw, stride=(1, 1), padding=(0, 0), input_mode: int = INPUT_EXACT) -> np.ndarray:
    """float64 gradient of conv2d w.r.t. its input: dx[n,c,ih,iw] = sum dy[n,oc,oh,ow] * w[oc,c,kh,kw]
    over the (oc, kh, kw) with oh*s - p + kh == ih (restates col2im_kernel + the weight^T GEMM,
    src/kernels/conv_kernel.cu:345-478)."""
    dy32, w32 = _f32(dy), _f32(w)
    if input_mode == INPUT_TF32_TRUNC:
        dy32, w32 = tf32_truncate(dy32), tf32_truncate(w32)
    dy64, w64 = dy32.astype(np.float64), w32.astype(np.float64)
    n, oc, oh, ow = dy64.shape
    _, c, kh, kw = w64.shape
    h, wd = in_hw
    sh, sw = stride
    ph, pw = padding
    dxp = np.zeros((n, c, h + 2 * ph, wd + 2 * pw), dtype=np.float64)
    for r in range(kh):
        for q in range(kw):
            contrib = np.einsum("nohw,oc->nchw", dy64, w64[:, :, r, q])
            dxp[:, :, r:r + sh * (oh - 1) + 1:sh, q:q + sw * (ow - 1) + 1:sw] += contrib
    return dxp[:, :, ph:ph + h, pw:pw + wd]


def conv2d_backward_weight_np(dy, x, k_hw, stride=(1, 1), padding=(0, 0), input_mode: int = INPUT_EXACT) -> np.ndarray:
    """float64 gradient of conv2d w.r.t. its filters: dw[oc,c,kh,kw] = sum over images and output
    pixels of dy[n,oc,oh,ow] * x[n,c,oh*s-p+kh,ow*s-p+kw] (src/kernels/conv_kernel.cu:486-545).
    input_mode INPUT_TF32_TRUNC first drops both operands to TF32 the way the tensor core does."""
    if input_mode == INPUT_TF32_TRUNC:
        dy, x = tf32_truncate(dy), tf32_truncate(x)
    dy64 = np.asarray(dy, dtype=np.float64)
    x64 = np.asarray(x, dtype=np.float64)
    n, oc, oh, ow = dy64.shape
    _, c, h, wd = x64.shape
    kh, kw = k_hw
    sh, sw = stride
    ph, pw = padding
    xp = np.zeros((n, c, h + 2 * ph, wd + 2 * pw), dtype=np.float64)
    xp[:, :, ph:ph + h, pw:pw + wd] = x64
    dw = np.zeros((oc, c, kh, kw), dtype=np.float64)
    for r in range(kh):
        for q in range(kw):
            patch = xp[:, :, r:r + sh * (oh - 1) + 1:sh, q:q + sw * (ow - 1) + 1:sw]
            dw[:, :, r, q] = np.einsum("nohw,nchw->oc", dy64, patch)
    return dw


def sgemm_f32(a, b) -> np.ndarray:
    """FP32-accumulating host GEMM (the timed CPU baseline kernel)."""
    a, b = _f32(a), _f32(b)
    m, k = a.shape
    n = b.shape[1]
    c = np.empty((m, n), dtype=np.float32)
    lib().oracle_sgemm_f32(_ptr(a), _ptr(b), _ptr(c), m, n, k)
    return c


def cpu_sgemm(a, b) -> np.ndarray:
    """FP32 host GEMM through NumPy's BLAS (all host threads): the timed CPU baseline."""
    return _f32(a) @ _f32(b)


def cpu_threads() -> int:
    """Threads the BLAS behind cpu_sgemm uses."""
    try:
        from threadpoolctl import threadpool_info
        counts = [int(i.get("num_threads", 0)) for i in threadpool_info() if i.get("user_api") == "blas"]
        if counts:
            return max(counts)
    except Exception:
        pass
    import os
    return os.cpu_count() or 1


# ---- error measures used by the parity tests -------------------------------------------

def rel_frobenius(got, want) -> float:
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    denom = np.linalg.norm(want.ravel())
    return float(np.linalg.norm((got - want).ravel()) / (denom if denom > 0 else 1.0))


def tf32_elementwise_bound(a, b, k: int) -> float:
    """Per-element bound 2^-9 * K * max|a| * max|b| for a TF32 product of depth K."""
    return float(2.0 ** -9 * k * np.max(np.abs(a)) * np.max(np.abs(b)))
