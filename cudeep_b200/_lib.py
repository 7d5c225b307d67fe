"""ctypes binding of libcudeep_b200.so (the C ABI declared in include/cudeep_b200.h).

The library is the product: there is no Python or CPU fallback.  If the shared
object is missing, `load()` raises and tells the user how to build it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_double, c_float, c_int, c_size_t, c_uint32, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libcudeep_b200.so"

_fp = c_void_p      # device or host pointers are passed as integers / c_void_p
_stream = c_void_p

# name -> (restype, argtypes); mirrors include/cudeep_b200.h declaration by declaration.
PROTOTYPES = {
    "cudeep_b200_version": (c_int, []),
    "cudeep_b200_last_error": (c_char_p, []),
    "cudeep_b200_device_status": (c_int, [c_int, POINTER(c_uint32)]),
    "cudeep_b200_matmul_f32": (c_int, [_fp, _fp, _fp, c_int, c_int, c_int, _stream]),
    "cudeep_b200_matmul_f32_strict": (c_int, [_fp, _fp, _fp, c_int, c_int, c_int, _stream]),
    "cudeep_b200_matmul_f64": (c_int, [_fp, _fp, _fp, c_int, c_int, c_int, _stream]),
    "cudeep_b200_matmul_fused_act": (c_int, [_fp, _fp, _fp, c_int, c_int, c_int, c_int, _stream]),
    "cudeep_b200_linear_forward_f32": (c_int, [_fp, _fp, _fp, _fp, c_int, c_int, c_int, c_int, _stream]),
    "cudeep_b200_linear_forward_f64": (c_int, [_fp, _fp, _fp, _fp, c_int, c_int, c_int, c_int, _stream]),
    "cudeep_b200_matmul_nt_f32": (c_int, [_fp, _fp, _fp, c_int, c_int, c_int, _stream]),
    "cudeep_b200_matmul_tn_f32": (c_int, [_fp, _fp, _fp, c_int, c_int, c_int, _stream]),
    "cudeep_b200_gemm_tf32_tuned": (c_int, [_fp, _fp, c_int, _fp, c_int, c_int, c_int, _fp, c_int, c_int,
                                            c_int, c_int, c_int, c_int, c_uint32, c_uint32, _stream]),
    "cudeep_b200_conv2d_forward_f32": (c_int, [_fp, _fp, _fp, _fp] + [c_int] * 11 + [_stream]),
    "cudeep_b200_conv2d_forward_fused_f32": (c_int, [_fp, _fp, _fp, _fp] + [c_int] * 12 + [_stream]),
    "cudeep_b200_conv2d_forward_fused_nhwc_f32": (c_int, [_fp, _fp, _fp, _fp] + [c_int] * 12 + [_stream]),
    "cudeep_b200_conv2d_forward_f64": (c_int, [_fp, _fp, _fp, _fp] + [c_int] * 11 + [_stream]),
    "cudeep_b200_conv2d_forward_noalloc_f32": (c_int, [_fp, _fp, _fp, _fp] + [c_int] * 12 + [_stream]),
    "cudeep_b200_conv2d_noalloc_capacity": (c_size_t, []),
    "cudeep_b200_conv2d_backward_data_f32": (c_int, [_fp, _fp, _fp] + [c_int] * 11 + [_stream]),
    "cudeep_b200_conv2d_backward_weight_f32": (c_int, [_fp, _fp, _fp] + [c_int] * 11 + [_stream]),
    "cudeep_b200_matmul_host_f32": (c_int, [_fp, _fp, _fp, c_int, c_int, c_int, c_int]),
    "cudeep_b200_linear_forward_host_f32": (c_int, [_fp, _fp, _fp, _fp, c_int, c_int, c_int, c_int]),
    "cudeep_b200_conv2d_forward_host_f32": (c_int, [_fp, _fp, _fp, _fp] + [c_int] * 12),
    "cudeep_b200_memcpy_h2d": (c_int, [c_void_p, c_void_p, c_size_t, _stream]),
    "cudeep_b200_memcpy_d2h": (c_int, [c_void_p, c_void_p, c_size_t, _stream]),
    "cudeep_b200_memcpy_d2d": (c_int, [c_void_p, c_void_p, c_size_t, _stream]),
    "cudeep_b200_stream_synchronize": (c_int, [_stream]),
    "cudeep_b200_device_synchronize": (c_int, []),
    "cudeep_b200_strided_copy": (c_int, [c_void_p, c_void_p, c_int, POINTER(ctypes.c_longlong),
                                         POINTER(ctypes.c_longlong), c_int, _stream]),
    "cudeep_b200_fill_f32": (c_int, [c_void_p, c_float, ctypes.c_longlong, _stream]),
    "cudeep_b200_fill_f64": (c_int, [c_void_p, c_double, ctypes.c_longlong, _stream]),
    "cudeep_b200_broadcast_add_f32": (c_int, [_fp, _fp, _fp, ctypes.c_longlong, c_int, _stream]),
    "cudeep_b200_broadcast_add_f64": (c_int, [_fp, _fp, _fp, ctypes.c_longlong, c_int, _stream]),
    "cudeep_b200_activation_f32": (c_int, [_fp, _fp, ctypes.c_longlong, c_int, _stream]),
    "cudeep_b200_stream_create": (c_int, [POINTER(c_void_p)]),
    "cudeep_b200_stream_destroy": (c_int, [_stream]),
    "cudeep_b200_event_create": (c_int, [POINTER(c_void_p)]),
    "cudeep_b200_event_destroy": (c_int, [c_void_p]),
    "cudeep_b200_event_record": (c_int, [c_void_p, _stream]),
    "cudeep_b200_event_synchronize": (c_int, [c_void_p]),
    "cudeep_b200_event_elapsed_ms": (c_int, [c_void_p, c_void_p, POINTER(c_float)]),
    "cudeep_b200_device_info": (c_int, [POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int),
                                        POINTER(c_size_t)]),
    "cudeep_b200_gemm_tf32_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, POINTER(c_int), POINTER(c_int),
                                           POINTER(c_int), POINTER(c_int), POINTER(c_double)]),
    "cudeep_b200_matmul_f16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "cudeep_b200_matmul_bf16": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "cudeep_b200_matmul_f16_tuned": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             ctypes.c_uint32, ctypes.c_uint32, c_void_p]),
    "cudeep_b200_pool_alloc": (c_int, [c_size_t, POINTER(c_void_p)]),
    "cudeep_b200_pool_free": (c_int, [c_void_p]),
    "cudeep_b200_pool_alloc_on_stream": (c_int, [c_size_t, c_void_p, POINTER(c_void_p)]),
    "cudeep_b200_pool_free_on_stream": (c_int, [c_void_p, c_void_p]),
    "cudeep_b200_pool_release_cached": (c_int, []),
    "cudeep_b200_pool_stats": (c_int, [POINTER(c_size_t), POINTER(c_size_t)]),
    "cudeep_b200_scratch_trim": (c_int, [c_size_t]),
    "cudeep_b200_sharded_gemm_create_local": (c_int, [POINTER(c_int), c_int, ctypes.c_longlong, c_int, c_int, c_int,
                                                      c_int, c_int, POINTER(c_void_p)]),
    "cudeep_b200_sharded_gemm_create_rank": (c_int, [c_int, c_int, c_int, ctypes.c_longlong, c_int, c_int, c_int,
                                                     c_int, c_int, POINTER(c_void_p)]),
    "cudeep_b200_sharded_gemm_destroy": (c_int, [c_void_p]),
    "cudeep_b200_sharded_gemm_rows": (c_int, [c_void_p, c_int, c_int, POINTER(ctypes.c_longlong),
                                              POINTER(ctypes.c_longlong)]),
    "cudeep_b200_sharded_gemm_buffers": (c_int, [c_void_p, c_int, POINTER(c_void_p), POINTER(c_void_p),
                                                 POINTER(c_void_p)]),
    "cudeep_b200_sharded_gemm_read_c": (c_int, [c_void_p, c_int, ctypes.c_longlong, ctypes.c_longlong, c_void_p]),
    "cudeep_b200_sharded_gemm_comm_id": (c_int, [c_void_p]),
    "cudeep_b200_sharded_gemm_init_comm": (c_int, [c_void_p, c_void_p]),
    "cudeep_b200_sharded_gemm_export_c": (c_int, [c_void_p, c_void_p]),
    "cudeep_b200_sharded_gemm_open_peers": (c_int, [c_void_p, c_void_p]),
    "cudeep_b200_sharded_gemm_multicast_fd": (c_int, [c_void_p, POINTER(c_int)]),
    "cudeep_b200_sharded_gemm_multicast_join": (c_int, [c_void_p, c_int]),
    "cudeep_b200_sharded_gemm_multicast_bind": (c_int, [c_void_p]),
    "cudeep_b200_sharded_gemm_run": (c_int, [c_void_p, c_int, _stream]),
    "cudeep_b200_sharded_gemm_synchronize": (c_int, [c_void_p]),
    "cudeep_b200_sharded_gemm_time": (c_int, [c_void_p, c_int, c_int, c_int, POINTER(c_float)]),
    "cudeep_b200_sharded_gemm_steps": (c_int, [c_void_p, c_int, POINTER(ctypes.c_longlong)]),
    "cudeep_b200_sharded_gemm_inject_failure": (c_int, [c_void_p, c_int]),
}

_lib = None


class CudeepError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference raises RuntimeError too)."""


def load() -> ctypes.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH.name} has not been built; run `python -m cudeep_b200.build` "
            "(needs nvcc; cross-compiles for sm_100a without a GPU)")
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        raise CudeepError(load().cudeep_b200_last_error().decode("utf-8", "replace"))


def device_status(clear: bool = True) -> int:
    """Kernel status word of the current device (0 = every pipeline wait completed)."""
    out = c_uint32(0)
    check(load().cudeep_b200_device_status(1 if clear else 0, ctypes.byref(out)))
    return out.value
