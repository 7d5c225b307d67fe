"""The C-ABI library loads without a GPU and exports everything the headers declare (CPU only)."""
import ctypes
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "cudeep_b200.h"

# Itanium-mangled launchers of the reference's C++ surface
# (include/cudeep/kernels/matmul.cuh:8-44 and conv.cuh:8-36 in the cuDeep tree).
CXX_SYMBOLS = [
    "_ZN6cudeep7kernels20launch_matmul_kernelIfEEvPKT_S4_PS2_iiiP11CUstream_st",
    "_ZN6cudeep7kernels20launch_matmul_kernelIdEEvPKT_S4_PS2_iiiP11CUstream_st",
    "_ZN6cudeep7kernels25launch_matmul_kernel_fp32IfEEvPKT_S4_PS2_iiiP11CUstream_st",
    "_ZN6cudeep7kernels25launch_matmul_kernel_fp32IdEEvPKT_S4_PS2_iiiP11CUstream_st",
    "_ZN6cudeep7kernels26launch_matmul_tiled_kernelIfEEvPKT_S4_PS2_iiiiP11CUstream_st",
    "_ZN6cudeep7kernels26launch_matmul_tiled_kernelIdEEvPKT_S4_PS2_iiiiP11CUstream_st",
    "_ZN6cudeep7kernels25launch_matmul_kernel_fp16EPK6__halfS3_PfiiiP11CUstream_st",
    "_ZN6cudeep7kernels23launch_matmul_fused_actEPKfS2_PfiiiNS0_12GemmEpilogueEP11CUstream_st",
    "_ZN6cudeep7kernels28launch_conv2d_forward_kernelIfEEvPKT_S4_S4_PS2_iiiiiiiiiiiP11CUstream_st",
    "_ZN6cudeep7kernels28launch_conv2d_forward_kernelIdEEvPKT_S4_S4_PS2_iiiiiiiiiiiP11CUstream_st",
    "_ZN6cudeep7kernels34launch_conv2d_backward_data_kernelIfEEvPKT_S4_PS2_iiiiiiiiiiiP11CUstream_st",
    "_ZN6cudeep7kernels34launch_conv2d_backward_data_kernelIdEEvPKT_S4_PS2_iiiiiiiiiiiP11CUstream_st",
    "_ZN6cudeep7kernels36launch_conv2d_backward_weight_kernelIfEEvPKT_S4_PS2_iiiiiiiiiiiP11CUstream_st",
    "_ZN6cudeep7kernels36launch_conv2d_backward_weight_kernelIdEEvPKT_S4_PS2_iiiiiiiiiiiP11CUstream_st",
]


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(cudeep_b200_\w+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "cudeep_b200_matmul_f32" in names and "cudeep_b200_conv2d_forward_f32" in names
    assert len(names) >= 20


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in cudeep_b200.h but not exported"


def test_python_prototypes_cover_header(lib):
    from cudeep_b200 import _lib
    assert sorted(_lib.PROTOTYPES) == declared_functions()


def test_cxx_launcher_symbols_exported(lib):
    from cudeep_b200 import _lib
    out = subprocess.run(["nm", "-D", "--defined-only", str(_lib.LIB_PATH)], capture_output=True, text=True,
                         check=True).stdout
    exported = {line.split()[-1] for line in out.splitlines() if line.strip()}
    for sym in CXX_SYMBOLS:
        assert sym in exported, f"missing C++ launcher {sym}"


def test_version_and_error_string(lib):
    assert lib.cudeep_b200_version() >= 100
    assert isinstance(lib.cudeep_b200_last_error(), bytes)


def test_bad_arguments_fail_with_message_not_crash(lib):
    """Argument checks run before any CUDA call, so they work without a GPU."""
    rc = lib.cudeep_b200_matmul_f32(None, None, None, 4, 4, 4, None)
    assert rc != 0 and b"null" in lib.cudeep_b200_last_error()
    buf = (ctypes.c_float * 16)()
    p = ctypes.cast(buf, ctypes.c_void_p)
    rc = lib.cudeep_b200_matmul_f32(p, p, p, 0, 4, 4, None)
    assert rc != 0 and b"positive" in lib.cudeep_b200_last_error()
    rc = lib.cudeep_b200_matmul_fused_act(p, p, p, 4, 4, 4, 9, None)
    assert rc != 0 and b"epilogue" in lib.cudeep_b200_last_error()
    rc = lib.cudeep_b200_conv2d_forward_f32(p, p, None, p, 1, 1, 1, 2, 2, 3, 3, 1, 1, 0, 0, None)
    assert rc != 0 and b"kernel larger" in lib.cudeep_b200_last_error()
    rc = lib.cudeep_b200_conv2d_forward_f32(p, p, None, p, 1, 1, 1, 4, 4, 3, 3, 0, 1, 0, 0, None)
    assert rc != 0


def test_missing_library_is_a_loud_error(monkeypatch, tmp_path):
    from cudeep_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libcudeep_b200.so")
    with pytest.raises(RuntimeError, match="has not been built"):
        _lib.load()
