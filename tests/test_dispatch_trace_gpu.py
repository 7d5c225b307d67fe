"""CUDEEP_LOG=1: every launcher says on stderr which kernel a call took (the only way a caller can
see that a shape went to the strict-precision or the direct kernel instead of the tensor cores)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parents[1]

SCRIPT = r"""
import ctypes, numpy as np, torch
from cudeep_b200 import _lib
lib = _lib.load()
P = lambda t: ctypes.c_void_p(t.data_ptr())
def mm(m, n, k):
    a, b, c = (torch.zeros(s, device="cuda") for s in ((m, k), (k, n), (m, n)))
    _lib.check(lib.cudeep_b200_matmul_f32(P(a), P(b), P(c), m, n, k, None))
mm(8, 8, 8)
mm(512, 512, 512)
x, w, y = torch.zeros((2, 64, 16, 16), device="cuda"), torch.zeros((64, 64, 3, 3), device="cuda"), torch.zeros((2, 64, 16, 16), device="cuda")
_lib.check(lib.cudeep_b200_conv2d_forward_f32(P(x), P(w), None, P(y), 2, 64, 64, 16, 16, 3, 3, 1, 1, 1, 1, None))
x, w, y = torch.zeros((1, 4, 6, 6), device="cuda"), torch.zeros((5, 4, 3, 3), device="cuda"), torch.zeros((1, 5, 4, 4), device="cuda")
_lib.check(lib.cudeep_b200_conv2d_forward_f32(P(x), P(w), None, P(y), 1, 4, 5, 6, 6, 3, 3, 1, 1, 0, 0, None))
x, w, y = torch.zeros((1, 32, 28, 28), device="cuda"), torch.zeros((256, 32, 3, 3), device="cuda"), torch.zeros((1, 256, 28, 28), device="cuda")
_lib.check(lib.cudeep_b200_conv2d_forward_f32(P(x), P(w), None, P(y), 1, 32, 256, 28, 28, 3, 3, 1, 1, 1, 1, None))
torch.cuda.synchronize()
"""


def run(log):
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    env.pop("CUDEEP_LOG", None)
    if log:
        env["CUDEEP_LOG"] = "1"
    return subprocess.run([sys.executable, "-c", SCRIPT], env=env, capture_output=True, text=True, timeout=300)


def test_trace_names_the_kernel_each_call_took(lib, cuda):
    proc = run(True)
    assert proc.returncode == 0, proc.stderr
    lines = [l for l in proc.stderr.splitlines() if l.startswith("[cudeep_b200]")]
    assert any("gemm strict FP32" in l and "M=8 N=8 K=8" in l for l in lines)
    assert any("gemm tf32 tcgen05" in l and "M=512 N=512 K=512" in l and "tile=" in l and "stages=" in l for l in lines)
    assert any("conv2d implicit GEMM tcgen05" in l and "OC=64" in l for l in lines)
    assert any("conv2d direct strict FP32" in l and "OC=5" in l for l in lines)
    assert any("rows shared by the taps of a filter row" in l and "OC=256" in l and "4 rows x 30 pixels" in l for l in lines)


def test_trace_is_silent_by_default(lib, cuda):
    proc = run(False)
    assert proc.returncode == 0, proc.stderr
    assert "[cudeep_b200]" not in proc.stderr
