"""Builds and runs tests/cpp/test_cxx_surface.cu against libcudeep_b200.so: the C++ surface
(cudeep::Tensor, MemoryPool, Stream/Event, cudeep::kernels launchers) as a cuDeep C++ caller uses it.
The compile step alone runs without a GPU."""
import shutil
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
SRC = ROOT / "tests" / "cpp" / "test_cxx_surface.cu"
SHARDED_SRC = ROOT / "tests" / "cpp" / "test_sharded_gemm.cu"


def build(tmp_path, lib, src=SRC):
    from cudeep_b200 import _lib
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = tmp_path / src.stem
    cmd = [nvcc, "-std=c++17", "-O1", "-gencode", "arch=compute_100a,code=sm_100a", f"-I{ROOT / 'include'}",
           str(src), "-o", str(exe), f"-L{_lib.LIB_PATH.parent}", "-lcudeep_b200",
           "-Xlinker", f"-rpath={_lib.LIB_PATH.parent}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    return exe


def test_cxx_surface_compiles_and_links(tmp_path, lib):
    assert build(tmp_path, lib).exists()


@pytest.mark.gpu
def test_cxx_surface_runs(tmp_path, lib, cuda):
    exe = build(tmp_path, lib)
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "ALL PASSED" in proc.stdout, proc.stdout + proc.stderr


def test_sharded_gemm_cxx_plan_and_failure_path(tmp_path, lib):
    """cudeep::dist::ShardedGemm from C++ in its dry-run form: partition, bands, and the two-phase step
    that turns a failed rank into a PeerFailure before anything is enqueued (no GPU needed)."""
    exe = build(tmp_path, lib, SHARDED_SRC)
    proc = subprocess.run([str(exe), "--dry"], capture_output=True, text=True, timeout=120)
    assert proc.returncode == 0 and "ALL PASSED" in proc.stdout, proc.stdout + proc.stderr


@pytest.mark.gpu
def test_sharded_gemm_cxx_runs_on_every_gpu(tmp_path, lib, cuda):
    exe = build(tmp_path, lib, SHARDED_SRC)
    env = dict(__import__("os").environ, NCCL_NVLS_ENABLE="0")
    proc = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0 and "ALL PASSED" in proc.stdout, proc.stdout + proc.stderr
