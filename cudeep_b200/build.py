"""Build libcudeep_b200.so from cudeep_b200/csrc with nvcc for sm_100a.

    python -m cudeep_b200.build            # incremental
    python -m cudeep_b200.build --force    # rebuild everything

Objects go to build/ (not tracked); the shared library is written next to this
file as cudeep_b200/libcudeep_b200.so.  nvcc cross-compiles, so no GPU is needed.
The pybind11 module _cudeep_core (csrc/bindings/module.cpp) is built against that
library into the same directory when pybind11 is importable.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
INCLUDE = ROOT / "include"
OBJ_DIR = ROOT / "build" / "obj"
LIB_PATH = PKG_DIR / "libcudeep_b200.so"

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    f"-I{INCLUDE}", f"-I{CSRC}",
]


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; libcudeep_b200.so cannot be built")
    return nvcc


def _newest_header_mtime() -> float:
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.rglob("*.h")) + \
        list(INCLUDE.rglob("*.cuh"))
    return max((h.stat().st_mtime for h in headers), default=0.0)


def _compile(nvcc: str, src: Path, obj: Path) -> tuple[Path, int, str]:
    cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    return src, proc.returncode, proc.stdout + proc.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_mtime = _newest_header_mtime()
    jobs = []
    objects = []
    for src in sources:
        obj = OBJ_DIR / (src.stem + ".o")
        objects.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_mtime)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
            for src, code, out in pool.map(lambda j: _compile(nvcc, *j), jobs):
                if verbose or code != 0:
                    sys.stderr.write(out)
                if code != 0:
                    raise RuntimeError(f"nvcc failed on {src.name}")
    relink = bool(jobs) or not LIB_PATH.exists() or \
        LIB_PATH.stat().st_mtime < max(o.stat().st_mtime for o in objects)
    if relink:
        cmd = [nvcc, "-shared", "-cudart", "static", "-o", str(LIB_PATH), *map(str, objects)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("linking libcudeep_b200.so failed")
    return LIB_PATH


def bindings_path() -> Path:
    import sysconfig
    return PKG_DIR / ("_cudeep_core" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_bindings(force: bool = False, verbose: bool = False) -> Path:
    """Compile the pybind11 module against libcudeep_b200.so (which must exist)."""
    import sysconfig
    import pybind11
    src = CSRC / "bindings" / "module.cpp"
    out = bindings_path()
    newest = max(src.stat().st_mtime, _newest_header_mtime(), LIB_PATH.stat().st_mtime)
    if not force and out.exists() and out.stat().st_mtime >= newest:
        return out
    cuda_include = Path(find_nvcc()).resolve().parent.parent / "include"
    cxx = "/usr/bin/g++" if Path("/usr/bin/g++").exists() else (shutil.which("g++") or "g++")
    cmd = [cxx, "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden",
           f"-I{INCLUDE}", f"-I{cuda_include}", f"-I{pybind11.get_include()}",
           f"-I{sysconfig.get_paths()['include']}", str(src), "-o", str(out),
           f"-L{PKG_DIR}", "-lcudeep_b200", "-Wl,-rpath,$ORIGIN"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError("building _cudeep_core failed")
    return out


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    print(build_bindings(force="--force" in sys.argv, verbose="-v" in sys.argv))
