"""Build the sm_100a kernel library in-tree with nvcc.

Every ``csrc/*.cu`` file is compiled to an object file and the objects are linked into one shared
library, ``halo_b200/lib/libhalo_b200.so``, which :mod:`halo_b200.ops._lib` loads with ctypes. The
library exposes plain ``extern "C"`` entry points that take device pointers and a stream, so no
torch headers are needed and a full rebuild takes seconds. nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC_DIR = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libhalo_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-cudart",
    "shared",
    "-Xcompiler",
    "-fPIC",
]


# Per-file additions: the optimizer's arithmetic is specified without fused multiply-adds so its CPU
# twin can reproduce it bit for bit.
EXTRA_FLAGS = {"optim.cu": ["-fmad=false"], "collectives_sm100.cu": ["-fmad=false"]}


def find_nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the sm_100a kernel library cannot be built")
    return nvcc


def _newest_header_mtime() -> float:
    return max((p.stat().st_mtime for p in list(CSRC_DIR.glob("*.cuh")) + list(CSRC_DIR.glob("*.h"))), default=0.0)


def _compile_one(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, *EXTRA_FLAGS.get(src.name, []), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")
    return proc.stderr


HOST_LIB_PATH = LIB_DIR / "libhalo_host.so"
# no fused multiply-add (the host optimizer reproduces the device kernel bit for bit); AVX2 is the widest vector
# set every B200 host CPU has
HOST_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-mavx2", "-ffp-contract=off", "-fno-math-errno"]


def build_host(force: bool = False) -> Path:
    """The CPU-side library (host optimizer): plain g++ with OpenMP, no CUDA."""
    LIB_DIR.mkdir(exist_ok=True)
    sources = sorted(CSRC_DIR.glob("*.cpp"))
    newest = max((s.stat().st_mtime for s in sources), default=0.0)
    if sources and (force or not HOST_LIB_PATH.exists() or HOST_LIB_PATH.stat().st_mtime < newest):
        gxx = shutil.which("g++") or "g++"
        proc = subprocess.run([gxx, *HOST_FLAGS, *map(str, sources), "-o", str(HOST_LIB_PATH)], capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"g++ failed on the host library:\n{proc.stdout}\n{proc.stderr}")
    return HOST_LIB_PATH


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what changed and link the library; returns its path."""
    build_host(force)
    nvcc = find_nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = LIB_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    sources = sorted(CSRC_DIR.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC_DIR}")
    header_mtime = _newest_header_mtime()
    jobs = []
    for src in sources:
        obj = obj_dir / (src.stem + ".o")
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_mtime)
        if stale:
            jobs.append((src, obj))
    logs = []
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            futs = [pool.submit(_compile_one, nvcc, s, o, verbose) for s, o in jobs]
            for f in futs:
                logs.append(f.result())
    objs = [obj_dir / (s.stem + ".o") for s in sources]
    relink = bool(jobs) or not LIB_PATH.exists()
    if relink:
        cmd = [nvcc, "-shared", "-cudart", "shared", "-o", str(LIB_PATH), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write("\n".join(logs))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
