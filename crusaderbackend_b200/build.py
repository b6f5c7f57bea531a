"""Builds libcrusader_b200.so (sm_100a only) in-tree with nvcc.

Usage: python -m crusaderbackend_b200.build [--force] [--verbose]
The shared library lands in crusaderbackend_b200/lib/. Objects are rebuilt when a source or header is newer.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
OBJ_DIR = PKG / "build"
LIB_PATH = LIB_DIR / "libcrusader_b200.so"

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-cudart", "shared",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA kernels cannot be built")
    return exe


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + sorted((PKG.parent / "include").glob("*.h"))


def needs_build() -> bool:
    if not LIB_PATH.exists():
        return True
    t = LIB_PATH.stat().st_mtime
    return any(p.stat().st_mtime > t for p in _sources() + _headers())


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, trace: bool = False) -> Path:
    """trace=True builds a second library, libcrusader_b200_trace.so, with the kernels' time-stamp instrumentation
    (-DCB_TRACE) compiled in; the product library never carries it."""
    lib_path = LIB_DIR / "libcrusader_b200_trace.so" if trace else LIB_PATH
    if not force and not trace and not needs_build():
        return LIB_PATH
    nvcc = _nvcc()
    LIB_DIR.mkdir(exist_ok=True)
    obj_dir = OBJ_DIR / "trace" if trace else OBJ_DIR
    obj_dir.mkdir(parents=True, exist_ok=True)
    hdr_time = max(p.stat().st_mtime for p in _headers())
    flags = list(NVCC_FLAGS)
    if ptxas_info:
        flags += ["-Xptxas", "-v"]
    if trace:
        flags += ["-DCB_TRACE"]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, hdr_time):
            return obj
        cmd = [nvcc, *flags, "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if (verbose or ptxas_info) and (r.stdout or r.stderr):
            print(r.stdout + r.stderr, flush=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, _sources()))
    cmd = [nvcc, "-shared", "-cudart", "shared", "-o", str(lib_path), *map(str, objs),
           "-Xlinker", "-rpath", "-Xlinker", "/usr/local/cuda/lib64"]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, ptxas_info="--ptxas" in sys.argv,
                 trace="--trace" in sys.argv)
    print(path)
