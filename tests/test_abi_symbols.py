"""The C-ABI library loads on a CPU-only machine and exports every symbol include/crusader_b200.h declares."""
import ctypes
import os
import re

from crusaderbackend_b200 import _lib
from crusaderbackend_b200 import build as cb_build

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "crusader_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_symbols():
    syms = declared_symbols()
    assert "cb_create" in syms and "cb_gemm" in syms


def test_library_builds_and_exports_every_declared_symbol():
    cb_build.build()
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_python_binding_covers_the_header():
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_version_string():
    lib = _lib.load()
    assert b"sm_100a" in lib.cb_version()


def test_no_gpu_means_loud_failure():
    """Without a device cb_create must fail (no CPU fallback); with one it must succeed."""
    import torch
    lib = _lib.load()
    h = ctypes.c_void_p()
    rc = lib.cb_create(ctypes.byref(h), 0, None)
    if torch.cuda.is_available():
        assert rc == 0
        lib.cb_destroy(h)
    else:
        assert rc != 0 and not h.value


def test_trainer_header_symbols_are_exported_and_bound():
    from crusaderbackend_b200 import train
    text = open(os.path.join(ROOT, "include", "crusader_b200_train.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    declared = sorted(set(re.findall(r"\b(cbt_[a-z0-9_]+)\s*\(", text)))
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    assert not [s for s in declared if not hasattr(lib, s)]
    assert sorted(train.TRAIN_SIGNATURES) == declared


def test_compat_shim_compiles_against_the_library():
    """The header shim with the reference's seblas signatures builds into a program that links the C ABI."""
    import subprocess
    cb_build.build()
    out = os.path.join(ROOT, "tests", "cpp", "compat_smoke")
    cmd = ["nvcc", "-std=c++17", "-x", "cu", "-I", os.path.join(ROOT, "crusaderbackend_b200", "compat"), "-o", out,
           os.path.join(ROOT, "tests", "cpp", "compat_smoke.cpp"), "-L", os.path.join(ROOT, "crusaderbackend_b200", "lib"),
           "-lcrusader_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../crusaderbackend_b200/lib"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
