"""Runs the C++ program built on the seblas header shim (tests/cpp/compat_smoke.cpp) on the GPU."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def test_compat_smoke_program():
    exe = os.path.join(ROOT, "tests", "cpp", "compat_smoke")
    assert os.path.exists(exe), "tests/cpp/compat_smoke is built by the CPU test suite (test_abi_symbols.py)"
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "compat smoke ok" in r.stdout
