"""numpy face of the CPU oracle (oracle/cpu_ref.c) and the seeded input generators.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU legs (the
`cpu_baseline` object and `--impl reference`). Nothing under crusaderbackend_b200/ imports it; the seeded input
generators it re-exports live in crusaderbackend_b200/seeds.py.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "liboracle.so"
_lib = None

_fp = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_dp = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_ip = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_i = C.c_int
_ll = C.c_longlong


def build(force: bool = False) -> Path:
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < (_DIR / "cpu_ref.c").stat().st_mtime:
        r = subprocess.run(["make", "-C", str(_DIR), "-B", "liboracle.so"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("oracle build failed:\n" + r.stdout + r.stderr)
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(_LIB_PATH))
        _lib.orc_cross_entropy_f64.restype = C.c_double
        _lib.orc_num_threads.restype = _i
    return _lib


def num_threads() -> int:
    return int(lib().orc_num_threads())


def use_all_cores() -> int:
    """Sets the OpenMP team to every core this process may run on (launchers often export OMP_NUM_THREADS=1)."""
    import os
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads.argtypes = [_i]
    lib().orc_set_num_threads(n)
    return num_threads()


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _opt(a):
    return None if a is None else _f32(a).ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------------ seeded inputs
# The generators live in the package (the executor and the benchmark draw from them too); the tests reach them
# through this module so that oracle and library always see the same streams.
import sys as _sys

if str(_DIR.parent) not in _sys.path:
    _sys.path.insert(0, str(_DIR.parent))
from crusaderbackend_b200.seeds import he_normal_filter, normal, rng_for, uniform_pm1  # noqa: E402,F401


# ------------------------------------------------------------------ error metrics
def max_err_norm(got, ref) -> float:
    """max|got - ref| / max|ref| — the 'max relative error' the tolerances 1e-5 / 2e-3 are stated for."""
    ref = np.asarray(ref, dtype=np.float64)
    d = np.abs(np.asarray(got, dtype=np.float64) - ref).max() if ref.size else 0.0
    return float(d / max(np.abs(ref).max() if ref.size else 1.0, 1e-300))


# ------------------------------------------------------------------ GEMM
def gemm_f64(A, B, transA=False, transB=False) -> np.ndarray:
    A, B = _f32(A), _f32(B)
    M = A.shape[1] if transA else A.shape[0]
    K = A.shape[0] if transA else A.shape[1]
    N = B.shape[0] if transB else B.shape[1]
    out = np.empty((M, N), dtype=np.float64)
    f = lib().orc_gemm_f64
    f.argtypes = [_i, _i, _i, _i, _i, _fp, _i, _fp, _i, _dp, _i]
    f(int(transA), int(transB), M, N, K, A, A.shape[1], B, B.shape[1], out, N)
    return out


def gemm_f64_rows(A, B, rows, transA=False, transB=False) -> np.ndarray:
    A, B = _f32(A), _f32(B)
    M = A.shape[1] if transA else A.shape[0]
    K = A.shape[0] if transA else A.shape[1]
    N = B.shape[0] if transB else B.shape[1]
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    out = np.empty((len(rows), N), dtype=np.float64)
    f = lib().orc_gemm_f64_rows
    f.argtypes = [_i, _i, _i, _i, _i, _fp, _i, _fp, _i, _ip, _i, _dp]
    f(int(transA), int(transB), M, N, K, A, A.shape[1], B, B.shape[1], rows, len(rows), out)
    return out


def gemm_f64_cols(A, B, cols, transA=False, transB=False) -> np.ndarray:
    A, B = _f32(A), _f32(B)
    M = A.shape[1] if transA else A.shape[0]
    K = A.shape[0] if transA else A.shape[1]
    N = B.shape[0] if transB else B.shape[1]
    cols = np.ascontiguousarray(cols, dtype=np.int32)
    out = np.empty((M, len(cols)), dtype=np.float64)
    f = lib().orc_gemm_f64_cols
    f.argtypes = [_i, _i, _i, _i, _i, _fp, _i, _fp, _i, _ip, _i, _dp]
    f(int(transA), int(transB), M, N, K, A, A.shape[1], B, B.shape[1], cols, len(cols), out)
    return out


def gemm_f32(A, B, transA=False, transB=False, C_init=None) -> np.ndarray:
    A, B = _f32(A), _f32(B)
    M = A.shape[1] if transA else A.shape[0]
    K = A.shape[0] if transA else A.shape[1]
    N = B.shape[0] if transB else B.shape[1]
    out = np.zeros((M, N), dtype=np.float32) if C_init is None else _f32(C_init).copy()
    f = lib().orc_gemm_f32
    f.argtypes = [_i, _i, _i, _i, _i, _fp, _i, _fp, _i, _fp, _i, _i]
    f(int(transA), int(transB), M, N, K, A, A.shape[1], B, B.shape[1], out, N, int(C_init is not None))
    return out


# ------------------------------------------------------------------ convolution
def conv_out_hw(IH, IW, FH, FW, sH, sW, pH, pW):
    return (IH - FH + 2 * pH) // sH + 1, (IW - FW + 2 * pW) // sW + 1


_conv_args = [_i] * 11


def conv_fwd(W, X, bias=None, stride=(1, 1), pad=(0, 0), f32=False) -> np.ndarray:
    W, X = _f32(W), _f32(X)
    N, IC, IH, IW = X.shape
    OC, _, FH, FW = W.shape
    OH, OW = conv_out_hw(IH, IW, FH, FW, *stride, *pad)
    Y = np.empty((N, OC, OH, OW), dtype=np.float32 if f32 else np.float64)
    f = lib().orc_conv_fwd_f32 if f32 else lib().orc_conv_fwd_f64
    f.argtypes = [_fp, _fp, C.c_void_p, _fp if f32 else _dp] + _conv_args
    f(W, X, _opt(bias), Y, N, IC, IH, IW, OC, FH, FW, stride[0], stride[1], pad[0], pad[1])
    return Y


def conv_dgrad(W, dY, x_shape, stride=(1, 1), pad=(0, 0), f32=False) -> np.ndarray:
    W, dY = _f32(W), _f32(dY)
    N, IC, IH, IW = x_shape
    OC, _, FH, FW = W.shape
    dX = np.empty((N, IC, IH, IW), dtype=np.float32 if f32 else np.float64)
    f = lib().orc_conv_dgrad_f32 if f32 else lib().orc_conv_dgrad_f64
    f.argtypes = [_fp, _fp, _fp if f32 else _dp] + _conv_args
    f(W, dY, dX, N, IC, IH, IW, OC, FH, FW, stride[0], stride[1], pad[0], pad[1])
    return dX


def conv_wgrad(dY, X, w_shape, stride=(1, 1), pad=(0, 0), f32=False, dW_init=None, refmap=False) -> np.ndarray:
    dY, X = _f32(dY), _f32(X)
    N, IC, IH, IW = X.shape
    OC, _, FH, FW = w_shape
    dt = np.float32 if f32 else np.float64
    dW = np.zeros(w_shape, dtype=dt) if dW_init is None else np.ascontiguousarray(dW_init, dtype=dt).copy()
    if refmap:
        f = lib().orc_conv_wgrad_refmap_f64
        f.argtypes = [_fp, _fp, _dp] + _conv_args
        f(dY, X, dW, N, IC, IH, IW, OC, FH, FW, stride[0], stride[1], pad[0], pad[1])
        return dW
    f = lib().orc_conv_wgrad_f32 if f32 else lib().orc_conv_wgrad_f64
    f.argtypes = [_fp, _fp, _fp if f32 else _dp] + _conv_args + [_i]
    f(dY, X, dW, N, IC, IH, IW, OC, FH, FW, stride[0], stride[1], pad[0], pad[1], int(dW_init is not None))
    return dW


def conv_bias_grad(dY) -> np.ndarray:
    dY = _f32(dY)
    N, Cc, H, Wd = dY.shape
    db = np.empty(Cc, dtype=np.float64)
    f = lib().orc_conv_bias_grad_f64
    f.argtypes = [_fp, _dp, _i, _i, _i]
    f(dY, db, N, Cc, H * Wd)
    return db


# ------------------------------------------------------------------ linear
def linear(X, W, b=None) -> np.ndarray:
    X, W = _f32(X), _f32(W)
    batch, IN = X.shape
    OUT = W.shape[0]
    Y = np.empty((batch, OUT), dtype=np.float64)
    f = lib().orc_linear_f64
    f.argtypes = [_fp, _fp, C.c_void_p, _dp, _i, _i, _i]
    f(X, W, _opt(b), Y, batch, IN, OUT)
    return Y


def linear_xgrad(dY, W) -> np.ndarray:
    dY, W = _f32(dY), _f32(W)
    batch, OUT = dY.shape
    IN = W.shape[1]
    dX = np.empty((batch, IN), dtype=np.float64)
    f = lib().orc_linear_xgrad_f64
    f.argtypes = [_fp, _fp, _dp, _i, _i, _i]
    f(dY, W, dX, batch, IN, OUT)
    return dX


def linear_paramgrad(dY, X, dW_init=None, db_init=None):
    dY, X = _f32(dY), _f32(X)
    batch, OUT = dY.shape
    IN = X.shape[1]
    dW = np.zeros((OUT, IN)) if dW_init is None else np.asarray(dW_init, dtype=np.float64).copy()
    db = np.zeros(OUT) if db_init is None else np.asarray(db_init, dtype=np.float64).copy()
    f = lib().orc_linear_paramgrad_f64
    f.argtypes = [_fp, _fp, _dp, _dp, _i, _i, _i]
    f(dY, X, dW, db, batch, IN, OUT)
    return dW, db


# ------------------------------------------------------------------ batch norm (per (c,h,w) over the batch)
def bn_fwd(X, beta, gamma):
    X = _f32(X)
    N = X.shape[0]
    P = X.size // N
    Y = np.empty(X.shape)
    xhat = np.empty(X.shape)
    mean = np.empty(P)
    var = np.empty(P)
    f = lib().orc_bn_fwd_f64
    f.argtypes = [_fp, _fp, _fp, _dp, _dp, _dp, _dp, _i, _i]
    f(X, _f32(beta).ravel(), _f32(gamma).ravel(), mean, var, Y, xhat, N, P)
    return Y, xhat, mean, var


def bn_bwd(dY, gamma, X) -> np.ndarray:
    X = _f32(X)
    N = X.shape[0]
    P = X.size // N
    dX = np.empty(X.shape)
    f = lib().orc_bn_bwd_f64
    f.argtypes = [_fp, _fp, _fp, _dp, _i, _i]
    f(_f32(dY), _f32(gamma).ravel(), X, dX, N, P)
    return dX


def bn_paramgrad(dY, xhat):
    dY = _f32(dY)
    N = dY.shape[0]
    P = dY.size // N
    dg = np.empty(P)
    db = np.empty(P)
    f = lib().orc_bn_paramgrad_f64
    f.argtypes = [_fp, _fp, _dp, _dp, _i, _i]
    f(dY, _f32(xhat), dg, db, N, P)
    return dg, db


# ------------------------------------------------------------------ activations, pooling, loss, optimizer
def bn_fwd_f32(X, beta, gamma, res=None, relu=False) -> np.ndarray:
    """fp32 OpenMP BatchNorm forward (+ shortcut add, + ReLU) for the timed CPU baseline."""
    X = _f32(X)
    N, P = X.shape[0], X.size // X.shape[0]
    Y = np.empty_like(X)
    f = lib().orc_bn_fwd_f32
    f.argtypes = [_fp, _fp, _fp, C.c_void_p, _fp, _i, _ll, _i]
    f(X, _f32(beta).ravel(), _f32(gamma).ravel(), _opt(res), Y, N, P, int(relu))
    return Y


def bn_bwd_f32(dY, gamma, X):
    """fp32 OpenMP BatchNorm backward for the timed CPU baseline: (dX, dgamma, dbeta)."""
    X, dY = _f32(X), _f32(dY)
    N, P = X.shape[0], X.size // X.shape[0]
    dX = np.empty_like(X)
    dg, db = np.empty(P, dtype=np.float32), np.empty(P, dtype=np.float32)
    f = lib().orc_bn_bwd_f32
    f.argtypes = [_fp, _fp, _fp, _fp, _fp, _fp, _i, _ll]
    f(dY, _f32(gamma).ravel(), X, dX, dg, db, N, P)
    return dX, dg, db


def relu(X) -> np.ndarray:
    X = _f32(X)
    Y = np.empty(X.shape)
    f = lib().orc_relu_f64
    f.argtypes = [_fp, _dp, _ll]
    f(X, Y, X.size)
    return Y


def relu_grad(X, dY) -> np.ndarray:
    X = _f32(X)
    dX = np.empty(X.shape)
    f = lib().orc_relu_grad_f64
    f.argtypes = [_fp, _fp, _dp, _ll]
    f(X, _f32(dY), dX, X.size)
    return dX


def avgpool(X, r=(2, 2)) -> np.ndarray:
    X = _f32(X)
    N, Cc, H, Wd = X.shape
    Y = np.empty((N, Cc, H // r[0], Wd // r[1]))
    f = lib().orc_avgpool_f64
    f.argtypes = [_fp, _dp, _i, _i, _i, _i, _i]
    f(X, Y, N * Cc, H, Wd, r[0], r[1])
    return Y


def avgpool_back(dY, x_shape, r=(2, 2)) -> np.ndarray:
    dY = _f32(dY)
    N, Cc, H, Wd = x_shape
    dX = np.empty(x_shape)
    f = lib().orc_avgpool_back_f64
    f.argtypes = [_fp, _dp, _i, _i, _i, _i, _i]
    f(dY, dX, N * Cc, H, Wd, r[0], r[1])
    return dX


def gap(X) -> np.ndarray:
    X = _f32(X)
    N, Cc, H, Wd = X.shape
    Y = np.empty((N, Cc))
    f = lib().orc_gap_f64
    f.argtypes = [_fp, _dp, _i, _i]
    f(X, Y, N * Cc, H * Wd)
    return Y


def gap_back(dY, x_shape) -> np.ndarray:
    dY = _f32(dY)
    N, Cc, H, Wd = x_shape
    dX = np.empty(x_shape)
    f = lib().orc_gap_back_f64
    f.argtypes = [_fp, _dp, _i, _i]
    f(dY, dX, N * Cc, H * Wd)
    return dX


def softmax(X) -> np.ndarray:
    X = _f32(X)
    rows, step = X.shape[0], X.size // X.shape[0]
    Y = np.empty(X.shape)
    f = lib().orc_softmax_f64
    f.argtypes = [_fp, _dp, _i, _i]
    f(X, Y, rows, step)
    return Y


def cross_entropy(Y, labels):
    """Returns (loss summed over the batch, dY = Y - labels)."""
    Y = _f32(Y)
    dY = np.empty(Y.shape)
    f = lib().orc_cross_entropy_f64
    f.argtypes = [_fp, _fp, _dp, _ll]
    loss = f(Y, _f32(labels), dY, Y.size)
    return float(loss), dY


def momentum(w, g, m, lr, beta, l2, is_weight):
    """fp64 Momentum step; returns new (w, m, g)."""
    w = np.asarray(w, dtype=np.float64).copy()
    g = np.asarray(g, dtype=np.float64).copy()
    m = np.asarray(m, dtype=np.float64).copy()
    f = lib().orc_momentum_f64
    f.argtypes = [_dp, _dp, _dp, _ll, C.c_double, C.c_double, C.c_double, _i]
    f(w.ravel(), g.ravel(), m.ravel(), w.size, lr, beta, l2, int(is_weight))
    return w, m, g


def momentum_f32(w, g, m, lr, beta, l2, is_weight):
    w, g, m = _f32(w).copy(), _f32(g).copy(), _f32(m).copy()
    f = lib().orc_momentum_f32
    f.argtypes = [_fp, _fp, _fp, _ll, C.c_float, C.c_float, C.c_float, _i]
    f(w.ravel(), g.ravel(), m.ravel(), w.size, lr, beta, l2, int(is_weight))
    return w, m, g
