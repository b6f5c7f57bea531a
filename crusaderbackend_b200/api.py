"""Thin Python face of the C ABI for tests and benchmarks.

torch is used only to own device memory and streams; every computation goes through
libcrusader_b200.so. Function names follow the reference's seblas operations
(seblas/operations/cuGEMM.cuh:12-21, cuConv.cuh:20-42, cuLinear.cuh:14-18).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import CB_MATH_3XTF32, CB_MATH_FP32, CB_MATH_TF32, CrusaderError

MATH_MODES = {"tf32": CB_MATH_TF32, "3xtf32": CB_MATH_3XTF32, "fp32": CB_MATH_FP32}


def _ptr(t: torch.Tensor | None) -> int | None:
    if t is None:
        return None
    if not t.is_cuda or t.dtype != torch.float32:
        raise ValueError("operands must be fp32 CUDA tensors")
    return t.data_ptr()


class Context:
    """One cb_ctx on one GPU. `stream=None` binds torch's current stream on that device."""

    def __init__(self, device: int = 0, math: str = "tf32", sync: bool = False, stream: torch.cuda.Stream | None = None):
        self.lib = _lib.load()
        if not torch.cuda.is_available():
            raise RuntimeError("crusader_b200 needs a CUDA device; there is no CPU path")
        self.device = device
        torch.cuda.set_device(device)
        st = stream if stream is not None else torch.cuda.current_stream(device)
        self._stream = st
        h = C.c_void_p()
        rc = self.lib.cb_create(C.byref(h), device, C.c_void_p(st.cuda_stream))
        if rc != 0:
            raise CrusaderError(rc, "cb_create failed")
        self.h = h
        self.set_math(math)
        self.set_sync(sync)

    # ---- plumbing
    def _check(self, rc: int) -> None:
        if rc != 0:
            raise CrusaderError(rc, self.lib.cb_last_error(self.h).decode())

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.cb_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_math(self, math: str) -> None:
        self._check(self.lib.cb_set_math(self.h, MATH_MODES[math]))
        self.math = math

    def set_sync(self, on: bool) -> None:
        self._check(self.lib.cb_set_sync(self.h, int(on)))

    def set_deterministic(self, on: bool) -> None:
        self._check(self.lib.cb_set_deterministic(self.h, int(on)))

    def synchronize(self) -> None:
        self._check(self.lib.cb_synchronize(self.h))

    @property
    def launches(self) -> int:
        return int(self.lib.cb_launch_count(self.h))

    @property
    def last_kernel(self) -> str:
        return self.lib.cb_last_kernel(self.h).decode()

    # ---- GEMM (raw)
    def gemm(self, A: torch.Tensor, B: torch.Tensor, C_: torch.Tensor, transA: bool = False, transB: bool = False,
             accumulate: bool = False) -> torch.Tensor:
        """C = op(A) @ op(B) (+ C). 2-D row-major operands, or 3-D with a leading batch dimension
        (a 2-D A or B is shared by every batch, as in seblas::sgemm)."""
        def mat(t):
            if t.dim() == 2:
                return 1, t.shape[0], t.shape[1], t.stride(0), 0
            return t.shape[0], t.shape[1], t.shape[2], t.stride(1), t.stride(0)
        for t in (A, B, C_):
            if t.stride(-1) != 1:
                raise ValueError("operands must be row-major (unit inner stride)")
        ba, ra, ca, lda, sa = mat(A)
        bb, rb, cb, ldb, sb = mat(B)
        bc, M, N, ldc, sc = mat(C_)
        K = ra if transA else ca
        if (ca if transA else ra) != M or (cb if transB else rb) != K or (rb if transB else cb) != N:
            raise ValueError("gemm: shapes do not agree")
        batch = bc
        if ba not in (1, batch) or bb not in (1, batch):
            raise ValueError("gemm: batch sizes do not agree")
        self._check(self.lib.cb_gemm(self.h, int(transA), int(transB), M, N, K, _ptr(A), lda, _ptr(B), ldb,
                                     _ptr(C_), ldc, batch, sa if ba == batch else 0, sb if bb == batch else 0, sc,
                                     int(accumulate)))
        return C_

    # ---- seblas-named GEMMs
    def sgemm(self, A, B, Cout):
        """seblas::sgemm: C[b] = A @ B[b] (seblas/operations/cuGEMM.cu:1649)."""
        return self.gemm(A, B, Cout)

    def sgemmTN(self, A, B, Cout):
        """seblas::sgemmTN: C[b] = A^T @ B[b], A stored K x M (seblas/operations/cuGEMM.cu:1667)."""
        return self.gemm(A, B, Cout, transA=True)

    def sgemmNT(self, A, B, Cout):
        """seblas::sgemmNT: C = A @ B^T, B stored N x K (seblas/operations/cuGEMM.cu:1685)."""
        return self.gemm(A, B, Cout, transB=True)
