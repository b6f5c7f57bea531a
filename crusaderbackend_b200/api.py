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

    def measure_umma_peak(self, n: int = 256, p_mn: bool = False, q_mn: bool = False, iters: int = 20000) -> float:
        """TFLOP/s of a resident-operand tcgen05.mma loop (M=128, N=n, K=8, TF32) on every SM."""
        out = C.c_float()
        self._check(self.lib.cb_measure_umma_peak(self.h, n, int(p_mn), int(q_mn), iters, C.byref(out)))
        return float(out.value)

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

    def sgemmNTA(self, A, B, Cout):
        """seblas::sgemmNTA: C += sum over n of A[n] @ B[n]^T, A n x M x K, B n x N x K, C M x N
        (seblas/operations/cuGEMM.cu:1701); the batch is folded into the contraction, one launch."""
        if A.dim() != 3 or B.dim() != 3 or Cout.dim() != 2:
            raise ValueError("sgemmNTA: A and B are 3-D (batch first), C is 2-D")
        for t in (A, B, Cout):
            if t.stride(-1) != 1:
                raise ValueError("operands must be row-major (unit inner stride)")
        n, M, K = A.shape
        if B.shape[0] != n or B.shape[2] != K or tuple(Cout.shape) != (M, B.shape[1]):
            raise ValueError("sgemmNTA: shapes do not agree")
        self._check(self.lib.cb_gemm_batch_reduce(self.h, 0, 1, M, B.shape[1], K, _ptr(A), A.stride(1), _ptr(B), B.stride(1),
                                                  _ptr(Cout), Cout.stride(0), n, A.stride(0), B.stride(0), 1))
        return Cout

    # ---- convolution: arguments in the order of seblas::conv / convDerive / convError
    @staticmethod
    def _geo(W, X, stride, pad):
        N, IC, IH, IW = X.shape
        OC, IC2, FH, FW = W.shape
        if IC2 != IC:
            raise ValueError("conv: channel counts do not agree")
        return [N, IC, IH, IW, OC, FH, FW, stride[0], stride[1], pad[0], pad[1]]

    def conv(self, A, B, Cout, strideH=1, strideW=1, padH=0, padW=0, biases=None, relu=False):
        """seblas::conv(A=filters OC x IC x FH x FW, B=input N x IC x IH x IW, C=output), seblas/operations/cuConv.cu:757."""
        geo = self._geo(A, B, (strideH, strideW), (padH, padW))
        self._check(self.lib.cb_conv_fwd(self.h, _ptr(A), _ptr(B), _ptr(Cout), _ptr(biases), *geo, int(relu)))
        return Cout

    def convDerive(self, A, B, Cout, strideH=1, strideW=1, padH=0, padW=0):
        """seblas::convDerive(A=filters, B=dY, C=dX), seblas/operations/cuConv.cu:774."""
        geo = self._geo(A, Cout, (strideH, strideW), (padH, padW))
        self._check(self.lib.cb_conv_dgrad(self.h, _ptr(A), _ptr(B), _ptr(Cout), *geo))
        return Cout

    def convError(self, A, B, Cout, strideH=1, strideW=1, padH=0, padW=0, accumulate=True):
        """seblas::convError(A=dY, B=input, C=filter gradient, accumulated), seblas/operations/cuConv.cu:793.
        Returns A, as the reference does."""
        geo = self._geo(Cout, B, (strideH, strideW), (padH, padW))
        self._check(self.lib.cb_conv_wgrad(self.h, _ptr(A), _ptr(B), _ptr(Cout), *geo, int(accumulate)))
        return A

    def convBias(self, Y, biases):
        N, Cc, H, W = Y.shape
        self._check(self.lib.cb_conv_bias(self.h, _ptr(Y), _ptr(biases), N, Cc, H * W))
        return Y

    def convBiasGrad(self, dY, db, accumulate=False):
        N, Cc, H, W = dY.shape
        self._check(self.lib.cb_conv_bias_grad(self.h, _ptr(dY), _ptr(db), N, Cc, H * W, int(accumulate)))
        return db

    # ---- linear: seblas::linear / linearXGrad / linearParamGrad (seblas/operations/cuLinear.cu:1052-1115)
    def linear(self, X, W, B, Y):
        batch, IN = X.shape[0], X.numel() // X.shape[0]
        self._check(self.lib.cb_linear_fwd(self.h, _ptr(X), _ptr(W), _ptr(B), _ptr(Y), batch, IN, W.shape[-2]))
        return Y

    def linearXGrad(self, dY, W, dX):
        batch = dX.shape[0]
        self._check(self.lib.cb_linear_xgrad(self.h, _ptr(dY), _ptr(W), _ptr(dX), batch, W.shape[-1], W.shape[-2]))
        return dX

    def linearParamGrad(self, dY, X, dW, dB):
        batch = X.shape[0]
        self._check(self.lib.cb_linear_paramgrad(self.h, _ptr(dY), _ptr(X), _ptr(dW), _ptr(dB), batch, dW.shape[-1],
                                                 dW.shape[-2]))
        return dW

    # ---- neighbours
    def batchNorm(self, X, beta, gamma, mean, var, Y, xHat):
        N = X.shape[0]
        self._check(self.lib.cb_bn_fwd(self.h, _ptr(X), _ptr(beta), _ptr(gamma), _ptr(mean), _ptr(var), _ptr(Y),
                                       _ptr(xHat), N, X.numel() // N))
        return Y

    def batchNormGrad(self, dY, gamma, X, dX):
        N = X.shape[0]
        self._check(self.lib.cb_bn_bwd(self.h, _ptr(dY), _ptr(gamma), _ptr(X), _ptr(dX), N, X.numel() // N))
        return dX

    def batchNormParamGrads(self, dY, xHat, dGamma, dBeta):
        N = dY.shape[0]
        self._check(self.lib.cb_bn_paramgrad(self.h, _ptr(dY), _ptr(xHat), _ptr(dGamma), _ptr(dBeta), N,
                                             dY.numel() // N))

    def batchNormGradFused(self, dY, gamma, X, dX, dGamma, dBeta, relu_out=None):
        N = X.shape[0]
        self._check(self.lib.cb_bn_bwd_fused(self.h, _ptr(dY), _ptr(gamma), _ptr(X), _ptr(dX), _ptr(dGamma), _ptr(dBeta),
                                             _ptr(relu_out), N, X.numel() // N))
        return dX

    def batchNormRelu(self, X, beta, gamma, Y):
        N = X.shape[0]
        self._check(self.lib.cb_bn_fwd_relu(self.h, _ptr(X), _ptr(beta), _ptr(gamma), _ptr(Y), N, X.numel() // N))
        return Y

    def addRelu(self, A, B, Out):
        self._check(self.lib.cb_add_relu(self.h, _ptr(A), _ptr(B), _ptr(Out), A.numel()))
        return Out

    def reluGrad2(self, Y, dY, dA, dB=None):
        self._check(self.lib.cb_relu_grad2(self.h, _ptr(Y), _ptr(dY), _ptr(dA), _ptr(dB), Y.numel()))
        return dA

    def relu(self, X, Y):
        self._check(self.lib.cb_relu(self.h, _ptr(X), _ptr(Y), X.numel()))
        return Y

    def reluGradFast(self, X, dY, dX):
        self._check(self.lib.cb_relu_grad(self.h, _ptr(X), _ptr(dY), _ptr(dX), X.numel()))
        return dX

    def tensor_op(self, op: int, A, B=None, scalar: float = 0.0):
        self._check(self.lib.cb_tensor_op(self.h, op, _ptr(A), _ptr(B), scalar, A.numel()))
        return A

    def grad_handover(self, dA, dAReserve):
        self._check(self.lib.cb_grad_handover(self.h, _ptr(dA), _ptr(dAReserve), dA.numel()))
        return dA

    def avgPool(self, X, Y, rangeH=2, rangeW=2):
        N, Cc, H, W = X.shape
        self._check(self.lib.cb_avgpool(self.h, _ptr(X), _ptr(Y), N * Cc, H, W, rangeH, rangeW))
        return Y

    def avgPoolBack(self, dX, dY, rangeH=2, rangeW=2):
        N, Cc, H, W = dX.shape
        self._check(self.lib.cb_avgpool_back(self.h, _ptr(dX), _ptr(dY), N * Cc, H, W, rangeH, rangeW))
        return dX

    def globalAvgPool(self, X, Y):
        N, Cc, H, W = X.shape
        self._check(self.lib.cb_global_avgpool(self.h, _ptr(X), _ptr(Y), N * Cc, H * W))
        return Y

    def globalAvgPoolBack(self, dX, dY):
        N, Cc, H, W = dX.shape
        self._check(self.lib.cb_global_avgpool_back(self.h, _ptr(dX), _ptr(dY), N * Cc, H * W))
        return dX

    def softmax(self, A, out, step=None):
        rows = A.shape[0]
        step = step or A.numel() // rows
        self._check(self.lib.cb_softmax(self.h, _ptr(A), _ptr(out), A.numel() // step, step))
        return out

    def crossEntropy(self, Y, labels, dY=None, loss=None):
        self._check(self.lib.cb_cross_entropy(self.h, _ptr(Y), _ptr(labels), _ptr(dY), _ptr(loss), Y.numel()))
        return loss

    def momentumApply(self, X, Xgrad, V, lr, beta, l2=0.0, is_weight=False):
        self._check(self.lib.cb_momentum(self.h, _ptr(X), _ptr(Xgrad), _ptr(V), X.numel(), lr, beta, l2,
                                         int(is_weight)))

    def momentumApplyMulti(self, params, grads, moms, is_weight, lr, beta, l2):
        n = len(params)
        arr = lambda ts: (C.c_void_p * n)(*[t.data_ptr() for t in ts])
        sizes = (C.c_longlong * n)(*[t.numel() for t in params])
        flags = (C.c_ubyte * n)(*[1 if f else 0 for f in is_weight])
        self._check(self.lib.cb_momentum_multi(self.h, n, arr(params), arr(grads), arr(moms), sizes, flags, lr, beta, l2))
