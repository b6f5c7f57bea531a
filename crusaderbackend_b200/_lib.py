"""ctypes binding of libcrusader_b200.so (the C ABI declared in include/crusader_b200.h).

There is no fallback: if the shared library is missing or does not load, importing a compute entry
point raises. Build it with `python -m crusaderbackend_b200.build`.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
# CRUSADER_B200_LIB: load another build of the same library (e.g. the instrumented one of `build --trace`)
LIB_PATH = Path(os.environ.get("CRUSADER_B200_LIB") or _PKG / "lib" / "libcrusader_b200.so")

CB_OK, CB_EINVAL, CB_ECUDA, CB_ETIMEOUT, CB_EUNSUPPORTED, CB_ENOMEM = 0, -1, -2, -3, -4, -5
CB_MATH_TF32, CB_MATH_3XTF32, CB_MATH_FP32 = 0, 1, 2

_f = C.c_void_p  # device pointers travel as integers
_i = C.c_int
_ll = C.c_longlong
_fl = C.c_float
_ctx = C.c_void_p

# name -> (restype, argtypes); must list every symbol include/crusader_b200.h declares
SIGNATURES = {
    "cb_version": (C.c_char_p, []),
    "cb_create": (_i, [C.POINTER(_ctx), _i, C.c_void_p]),
    "cb_destroy": (_i, [_ctx]),
    "cb_set_stream": (_i, [_ctx, C.c_void_p]),
    "cb_set_math": (_i, [_ctx, _i]),
    "cb_get_math": (_i, [_ctx]),
    "cb_set_sync": (_i, [_ctx, _i]),
    "cb_set_deterministic": (_i, [_ctx, _i]),
    "cb_freeze_workspace": (_i, [_ctx, _i]),
    "cb_synchronize": (_i, [_ctx]),
    "cb_last_error": (C.c_char_p, [_ctx]),
    "cb_launch_count": (_ll, [_ctx]),
    "cb_last_kernel": (C.c_char_p, [_ctx]),
    "cb_gemm": (_i, [_ctx, _i, _i, _i, _i, _i, _f, _i, _f, _i, _f, _i, _i, _ll, _ll, _ll, _i]),
    "cb_gemm_batch_reduce": (_i, [_ctx, _i, _i, _i, _i, _i, _f, _i, _f, _i, _f, _i, _i, _ll, _ll, _i]),
    "cb_measure_umma_peak": (_i, [_ctx, _i, _i, _i, _i, C.POINTER(_fl)]),
    "cb_conv_fwd": (_i, [_ctx, _f, _f, _f, _f] + [_i] * 12),
    "cb_conv_dgrad": (_i, [_ctx, _f, _f, _f] + [_i] * 11),
    "cb_conv_wgrad": (_i, [_ctx, _f, _f, _f] + [_i] * 12),
    "cb_conv_fwd_ex": (_i, [_ctx, _f, _f, _f] + [_i] * 11 + [C.c_void_p]),
    "cb_conv_dgrad_ex": (_i, [_ctx, _f, _f, _f] + [_i] * 12 + [_ll, _ll]),
    "cb_conv_wgrad_ex": (_i, [_ctx, _f, _f, _f] + [_i] * 12 + [_ll, _ll]),
    "cb_conv_cache_filters": (_i, [_ctx, _i]),
    "cb_filters_changed": (_i, [_ctx]),
    "cb_conv_bias": (_i, [_ctx, _f, _f, _i, _i, _i]),
    "cb_conv_bias_grad": (_i, [_ctx, _f, _f, _i, _i, _i, _i]),
    "cb_linear_fwd": (_i, [_ctx, _f, _f, _f, _f, _i, _i, _i]),
    "cb_linear_xgrad": (_i, [_ctx, _f, _f, _f, _i, _i, _i]),
    "cb_linear_paramgrad": (_i, [_ctx, _f, _f, _f, _f, _i, _i, _i]),
    "cb_bn_fwd": (_i, [_ctx, _f, _f, _f, _f, _f, _f, _f, _i, _ll]),
    "cb_bn_bwd": (_i, [_ctx, _f, _f, _f, _f, _i, _ll]),
    "cb_bn_paramgrad": (_i, [_ctx, _f, _f, _f, _f, _i, _ll]),
    "cb_bn_bwd_fused": (_i, [_ctx, _f, _f, _f, _f, _f, _f, _f, _i, _ll]),
    "cb_bn_fwd_relu": (_i, [_ctx, _f, _f, _f, _f, _i, _ll]),
    "cb_bn_fwd_relu_ex": (_i, [_ctx, _f, _f, _f, _f, _i, _ll, _ll]),
    "cb_bn_bwd_fused_ex": (_i, [_ctx, _f, _f, _f, _f, _f, _f, _f, _i, _ll, _ll, _ll, _i]),
    "cb_avgpool_ex": (_i, [_ctx, _f, _f, _i, _i, _i, _i, _i, _i, _ll]),
    "cb_avgpool_back_ex": (_i, [_ctx, _f, _f, _i, _i, _i, _i, _i, _i, _ll]),
    "cb_bn_fwd_add_relu": (_i, [_ctx, _f, _f, _f, _f, _f, _i, _ll]),
    "cb_bn_bwd_fused_res": (_i, [_ctx, _f, _f, _f, _f, _f, _f, _f, _f, _i, _i, _ll]),
    "cb_add_relu": (_i, [_ctx, _f, _f, _f, _ll]),
    "cb_relu_grad2": (_i, [_ctx, _f, _f, _f, _f, _ll]),
    "cb_relu": (_i, [_ctx, _f, _f, _ll]),
    "cb_relu_grad": (_i, [_ctx, _f, _f, _f, _ll]),
    "cb_tensor_op": (_i, [_ctx, _i, _f, _f, _fl, _ll]),
    "cb_grad_handover": (_i, [_ctx, _f, _f, _ll]),
    "cb_concat_channels": (_i, [_ctx, _i, C.POINTER(C.c_void_p), C.POINTER(_i), _f, _i, _i]),
    "cb_concat_grads": (_i, [_ctx, _i, C.POINTER(C.c_void_p), C.POINTER(_i), _f, _i, _i]),
    "cb_avgpool": (_i, [_ctx, _f, _f, _ll, _i, _i, _i, _i]),
    "cb_avgpool_back": (_i, [_ctx, _f, _f, _ll, _i, _i, _i, _i]),
    "cb_global_avgpool": (_i, [_ctx, _f, _f, _ll, _i]),
    "cb_global_avgpool_back": (_i, [_ctx, _f, _f, _ll, _i]),
    "cb_softmax": (_i, [_ctx, _f, _f, _i, _i]),
    "cb_cross_entropy": (_i, [_ctx, _f, _f, _f, _f, _ll]),
    "cb_head_fwd": (_i, [_ctx] + [_f] * 9 + [_i] * 4),
    "cb_head_bwd": (_i, [_ctx] + [_f] * 8 + [_i] * 4),
    "cb_momentum": (_i, [_ctx, _f, _f, _f, _ll, _fl, _fl, _fl, _i]),
    "cb_conv_fwd_noalloc": (_i, [_i, C.c_void_p, _f, _f, _f, _f] + [_i] * 12 + [C.c_char_p, _i]),
    "cb_conv_fwd_noalloc_status": (_i, [_i, C.c_void_p, C.c_char_p, _i]),
    "cb_crseq_inspect": (_i, [C.c_char_p, C.POINTER(C.c_uint), C.POINTER(C.c_uint), C.POINTER(C.c_ulonglong), C.c_char_p, _i]),
    "cb_crseq_read_params": (_i, [C.c_char_p, C.c_void_p, C.c_ulonglong, C.c_char_p, _i]),
    "cb_selftest_wait_timeout": (_i, [_ctx, _i]),
    "cb_momentum_multi": (_i, [_ctx, _i, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                               C.POINTER(_ll), C.POINTER(C.c_ubyte), _fl, _fl, _fl]),
}

CB_OP_ADD, CB_OP_SUB, CB_OP_MUL, CB_OP_DIV = 0, 1, 2, 3
CB_OP_ADD_SCALAR, CB_OP_SUB_SCALAR, CB_OP_MUL_SCALAR, CB_OP_DIV_SCALAR, CB_OP_FILL = 4, 5, 6, 7, 8

_lib = None


def load() -> C.CDLL:
    """Loads the shared library (once) and attaches the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built "
            "(python -m crusaderbackend_b200.build). There is no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


class CrusaderError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"crusader_b200 error {code}: {msg}")
        self.code = code
