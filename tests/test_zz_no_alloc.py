"""cb_conv_fwd_noalloc — the forward convolution for callers that cannot allocate device memory (a memory manager
owns the whole GPU, a latency-critical loop cannot take cudaMalloc's device synchronisation, or a stream is being
captured). Called through the C ABI and compared with the ordinary cb_conv_fwd on the same inputs, twice in a
row with different shapes so that stale contents of the shared static scratch would show. Collected last."""
import ctypes

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TOL_TF32 = 2e-3  # the tolerance the TF32 convolution tests use, on max|a - b| / max|b|


def _run_pair(torch, lib, ctx, key, N, IC, H, OC, F, bias, relu):
    p = 1 if F == 3 else 0
    W = torch.from_numpy(orc.he_normal_filter(OC, IC, F, F, key)).cuda()
    X = torch.from_numpy(orc.normal((N, IC, H, H), key, "X")).cuda()
    b = torch.from_numpy(orc.normal((OC,), key, "b")).cuda() if bias else None
    want = torch.full((N, OC, H, H), float("nan"), device="cuda")
    ctx.conv(W, X, want, 1, 1, p, p, b, relu=relu)
    assert ctx.last_kernel == "umma_tf32"
    got = torch.full((N, OC, H, H), float("nan"), device="cuda")
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.cb_conv_fwd_noalloc(0, ctypes.c_void_p(stream), W.data_ptr(), X.data_ptr(), got.data_ptr(),
                                 None if b is None else b.data_ptr(), N, IC, H, H, OC, F, F, 1, 1, p, p, int(relu),
                                 err, 256)
    assert rc == 0, err.value.decode()
    torch.cuda.synchronize()
    assert torch.isfinite(got).all()
    assert orc.max_err_norm(got.cpu().numpy(), want.cpu().numpy()) <= TOL_TF32
    # and both agree with the fp64 oracle
    ref = orc.conv_fwd(W.cpu().numpy(), X.cpu().numpy(), None if b is None else b.cpu().numpy(), (1, 1), (p, p))
    if relu:
        ref = np.maximum(ref, 0)
    assert orc.max_err_norm(got.cpu().numpy(), ref) <= TOL_TF32


def test_noalloc_forward_matches_regular_entry_point_twice():
    import torch
    from crusaderbackend_b200 import _lib
    from crusaderbackend_b200.api import Context
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    lib = _lib.load()
    ctx = Context(0, math="tf32", sync=True)
    # first call: the largest filter the static scratch is sized for; second call: a smaller, different layer
    _run_pair(torch, lib, ctx, "na1", 8, 64, 32, 64, 3, bias=False, relu=False)
    _run_pair(torch, lib, ctx, "na2", 4, 16, 16, 12, 3, bias=True, relu=True)
    _run_pair(torch, lib, ctx, "na3", 4, 40, 8, 48, 1, bias=True, relu=False)
    # no bounded device-side wait expired in any of the three calls
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.cb_conv_fwd_noalloc_status(0, ctypes.c_void_p(stream), err, 256) == 0, err.value.decode()
    ctx.close()


def test_noalloc_leaves_device_memory_and_current_device_alone():
    """The property the entry point exists for: a call (after the first one on the device, which only resolves symbol
    addresses) takes no device memory — the driver reports the same free byte count before and after — and the
    caller's current device is what it was."""
    import torch
    from crusaderbackend_b200 import _lib
    lib = _lib.load()
    W = torch.from_numpy(orc.he_normal_filter(32, 32, 3, 3, "na_mem")).cuda()
    X = torch.from_numpy(orc.normal((8, 32, 16, 16), "na_mem", "X")).cuda()
    Y = torch.empty(8, 32, 16, 16, device="cuda")
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        rc = lib.cb_conv_fwd_noalloc(0, ctypes.c_void_p(stream), W.data_ptr(), X.data_ptr(), Y.data_ptr(), None, 8, 32, 16,
                                     16, 32, 3, 3, 1, 1, 1, 1, 0, err, 256)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()

    call()  # first call on this device: set-up
    before = torch.cuda.current_device()
    free0, _ = torch.cuda.mem_get_info()   # cudaMemGetInfo: the driver's count, not torch's allocator's
    for _ in range(3):
        call()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
    assert torch.cuda.current_device() == before


def test_noalloc_rejects_what_does_not_fit():
    import torch
    from crusaderbackend_b200 import _lib
    from crusaderbackend_b200._lib import CB_EINVAL, CB_EUNSUPPORTED
    lib = _lib.load()
    buf = torch.zeros(1024, device="cuda")
    err = ctypes.create_string_buffer(256)
    p = buf.data_ptr()
    # 128 -> 64 channels, 3x3: packed filter 3 * 4 * 192 * 128 = 294 912 bytes > 163 840
    rc = lib.cb_conv_fwd_noalloc(0, None, p, p, p, None, 1, 128, 8, 8, 64, 3, 3, 1, 1, 1, 1, 0, err, 256)
    assert rc == CB_EINVAL and b"static scratch" in err.value
    # stride 2 is outside the covered geometry
    rc = lib.cb_conv_fwd_noalloc(0, None, p, p, p, None, 1, 16, 8, 8, 16, 3, 3, 2, 2, 1, 1, 0, err, 256)
    assert rc == CB_EUNSUPPORTED and err.value
    torch.cuda.synchronize()
    assert not buf.any()
