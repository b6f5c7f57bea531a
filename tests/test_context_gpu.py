"""Context behaviour on the GPU: the bounded-wait path, the workspace freeze, the device check."""
import ctypes

import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_the_context_stays_usable():
    """A kernel waits (limit 5 ms) on a barrier nothing ever arrives at: it must RETURN, leaving its status; the host
    reads CB_ETIMEOUT from cb_synchronize, and the next call on the same context succeeds."""
    import torch
    from crusaderbackend_b200._lib import CB_ETIMEOUT
    from crusaderbackend_b200.api import Context, CrusaderError
    ctx = Context(0, math="tf32", sync=False)
    assert ctx.lib.cb_selftest_wait_timeout(ctx.h, 5) == 0
    with pytest.raises(CrusaderError) as exc:
        ctx.synchronize()
    assert exc.value.code == CB_ETIMEOUT and "timed out" in str(exc.value)
    ctx.synchronize()  # the status word was cleared
    A = torch.randn(256, 128, device="cuda")
    B = torch.randn(128, 64, device="cuda")
    Cc = torch.empty(256, 64, device="cuda")
    ctx.gemm(A, B, Cc)
    ctx.synchronize()
    assert torch.allclose(Cc, A @ B, atol=0.5, rtol=2e-2)
    # in sync mode the call itself reports it
    ctx.set_sync(True)
    assert ctx.lib.cb_selftest_wait_timeout(ctx.h, 2) == CB_ETIMEOUT
    ctx.synchronize()
    ctx.close()


def test_frozen_workspace_refuses_to_grow():
    import torch
    from crusaderbackend_b200._lib import CB_ENOMEM
    from crusaderbackend_b200.api import Context, CrusaderError
    ctx = Context(0, math="tf32", sync=True)
    W = torch.randn(16, 16, 3, 3, device="cuda")
    X = torch.randn(2, 16, 32, 32, device="cuda")
    Y = torch.empty(2, 16, 32, 32, device="cuda")
    ctx.conv(W, X, Y, 1, 1, 1, 1)                      # small packed filter in the workspace
    assert ctx.lib.cb_freeze_workspace(ctx.h, 1) == 0
    W2 = torch.randn(64, 64, 3, 3, device="cuda")
    X2 = torch.randn(2, 64, 32, 32, device="cuda")
    Y2 = torch.empty(2, 64, 32, 32, device="cuda")
    with pytest.raises(CrusaderError) as exc:
        ctx.conv(W2, X2, Y2, 1, 1, 1, 1)               # needs a larger block
    assert exc.value.code == CB_ENOMEM and "frozen" in str(exc.value)
    ctx.conv(W, X, Y, 1, 1, 1, 1)                      # what fits still runs
    assert ctx.lib.cb_freeze_workspace(ctx.h, 0) == 0
    ctx.conv(W2, X2, Y2, 1, 1, 1, 1)
    ctx.close()


def test_tensor_maps_are_encoded_once_per_tensor_and_tiling():
    """A context keeps the tensor maps it has encoded, keyed by (pointer, extents, strides, box, swizzle): repeating a
    call on the same tensors encodes nothing new and gives the same bits; other tensors of the same shape get maps of
    their own."""
    import torch
    from crusaderbackend_b200.api import Context
    ctx = Context(0, math="tf32", sync=True)
    ctx.set_deterministic(True)  # no split-K atomics: repeated products are bit-identical
    stats = ctx.lib.cb_debug_tmap_stats
    stats.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong)]
    stats.restype = ctypes.c_int

    def read():
        h, m = ctypes.c_longlong(0), ctypes.c_longlong(0)
        assert stats(ctx.h, ctypes.byref(h), ctypes.byref(m)) == 0
        return h.value, m.value

    A = torch.randn(256, 128, device="cuda")
    B = torch.randn(128, 192, device="cuda")
    C1, C2 = torch.empty(256, 192, device="cuda"), torch.empty(256, 192, device="cuda")
    W = torch.randn(16, 16, 3, 3, device="cuda")
    X = torch.randn(4, 16, 32, 32, device="cuda")
    Y1, Y2 = torch.empty(4, 16, 32, 32, device="cuda"), torch.empty(4, 16, 32, 32, device="cuda")
    ctx.gemm(A, B, C1)
    ctx.conv(W, X, Y1, 1, 1, 1, 1)
    h0, m0 = read()
    assert m0 >= 4  # two operand maps for the product, input / filter (/ output) maps for the convolution
    ctx.gemm(A, B, C1)
    ctx.conv(W, X, Y1, 1, 1, 1, 1)
    h1, m1 = read()
    assert m1 == m0 and h1 - h0 == m0 + h0
    ctx.gemm(A, B, C2)
    ctx.conv(W, X, Y2, 1, 1, 1, 1)
    h2, m2 = read()
    assert torch.equal(C1, C2) and torch.equal(Y1, Y2)
    assert m2 - m1 <= 2  # only the outputs differ: at most their maps are new
    A2 = A.clone()
    ctx.gemm(A2, B, C2)
    _, m3 = read()
    assert m3 == m2 + 1 and torch.equal(C1, C2)
    ctx.close()
