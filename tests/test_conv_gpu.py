"""Convolution forward / data-gradient / weight-gradient parity on a B200 against the fp64 CPU oracle and the
golden vectors recorded from the reference's own kernels. Tolerances on max|y - y64| / max|y64|:
TF32 <= 2e-3, 3xTF32 <= 1e-5, fp32 CUDA-core path <= 2e-6 (5e-6 for the long weight-gradient sums)."""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TOL = {"tf32": 2e-3, "3xtf32": 1e-5, "fp32": 5e-6}
MATHS = ["tf32", "3xtf32", "fp32"]


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch


@pytest.fixture(scope="module")
def ctxs(torch_cuda):
    from crusaderbackend_b200.api import Context
    c = {m: Context(0, math=m, sync=True) for m in MATHS}
    yield c
    for v in c.values():
        v.close()


def tol_for(ctx, math):
    return TOL["fp32"] if ctx.last_kernel == "simt_fp32" else TOL[math]


def conv_case(key, N, IC, H, W, OC, F, s, p, bias=False):
    OH, OW = orc.conv_out_hw(H, W, F, F, s, s, p, p)
    return dict(W=orc.he_normal_filter(OC, IC, F, F, key), X=orc.normal((N, IC, H, W), key, "X"),
                dY=orc.normal((N, OC, OH, OW), key, "dY"), bias=orc.normal((OC,), key, "b") if bias else None,
                s=(s, s), p=(p, p))


def run_three_passes(torch, ctx, c, dW0=None, relu=False):
    W, X, dY = (torch.from_numpy(c[k]).cuda() for k in ("W", "X", "dY"))
    b = None if c["bias"] is None else torch.from_numpy(c["bias"]).cuda()
    (sH, sW), (pH, pW) = c["s"], c["p"]
    Y = torch.full(dY.shape, float("nan"), device="cuda")
    ctx.conv(W, X, Y, sH, sW, pH, pW, b, relu=relu)
    kY = ctx.last_kernel
    dX = torch.full(X.shape, float("nan"), device="cuda")
    ctx.convDerive(W, dY, dX, sH, sW, pH, pW)
    kX = ctx.last_kernel
    dW = torch.zeros(W.shape, device="cuda") if dW0 is None else torch.from_numpy(dW0).cuda()
    ctx.convError(dY, X, dW, sH, sW, pH, pW, accumulate=True)
    kW = ctx.last_kernel
    return Y.cpu().numpy(), dX.cpu().numpy(), dW.cpu().numpy(), (kY, kX, kW)


def check_three_passes(torch, ctx, math, c, dW0=None):
    Y, dX, dW, kern = run_three_passes(torch, ctx, c, dW0)
    t = [TOL["fp32"] if k == "simt_fp32" else TOL[math] for k in kern]
    assert orc.max_err_norm(Y, orc.conv_fwd(c["W"], c["X"], c["bias"], c["s"], c["p"])) <= t[0], ("fwd", kern)
    assert orc.max_err_norm(dX, orc.conv_dgrad(c["W"], c["dY"], c["X"].shape, c["s"], c["p"])) <= t[1], ("dgrad", kern)
    want = orc.conv_wgrad(c["dY"], c["X"], c["W"].shape, c["s"], c["p"], dW_init=dW0)
    assert orc.max_err_norm(dW, want) <= t[2], ("wgrad", kern)
    return kern


@pytest.mark.parametrize("math", MATHS)
@pytest.mark.parametrize("name", ["conv_s1_bias", "conv_s2", "conv_1x1", "conv_wide"])
def test_golden_cases(torch_cuda, ctxs, golden, name, math):
    """Same seeded inputs as the recorded runs of the reference's conv / convDerive / convError."""
    from tests.golden.make_golden import CASES, inputs
    c0 = CASES[name]
    x = inputs(name, c0)
    c = dict(W=x["W"], X=x["X"], dY=x["dY"], bias=x["bias"], s=(c0["s"], c0["s"]), p=(c0["p"], c0["p"]))
    Y, dX, dW, kern = run_three_passes(torch_cuda, ctxs[math], c, dW0=x["dW0"])
    t = [TOL["fp32"] if k == "simt_fp32" else TOL[math] for k in kern]
    assert orc.max_err_norm(Y, golden[name + "/Y"]) <= max(t[0], 2e-5)
    assert orc.max_err_norm(dX, golden[name + "/dX"]) <= max(t[1], 2e-5)
    if c0["s"] == 1:  # the reference's weight gradient is only right for stride 1
        assert orc.max_err_norm(dW, golden[name + "/dW"]) <= max(t[2], 2e-5)
    check_three_passes(torch_cuda, ctxs[math], math, c, dW0=x["dW0"])


RESNET56_LAYERS = [  # (IC, H, OC, F, s, p) at a reduced batch
    (3, 32, 16, 3, 1, 1), (16, 32, 16, 3, 1, 1), (16, 32, 32, 3, 2, 1), (16, 32, 32, 1, 2, 0),
    (32, 16, 32, 3, 1, 1), (32, 16, 64, 3, 2, 1), (32, 16, 64, 1, 2, 0), (64, 8, 64, 3, 1, 1),
]


@pytest.mark.parametrize("math", MATHS)
@pytest.mark.parametrize("layer", RESNET56_LAYERS)
def test_resnet56_layer_shapes(torch_cuda, ctxs, layer, math):
    IC, H, OC, F, s, p = layer
    c = conv_case(("r56", layer), 6, IC, H, H, OC, F, s, p)
    check_three_passes(torch_cuda, ctxs[math], math, c)


DENSENET_LAYERS = [  # (IC, H, OC, F): the widest 1x1 bottleneck / transition convolutions and a 3x3 growth layer of BC-100
    (300, 16, 150, 1), (264, 16, 48, 1), (342, 8, 48, 1), (200, 16, 40, 3), (48, 8, 12, 3),
]


@pytest.mark.parametrize("math", ["tf32", "3xtf32"])
@pytest.mark.parametrize("layer", DENSENET_LAYERS)
def test_densenet_layer_shapes_stay_on_the_tensor_cores(torch_cuda, ctxs, layer, math):
    """Filters wider than one launch covers (more than 256 input or 128 output channels in the weight gradient, more
    than 256 accumulator columns in the data gradient) are cut into channel blocks resp. split over more CTAs; all three
    passes must come from the tensor-core kernels and match the oracle."""
    IC, H, OC, F = layer
    c = conv_case(("dn", layer), 4, IC, H, H, OC, F, 1, 1 if F == 3 else 0)
    kern = check_three_passes(torch_cuda, ctxs[math], math, c, dW0=orc.normal((OC, IC, F, F), "dn", "dW0", IC))
    assert all(k.startswith("umma") for k in kern), kern


@pytest.mark.parametrize("deterministic", [False, True])
@pytest.mark.parametrize("math", ["tf32", "3xtf32"])
@pytest.mark.parametrize("geo", [(8, 16, 32, 16, 3, 1), (4, 342, 8, 48, 1, 1), (4, 300, 16, 150, 1, 1), (8, 32, 32, 64, 3, 2),
                                 (8, 16, 32, 32, 1, 2), (8, 3, 32, 16, 3, 1)])
def test_weight_gradient_overwrite_and_accumulate(torch_cuda, geo, math, deterministic):
    """convError in both of its output modes on the tensor-core kernel: `dW =` over a buffer full of NaN (the default
    context clears the filter block, or the strided rows of a block of a wide filter, before its CTAs add into it)
    and `dW +=` on top of the result (twice the gradient), one-launch and fixed-order forms, stride 1 and 2."""
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    N, IC, H, OC, F, s = geo
    p = 1 if F == 3 else 0
    c = conv_case(("wmode", geo), N, IC, H, H, OC, F, s, p)
    ctx = Context(0, math=math, sync=True)
    ctx.set_deterministic(deterministic)
    X, dY = torch.from_numpy(c["X"]).cuda(), torch.from_numpy(c["dY"]).cuda()
    dW = torch.full((OC, IC, F, F), float("nan"), device="cuda")
    ctx.convError(dY, X, dW, s, s, p, p, accumulate=False)
    assert ctx.last_kernel.startswith("umma"), ctx.last_kernel
    want = orc.conv_wgrad(c["dY"], c["X"], (OC, IC, F, F), (s, s), (p, p))
    assert orc.max_err_norm(dW.cpu().numpy(), want) <= TOL[math]
    ctx.convError(dY, X, dW, s, s, p, p, accumulate=True)
    assert orc.max_err_norm(dW.cpu().numpy(), 2.0 * want) <= 2 * TOL[math]
    ctx.close()


@pytest.mark.parametrize("math", MATHS)
@pytest.mark.parametrize("geo", [(2, 3, 7, 9, 5, 3, 1, 1), (1, 4, 11, 11, 6, 5, 1, 2), (3, 8, 12, 12, 8, 3, 2, 1),
                                 (2, 5, 6, 6, 4, 1, 1, 0), (2, 12, 8, 8, 24, 3, 1, 1), (4, 48, 16, 16, 12, 3, 1, 1)])
def test_odd_geometries(torch_cuda, ctxs, geo, math):
    N, IC, H, W, OC, F, s, p = geo
    c = conv_case(("odd", geo), N, IC, H, W, OC, F, s, p, bias=True)
    check_three_passes(torch_cuda, ctxs[math], math, c, dW0=orc.normal((OC, IC, F, F), "odd", geo, "dW0"))


@pytest.mark.parametrize("math", MATHS)
def test_fused_bias_relu_epilogue(torch_cuda, ctxs, math):
    torch = torch_cuda
    c = conv_case("relu", 4, 16, 16, 16, 32, 3, 1, 1, bias=True)
    W, X, b = (torch.from_numpy(c[k]).cuda() for k in ("W", "X", "bias"))
    Y = torch.empty((4, 32, 16, 16), device="cuda")
    ctxs[math].conv(W, X, Y, 1, 1, 1, 1, b, relu=True)
    ref = np.maximum(orc.conv_fwd(c["W"], c["X"], c["bias"], (1, 1), (1, 1)), 0.0)
    assert orc.max_err_norm(Y.cpu().numpy(), ref) <= tol_for(ctxs[math], math)


@pytest.mark.parametrize("math", ["tf32", "3xtf32"])
@pytest.mark.parametrize("stride2", [False, True])
def test_config3_full_size(torch_cuda, ctxs, math, stride2):
    """3x3 conv, NCHW fp32, N=128: C=K=64 at 32x32 stride 1, and the 32->64 stride-2 downsample. The fp64 oracle
    replays three images of the batch for forward / data-gradient; the weight gradient (a sum over the whole
    batch) is checked through the adjoint identity <dW, V> = <dY, conv(V, X)> on a seeded direction V, with
    conv(V, X) taken from the oracle on a batch slice and from the checked forward pass on the rest."""
    torch = torch_cuda
    ctx = ctxs[math]
    IC, OC, s = (32, 64, 2) if stride2 else (64, 64, 1)
    c = conv_case(("c3", stride2), 128, IC, 32, 32, OC, 3, s, 1)
    Y, dX, dW, kern = run_three_passes(torch, ctx, c)
    t = [TOL["fp32"] if k == "simt_fp32" else TOL[math] for k in kern]
    sel = [0, 77, 127]
    ref_Y = orc.conv_fwd(c["W"], c["X"][sel], None, c["s"], c["p"])
    assert orc.max_err_norm(Y[sel], ref_Y) <= t[0]
    ref_dX = orc.conv_dgrad(c["W"], c["dY"][sel], c["X"][sel].shape, c["s"], c["p"])
    assert orc.max_err_norm(dX[sel], ref_dX) <= t[1]
    # weight gradient: exact oracle on the first 8 images' contribution is not separable, so use the adjoint
    V = orc.he_normal_filter(OC, IC, 3, 3, "c3", "V")
    Yv = torch.empty(Y.shape, device="cuda")
    ctxs["3xtf32"].conv(torch.from_numpy(V).cuda(), torch.from_numpy(c["X"]).cuda(), Yv, s, s, 1, 1)
    rhs = float((Yv.double().cpu().numpy() * c["dY"].astype(np.float64)).sum())
    lhs = float((dW.astype(np.float64) * V).sum())
    scale = float(np.abs(Yv.double().cpu().numpy() * c["dY"]).sum())
    assert abs(lhs - rhs) / scale <= t[2]
    # and a direct oracle comparison at reduced batch, full spatial / channel size
    c8 = {k: (v[:8] if k in ("X", "dY") else v) for k, v in c.items()}
    _, _, dW8, k8 = run_three_passes(torch, ctx, c8)
    want = orc.conv_wgrad(c8["dY"], c8["X"], c["W"].shape, c["s"], c["p"])
    assert orc.max_err_norm(dW8, want) <= (TOL["fp32"] if k8[2] == "simt_fp32" else TOL[math])


def test_empty_batch_and_argument_errors(torch_cuda, ctxs):
    import ctypes
    from crusaderbackend_b200._lib import CB_EINVAL
    torch = torch_cuda
    ctx = ctxs["tf32"]
    buf = torch.full((64,), 3.0, device="cuda")
    p = ctypes.c_void_p(buf.data_ptr())
    lib, h = ctx.lib, ctx.h
    assert lib.cb_conv_fwd(h, p, p, p, None, 0, 2, 4, 4, 2, 3, 3, 1, 1, 1, 1, 0) == 0          # empty batch
    assert lib.cb_conv_dgrad(h, p, p, p, 0, 2, 4, 4, 2, 3, 3, 1, 1, 1, 1) == 0
    assert (buf == 3.0).all()
    dW = torch.full((2, 2, 3, 3), 5.0, device="cuda")
    pw = ctypes.c_void_p(dW.data_ptr())
    assert lib.cb_conv_wgrad(h, p, p, pw, 0, 2, 4, 4, 2, 3, 3, 1, 1, 1, 1, 1) == 0              # accumulate: unchanged
    ctx.synchronize()
    assert (dW == 5.0).all()
    assert lib.cb_conv_wgrad(h, p, p, pw, 0, 2, 4, 4, 2, 3, 3, 1, 1, 1, 1, 0) == 0              # overwrite: zeros
    ctx.synchronize()
    assert (dW == 0.0).all()
    assert lib.cb_conv_fwd(h, p, p, p, None, 1, 2, 4, 4, 2, 3, 3, 0, 1, 1, 1, 0) == CB_EINVAL   # stride 0
    assert lib.cb_conv_fwd(h, p, p, p, None, 1, 2, 2, 2, 2, 5, 5, 1, 1, 0, 0, 0) == CB_EINVAL   # filter > input
    assert lib.cb_conv_fwd(h, None, p, p, None, 1, 2, 4, 4, 2, 3, 3, 1, 1, 1, 1, 0) == CB_EINVAL


def test_bias_add_and_bias_grad(torch_cuda, ctxs):
    torch = torch_cuda
    ctx = ctxs["fp32"]
    Y0 = orc.normal((3, 5, 4, 6), "bias", "Y")
    b = orc.normal((5,), "bias", "b")
    Y = torch.from_numpy(Y0).cuda()
    ctx.convBias(Y, torch.from_numpy(b).cuda())
    assert np.allclose(Y.cpu().numpy(), Y0 + b[None, :, None, None], atol=1e-6)
    db = torch.ones(5, device="cuda")
    ctx.convBiasGrad(torch.from_numpy(Y0).cuda(), db, accumulate=True)
    assert orc.max_err_norm(db.cpu().numpy(), orc.conv_bias_grad(Y0) + 1.0) <= 2e-6
    ctx.convBiasGrad(torch.from_numpy(Y0).cuda(), db, accumulate=False)
    assert orc.max_err_norm(db.cpu().numpy(), orc.conv_bias_grad(Y0)) <= 2e-6
