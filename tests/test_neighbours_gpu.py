"""Linear layers and the memory-bound neighbours (BatchNorm, ReLU, pooling, softmax / cross-entropy, Momentum,
tensor arithmetic) on a B200 against the fp64 oracle and the golden vectors of the reference's kernels."""
import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

F32 = 5e-6
TOL = {"tf32": 2e-3, "3xtf32": 1e-5, "fp32": F32}


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch


@pytest.fixture(scope="module")
def ctxs(torch_cuda):
    from crusaderbackend_b200.api import Context
    c = {m: Context(0, math=m, sync=True) for m in TOL}
    yield c
    for v in c.values():
        v.close()


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


@pytest.mark.parametrize("math", list(TOL))
@pytest.mark.parametrize("batch,IN,OUT", [(128, 64, 10), (12, 20, 10), (7, 13, 5), (128, 4096, 10), (64, 342, 10),
                                          (128, 1024, 1024), (1, 8, 3)])
def test_linear_three_passes(torch_cuda, ctxs, batch, IN, OUT, math):
    torch = torch_cuda
    ctx = ctxs[math]
    key = ("lin", batch, IN, OUT)
    X, W, b = orc.normal((batch, IN), key, "X"), orc.normal((OUT, IN), key, "W"), orc.normal((OUT,), key, "b")
    dY, dW0, db0 = orc.normal((batch, OUT), key, "dY"), orc.normal((OUT, IN), key, "dW0"), orc.normal((OUT,), key, "db0")
    Y = torch.full((batch, OUT), float("nan"), device="cuda")
    ctx.linear(dev(torch, X), dev(torch, W), dev(torch, b), Y)
    t = F32 if ctx.last_kernel == "simt_fp32" else TOL[math]
    assert orc.max_err_norm(Y.cpu().numpy(), orc.linear(X, W, b)) <= t
    dX = torch.full((batch, IN), float("nan"), device="cuda")
    ctx.linearXGrad(dev(torch, dY), dev(torch, W), dX)
    t = F32 if ctx.last_kernel == "simt_fp32" else TOL[math]
    assert orc.max_err_norm(dX.cpu().numpy(), orc.linear_xgrad(dY, W)) <= t
    dW, db = dev(torch, dW0), dev(torch, db0)
    ctx.linearParamGrad(dev(torch, dY), dev(torch, X), dW, db)
    t = F32 if ctx.last_kernel == "simt_fp32" else TOL[math]
    rW, rb = orc.linear_paramgrad(dY, X, dW0, db0)
    assert orc.max_err_norm(dW.cpu().numpy(), rW) <= t
    assert orc.max_err_norm(db.cpu().numpy(), rb) <= F32


def test_golden_linear(torch_cuda, ctxs, golden):
    from tests.golden.make_golden import CASES, inputs
    torch = torch_cuda
    ctx = ctxs["3xtf32"]
    for name in ("linear", "linear_scalar"):
        c = CASES[name]
        x = inputs(name, c)
        Y = torch.empty((c["batch"], c["OUT"]), device="cuda")
        ctx.linear(dev(torch, x["X"]), dev(torch, x["W"]), dev(torch, x["b"]), Y)
        assert orc.max_err_norm(Y.cpu().numpy(), golden[name + "/Y"]) <= 2e-5
        dX = torch.empty((c["batch"], c["IN"]), device="cuda")
        ctx.linearXGrad(dev(torch, x["dY"]), dev(torch, x["W"]), dX)
        assert orc.max_err_norm(dX.cpu().numpy(), golden[name + "/dX"]) <= 2e-5
        dW = dev(torch, x["dW0"])
        ctx.linearParamGrad(dev(torch, x["dY"]), dev(torch, x["X"]), dW, None)
        assert orc.max_err_norm(dW.cpu().numpy(), golden[name + "/dW"]) <= 2e-5


@pytest.mark.parametrize("shape", [(8, 3, 5, 5), (128, 16, 32, 32), (96, 7, 3, 3), (130, 64, 8, 8), (2, 1, 1, 1), (16, 32, 16, 16),
                                   (300, 4, 4, 4), (64, 342, 8, 8)])
def test_batchnorm(torch_cuda, ctxs, shape):
    """Statistics per (c,h,w) over the batch; batch sizes above the reference's limit of 96 are accepted."""
    torch = torch_cuda
    ctx = ctxs["fp32"]
    X = orc.normal(shape, "bn", shape, "X") * 2 + 0.5
    dY = orc.normal(shape, "bn", shape, "dY")
    g = orc.uniform_pm1(shape[1:], "bn", shape, "g") + 1.5
    b = orc.uniform_pm1(shape[1:], "bn", shape, "b")
    dX_, Y, xh = (torch.full(shape, float("nan"), device="cuda") for _ in range(3))
    mean, var, dg, db = (torch.full(shape[1:], float("nan"), device="cuda") for _ in range(4))
    ctx.batchNorm(dev(torch, X), dev(torch, b), dev(torch, g), mean, var, Y, xh)
    rY, rxh, rmean, rvar = orc.bn_fwd(X, b, g)
    assert orc.max_err_norm(Y.cpu().numpy(), rY) <= F32
    assert orc.max_err_norm(xh.cpu().numpy(), rxh) <= F32
    assert orc.max_err_norm(mean.cpu().numpy().ravel(), rmean) <= F32
    assert orc.max_err_norm(var.cpu().numpy().ravel(), rvar) <= F32
    ctx.batchNormGrad(dev(torch, dY), dev(torch, g), dev(torch, X), dX_)
    # the backward cancels to ~0 for tiny batches: measure the error against the size of the terms that cancel
    ref_dX = orc.bn_bwd(dY, g, X)
    term = np.abs(dY.astype(np.float64) * g / np.sqrt(rvar.reshape(shape[1:]) + 1e-8)).max()
    assert np.abs(dX_.cpu().numpy() - ref_dX).max() <= 2e-5 * max(np.abs(ref_dX).max(), term)
    ctx.batchNormParamGrads(dev(torch, dY), xh, dg, db)
    rdg, rdb = orc.bn_paramgrad(dY, xh.cpu().numpy())
    assert orc.max_err_norm(dg.cpu().numpy().ravel(), rdg) <= F32
    assert orc.max_err_norm(db.cpu().numpy().ravel(), rdb) <= F32
    # the fused backward (dX, dgamma, dbeta in one pass, x-hat recomputed) agrees with the two separate calls
    if shape[0] <= 256 and np.prod(shape[1:]) % 4 == 0:
        dX2 = torch.full(shape, float("nan"), device="cuda")
        dg2, db2 = (torch.full(shape[1:], float("nan"), device="cuda") for _ in range(2))
        ctx.batchNormGradFused(dev(torch, dY), dev(torch, g), dev(torch, X), dX2, dg2, db2)
        assert np.abs(dX2.cpu().numpy() - ref_dX).max() <= 2e-5 * max(np.abs(ref_dX).max(), term)
        assert orc.max_err_norm(dg2.cpu().numpy().ravel(), rdg) <= 2e-5
        assert orc.max_err_norm(db2.cpu().numpy().ravel(), rdb) <= F32
        # BatchNorm -> ReLU folded: forward relu(bn(X)); backward with dY masked by the ReLU output
        R = torch.full(shape, float("nan"), device="cuda")
        ctx.batchNormRelu(dev(torch, X), dev(torch, b), dev(torch, g), R)
        assert orc.max_err_norm(R.cpu().numpy(), np.maximum(rY, 0)) <= F32
        dYm = np.where(R.cpu().numpy() > 0, dY, 0).astype(np.float32)
        ctx.batchNormGradFused(dev(torch, dY), dev(torch, g), dev(torch, X), dX2, dg2, db2, relu_out=R)
        ref_m = orc.bn_bwd(dYm, g, X)
        assert np.abs(dX2.cpu().numpy() - ref_m).max() <= 2e-5 * max(np.abs(ref_m).max(), term)
        rdg_m, rdb_m = orc.bn_paramgrad(dYm, xh.cpu().numpy())
        assert orc.max_err_norm(dg2.cpu().numpy().ravel(), rdg_m) <= 2e-5
        assert orc.max_err_norm(db2.cpu().numpy().ravel(), rdb_m) <= F32


def test_golden_batchnorm(torch_cuda, ctxs, golden):
    from tests.golden.make_golden import CASES, inputs
    torch = torch_cuda
    ctx = ctxs["fp32"]
    x = inputs("bn", CASES["bn"])
    shape = x["X"].shape
    Y, xh, dX_ = (torch.empty(shape, device="cuda") for _ in range(3))
    mean, var, dg, db = (torch.empty(shape[1:], device="cuda") for _ in range(4))
    ctx.batchNorm(dev(torch, x["X"]), dev(torch, x["beta"]), dev(torch, x["gamma"]), mean, var, Y, xh)
    ctx.batchNormGrad(dev(torch, x["dY"]), dev(torch, x["gamma"]), dev(torch, x["X"]), dX_)
    ctx.batchNormParamGrads(dev(torch, x["dY"]), xh, dg, db)
    for k, v in dict(Y=Y, xhat=xh, mean=mean, var=var, dgamma=dg, dbeta=db).items():
        assert orc.max_err_norm(v.cpu().numpy(), golden["bn/" + k]) <= 2e-5, k
    assert orc.max_err_norm(dX_.cpu().numpy(), golden["bn/dX"]) <= 1e-4


@pytest.mark.parametrize("n", [0, 1, 3, 1000, 1 << 20, (1 << 20) + 3])
def test_relu_and_tensor_ops_bit_exact(torch_cuda, ctxs, n):
    from crusaderbackend_b200 import _lib as L
    torch = torch_cuda
    ctx = ctxs["fp32"]
    X, dY = orc.normal((n,), "relu", n, "X"), orc.normal((n,), "relu", n, "dY")
    dXd, Yd = torch.full((n,), 9.0, device="cuda"), torch.full((n,), 9.0, device="cuda")
    ctx.relu(dev(torch, X), Yd)
    ctx.reluGradFast(dev(torch, X), dev(torch, dY), dXd)
    assert np.array_equal(Yd.cpu().numpy(), np.maximum(X, 0))
    assert np.array_equal(dXd.cpu().numpy(), np.where(X > 0, dY, 0).astype(np.float32))
    A = dev(torch, X)
    ctx.tensor_op(L.CB_OP_ADD, A, dev(torch, dY))
    assert np.array_equal(A.cpu().numpy(), X + dY)
    ctx.tensor_op(L.CB_OP_MUL_SCALAR, A, None, 1.0 - 1e-4)
    assert np.array_equal(A.cpu().numpy(), (X + dY) * np.float32(1.0 - 1e-4))
    ctx.tensor_op(L.CB_OP_SUB, A, dev(torch, dY))
    ctx.tensor_op(L.CB_OP_DIV_SCALAR, A, None, 3.0)
    ctx.tensor_op(L.CB_OP_FILL, A, None, 2.5)
    assert (A == 2.5).all()
    dA, res = dev(torch, X), dev(torch, dY)
    ctx.grad_handover(dA, res)
    assert np.array_equal(dA.cpu().numpy(), X + dY) and not res.any()
    out = torch.full((n,), 9.0, device="cuda")
    ctx.addRelu(dev(torch, X), dev(torch, dY), out)
    assert np.array_equal(out.cpu().numpy(), np.maximum(X + dY, 0))
    ga, gb = torch.full((n,), 9.0, device="cuda"), torch.full((n,), 9.0, device="cuda")
    ctx.reluGrad2(out, dev(torch, dY), ga, gb)
    want = np.where(np.maximum(X + dY, 0) > 0, dY, 0).astype(np.float32)
    assert np.array_equal(ga.cpu().numpy(), want) and np.array_equal(gb.cpu().numpy(), want)


def test_pooling_softmax_loss(torch_cuda, ctxs, golden):
    from tests.golden.make_golden import CASES, inputs
    torch = torch_cuda
    ctx = ctxs["fp32"]
    for shape in [(2, 3, 8, 8), (128, 64, 8, 8), (64, 108, 32, 32), (3, 5, 6, 10)]:
        X = orc.normal(shape, "pool", shape)
        N, Cc, H, W = shape
        Yp = torch.empty((N, Cc, H // 2, W // 2), device="cuda")
        ctx.avgPool(dev(torch, X), Yp)
        assert orc.max_err_norm(Yp.cpu().numpy(), orc.avgpool(X)) <= F32
        dYp = orc.normal(Yp.shape, "pool", shape, "dY")
        dXp = torch.full(shape, float("nan"), device="cuda")
        ctx.avgPoolBack(dXp, dev(torch, dYp))
        assert orc.max_err_norm(dXp.cpu().numpy(), orc.avgpool_back(dYp, shape)) <= F32
        Yg = torch.empty((N, Cc), device="cuda")
        ctx.globalAvgPool(dev(torch, X), Yg)
        assert orc.max_err_norm(Yg.cpu().numpy(), orc.gap(X)) <= F32
        dYg = orc.normal((N, Cc), "pool", shape, "dYg")
        dXg = torch.full(shape, float("nan"), device="cuda")
        ctx.globalAvgPoolBack(dXg, dev(torch, dYg))
        assert orc.max_err_norm(dXg.cpu().numpy(), orc.gap_back(dYg, shape)) <= F32
    x = inputs("pool", CASES["pool"])
    Yp = torch.empty(golden["pool/Yp"].shape, device="cuda")
    ctx.avgPool(dev(torch, x["X"]), Yp)
    assert orc.max_err_norm(Yp.cpu().numpy(), golden["pool/Yp"]) <= 2e-6
    # softmax + cross entropy
    for rows, step in [(6, 10), (128, 10), (5, 1000), (3, 1)]:
        X = orc.normal((rows, step), "sm", rows, step) * 3
        S = torch.empty((rows, step), device="cuda")
        ctx.softmax(dev(torch, X), S)
        assert orc.max_err_norm(S.cpu().numpy(), orc.softmax(X)) <= F32
        lab = np.zeros((rows, step), dtype=np.float32)
        lab[np.arange(rows), orc.rng_for("lab", rows, step).integers(0, step, rows)] = 1
        dS, loss = torch.empty_like(S), torch.full((1,), 7.0, device="cuda")
        ctx.crossEntropy(S, dev(torch, lab), dS, loss)
        rl, rdS = orc.cross_entropy(S.cpu().numpy(), lab)
        assert abs(loss.item() - rl) <= 1e-5 * max(1.0, abs(rl))
        assert orc.max_err_norm(dS.cpu().numpy(), rdS) <= 1e-6
    x = inputs("softmax", CASES["softmax"])
    S = torch.empty(x["X"].shape, device="cuda")
    ctx.softmax(dev(torch, x["X"]), S)
    assert orc.max_err_norm(S.cpu().numpy(), golden["softmax/Y"]) <= 2e-6


def test_momentum_single_and_multi(torch_cuda, ctxs, golden):
    from tests.golden.make_golden import CASES, inputs
    torch = torch_cuda
    ctx = ctxs["fp32"]
    c = CASES["momentum"]
    x = inputs("momentum", c)
    w, g, m = dev(torch, x["w"]), dev(torch, x["g"]), dev(torch, x["m"])
    ctx.momentumApply(w, g, m, c["lr"], c["beta"], c["l2"], True)
    assert orc.max_err_norm(w.cpu().numpy(), golden["momentum/w"]) <= 1e-6
    assert orc.max_err_norm(m.cpu().numpy(), golden["momentum/m"]) <= 1e-6
    assert not g.any()
    sizes = [1000, 36864, 10, 16384, 7]
    flags = [True, True, False, False, True]
    ws = [orc.normal((n,), "mm", i, "w") for i, n in enumerate(sizes)]
    gs = [orc.normal((n,), "mm", i, "g") for i, n in enumerate(sizes)]
    ms = [orc.normal((n,), "mm", i, "m") for i, n in enumerate(sizes)]
    dw, dg, dm = ([dev(torch, a) for a in t] for t in (ws, gs, ms))
    ctx.momentumApplyMulti(dw, dg, dm, flags, 0.01 / 128, 0.9, 1e-4)
    for i in range(len(sizes)):
        rw, rm, _ = orc.momentum(ws[i], gs[i], ms[i], 0.01 / 128, 0.9, 1e-4, flags[i])
        assert orc.max_err_norm(dw[i].cpu().numpy(), rw) <= 1e-6
        assert orc.max_err_norm(dm[i].cpu().numpy(), rm) <= 1e-6
        assert not dg[i].any()


def test_strided_batchnorm_and_pooling_match_dense_forms(torch_cuda, ctxs):
    """The batch-strided entry points (a channel prefix of a wider NCHW buffer, as a DenseNet block is laid out) give
    bit for bit what the dense entry points give on a contiguous copy of the same values; the backward form also adds
    onto an existing gradient."""
    import ctypes as C
    torch = torch_cuda
    ctx = ctxs["fp32"]
    lib = ctx.lib
    N, Ct, Cv, H = 48, 20, 12, 8
    P, HW = Cv * H * H, H * H
    wide = torch.from_numpy(orc.normal((N, Ct, H, H), "sbn", "X")).cuda()
    view = wide[:, :Cv]                       # strided: samples Ct*HW apart
    dense = view.contiguous()
    gamma = torch.from_numpy(orc.uniform_pm1((P,), "sbn", "g") + 1.5).cuda()
    beta = torch.from_numpy(orc.uniform_pm1((P,), "sbn", "b")).cuda()
    p = lambda t: C.c_void_p(t.data_ptr())
    y1, y2 = torch.empty(N, P, device="cuda"), torch.empty(N, P, device="cuda")
    ctx._check(lib.cb_bn_fwd_relu_ex(ctx.h, p(view), p(beta), p(gamma), p(y1), N, P, Ct * HW))
    ctx._check(lib.cb_bn_fwd_relu(ctx.h, p(dense), p(beta), p(gamma), p(y2), N, P))
    ctx.synchronize()
    assert torch.equal(y1, y2)
    dy = torch.from_numpy(orc.normal((N, P), "sbn", "dY")).cuda()
    g0 = torch.from_numpy(orc.normal((N, Ct, H, H), "sbn", "G0")).cuda()
    dwide = g0.clone()
    dg1, db1, dg2, db2 = (torch.empty(P, device="cuda") for _ in range(4))
    dx2 = torch.empty(N, P, device="cuda")
    ctx._check(lib.cb_bn_bwd_fused_ex(ctx.h, p(dy), p(gamma), p(view), p(dwide), p(dg1), p(db1), p(y1), N, P, Ct * HW, Ct * HW, 1))
    ctx._check(lib.cb_bn_bwd_fused(ctx.h, p(dy), p(gamma), p(dense), p(dx2), p(dg2), p(db2), p(y2), N, P))
    ctx.synchronize()
    assert torch.equal(dg1, dg2) and torch.equal(db1, db2)
    assert torch.equal(dwide[:, :Cv], g0[:, :Cv] + dx2.view(N, Cv, H, H))
    assert torch.equal(dwide[:, Cv:], g0[:, Cv:])          # the channels beyond the view are untouched
    # pooling into / out of a channel prefix of a wider pooled buffer
    X = torch.from_numpy(orc.normal((N, Cv, H, H), "sbn", "PX")).cuda()
    pooled_wide = torch.zeros(N, Ct, H // 2, H // 2, device="cuda")
    pooled = torch.empty(N, Cv, H // 2, H // 2, device="cuda")
    ctx._check(lib.cb_avgpool_ex(ctx.h, p(X), p(pooled_wide), N, Cv, H, H, 2, 2, Ct * HW // 4))
    ctx._check(lib.cb_avgpool(ctx.h, p(X), p(pooled), N * Cv, H, H, 2, 2))
    ctx.synchronize()
    assert torch.equal(pooled_wide[:, :Cv], pooled) and not pooled_wide[:, Cv:].any()
    dX1, dX2 = torch.empty_like(X), torch.empty_like(X)
    ctx._check(lib.cb_avgpool_back_ex(ctx.h, p(dX1), p(pooled_wide), N, Cv, H, H, 2, 2, Ct * HW // 4))
    ctx._check(lib.cb_avgpool_back(ctx.h, p(dX2), p(pooled), N * Cv, H, H, 2, 2))
    ctx.synchronize()
    assert torch.equal(dX1, dX2)
