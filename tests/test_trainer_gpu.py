"""The ResNet training step on a B200 against the CPU oracle composed from the per-op fp64 oracle
(tests/resnet_oracle.py), and loss tracking of the tensor-core modes against the CUDA-core fp32 run."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.resnet_oracle import ResNetOracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch


def make_batch(torch, batch, hw, classes, key):
    images = orc.normal((batch, 3, hw, hw), key, "img")
    lab = orc.rng_for(key, "lab").integers(0, classes, batch)
    onehot = np.zeros((batch, classes), dtype=np.float32)
    onehot[np.arange(batch), lab] = 1
    return images, onehot, torch.from_numpy(images).cuda(), torch.from_numpy(onehot).cuda()


@pytest.mark.parametrize("math,tol", [("fp32", 2e-4), ("3xtf32", 2e-4), ("tf32", 5e-2)])
def test_resnet8_step_matches_oracle(torch_cuda, math, tol):
    """ResNet-8 (one block per stage), batch 8, 32x32: loss, logits and every parameter gradient. In fp32 and 3xTF32 mode
    every gradient tensor matches the oracle to 2e-4. TF32 rounding is amplified by the batch-of-8 BatchNorm layers
    (division by the spread of 8 samples), so there each gradient tensor is held to a cosine of 0.995 with the
    oracle's and 5e-2 on loss and logits."""
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    ctx = Context(0, math=math, sync=True)
    tr = ResNetTrainer(ctx, batch=8, blocks_per_stage=1, image_hw=32, classes=10)
    oracle = ResNetOracle(1, 32, 10)
    shapes = oracle.param_shapes()
    assert [e["kind"] for e in tr.entries] == [k for k, _ in shapes]
    assert [e["size"] for e in tr.entries] == [int(np.prod(s)) for _, s in shapes]
    host = tr.init_params("r8")
    # perturb gamma / beta so their gradients are exercised away from (1, 0)
    for i, e in enumerate(tr.entries):
        if e["kind"].startswith("bn"):
            host[e["offset"]:e["offset"] + e["size"]] += 0.1 * orc.uniform_pm1((e["size"],), "r8", "bnp", i)
    tr.set_params(host)
    P = [host[e["offset"]:e["offset"] + e["size"]].reshape(s) for e, (_, s) in zip(tr.entries, shapes)]
    images, onehot, dimg, dlab = make_batch(torch, 8, 32, 10, "r8")
    tr.forward(dimg, dlab)
    tr.backward()
    ctx.synchronize()
    loss_ref, G_ref, logits_ref = oracle.run(P, images, onehot)
    assert abs(tr.loss() - loss_ref) <= tol * max(1.0, abs(loss_ref))
    logits = tr.tensor(-1, (8, 10)).cpu().numpy()
    assert orc.max_err_norm(logits, logits_ref) <= tol
    g = tr.grads.cpu().numpy()
    for e, gr in zip(tr.entries, G_ref):
        got = g[e["offset"]:e["offset"] + e["size"]].astype(np.float64)
        want = np.asarray(gr, dtype=np.float64).ravel()
        if math != "tf32":
            assert orc.max_err_norm(got, want) <= tol, (e["kind"], e["dims"])
        else:
            cos = float(got @ want) / max(float(np.linalg.norm(got) * np.linalg.norm(want)), 1e-300)
            assert cos >= 0.995, (e["kind"], e["dims"], cos)
    # one Momentum step: identical to the oracle update applied to the GPU's own gradients
    before_w, before_g = tr.params.cpu().numpy().copy(), g.copy()
    tr.update(0.01 / 8, 0.9, 1e-4)
    ctx.synchronize()
    after = tr.params.cpu().numpy()
    for e in tr.entries:
        sl = slice(e["offset"], e["offset"] + e["size"])
        w, m_, _ = orc.momentum(before_w[sl], before_g[sl], np.zeros(e["size"]), 0.01 / 8, 0.9, 1e-4, e["is_weight"])
        assert orc.max_err_norm(after[sl], w) <= 1e-6
    assert not tr.grads.any()
    tr.close()
    ctx.close()


@pytest.mark.parametrize("math", ["fp32", "3xtf32"])
def test_resnet8_ten_steps_match_oracle(torch_cuda, math):
    """ResNet-8, batch 8: ten consecutive training steps (forward, backward, Momentum update, next forward on the updated
    weights) against the fp64 oracle stepped the same way: every parameter tensor after the tenth step within 2e-4, every
    step's loss within 2e-4."""
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    steps, lr, beta, l2 = 10, 0.01 / 8, 0.9, 1e-4
    ctx = Context(0, math=math, sync=True)
    tr = ResNetTrainer(ctx, batch=8, blocks_per_stage=1, image_hw=32, classes=10)
    oracle = ResNetOracle(1, 32, 10)
    shapes = oracle.param_shapes()
    host = tr.init_params("r8x10")
    for i, e in enumerate(tr.entries):
        if e["kind"].startswith("bn"):
            host[e["offset"]:e["offset"] + e["size"]] += 0.1 * orc.uniform_pm1((e["size"],), "r8x10", "bnp", i)
    tr.set_params(host)
    P = [host[e["offset"]:e["offset"] + e["size"]].reshape(s).astype(np.float32) for e, (_, s) in zip(tr.entries, shapes)]
    M = [np.zeros(p.size) for p in P]
    images, onehot, dimg, dlab = make_batch(torch, 8, 32, 10, "r8x10")
    for s in range(steps):
        tr.forward(dimg, dlab)
        tr.backward()
        got_loss = tr.loss()
        tr.update(lr, beta, l2)
        loss_ref, G_ref, _ = oracle.run(P, images, onehot)
        assert abs(got_loss - loss_ref) <= 2e-4 * max(1.0, abs(loss_ref)), s
        for i, e in enumerate(tr.entries):
            w, m_, _ = orc.momentum(P[i].ravel(), np.asarray(G_ref[i]).ravel(), M[i], lr, beta, l2, e["is_weight"])
            P[i], M[i] = np.asarray(w, dtype=np.float32).reshape(P[i].shape), np.asarray(m_, dtype=np.float64)
    ctx.synchronize()
    after = tr.params.cpu().numpy()
    for i, e in enumerate(tr.entries):
        assert orc.max_err_norm(after[e["offset"]:e["offset"] + e["size"]], P[i].ravel()) <= 2e-4, (e["kind"], e["dims"])
    tr.close()
    ctx.close()


def test_bn_groups_reproduce_sharded_gradients(torch_cuda):
    """Data-parallel ranks take BatchNorm statistics on their own shard. A one-GPU run with two BatchNorm groups on a
    batch of 32 must give the gradients two ranks would sum: the executor run separately on each half of the batch
    (what each rank computes; 2e-5) and the fp64 oracle on each half, summed (2e-4; groups of 16 samples keep the
    per-position variances away from the eps = 1e-8 regime in which fp32 rounding is amplified); the loss is the mean
    over all samples."""
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    B, H = 32, 16
    ctx = Context(0, math="fp32", sync=True)
    full = ResNetTrainer(ctx, batch=B, blocks_per_stage=1, image_hw=32, classes=10)
    half = ResNetTrainer(ctx, batch=H, blocks_per_stage=1, image_hw=32, classes=10)
    host = full.init_params("ghost")
    half.set_params(host)
    full.set_bn_groups(2)
    images, onehot, dimg, dlab = make_batch(torch, B, 32, 10, "ghost")
    full.forward(dimg, dlab)
    full.backward()
    g_full, loss_full = full.grads.cpu().numpy().copy(), full.loss()
    g_sum, loss_sum = np.zeros_like(g_full), 0.0
    oracle = ResNetOracle(1, 32, 10)
    shapes = oracle.param_shapes()
    P = [host[e["offset"]:e["offset"] + e["size"]].reshape(s) for e, (_, s) in zip(full.entries, shapes)]
    G_or = [np.zeros(int(np.prod(s))) for _, s in shapes]
    for h in range(2):
        sl = slice(H * h, H * h + H)
        half.grads.zero_()
        img_h, lab_h = dimg[sl].contiguous(), dlab[sl].contiguous()  # read in place until the backward pass is done
        half.forward(img_h, lab_h)
        half.backward()
        g_sum += half.grads.cpu().numpy()
        loss_sum += half.loss() * H
        _, G_ref, _ = oracle.run(P, images[sl], onehot[sl])
        for i, g in enumerate(G_ref):
            G_or[i] += np.asarray(g, dtype=np.float64).ravel()
    assert abs(loss_full - loss_sum / B) <= 1e-5 * max(1.0, abs(loss_full))
    for i, e in enumerate(full.entries):
        sl = slice(e["offset"], e["offset"] + e["size"])
        assert orc.max_err_norm(g_full[sl], g_sum[sl]) <= 2e-5, (e["kind"], e["dims"])
        assert orc.max_err_norm(g_full[sl], G_or[i]) <= 2e-4, (e["kind"], e["dims"])
    full.close()
    half.close()
    ctx.close()


def test_wgrad_streams_do_not_change_results(torch_cuda):
    """The weight gradients run on streams of their own, concurrently with the rest of the backward pass. On a
    deterministic context (per-CTA partial sums added in a fixed order) gradients after one step and parameters after
    three (eager and as a replayed CUDA graph) are bit-identical for 1 and 3 streams; the inline run (0 streams: its
    kernels split the pixels over more CTAs) and the default context (CTAs add into one accumulator with atomics, in
    whatever order they finish) agree with them to fp32 rounding."""
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    _, _, dimg, dlab = make_batch(torch, 16, 32, 10, "wstreams")
    results = []
    for n, det in ((1, True), (3, True), (0, True), (2, False)):
        ctx = Context(0, math="tf32", sync=False)
        ctx.set_deterministic(det)
        tr = ResNetTrainer(ctx, batch=16, blocks_per_stage=2, image_hw=32, classes=10)
        tr.set_wgrad_streams(n)
        tr.init_params("wstreams")
        l0 = tr.launches
        tr.forward(dimg, dlab)
        tr.backward()
        ctx.synchronize()
        launches = tr.launches - l0
        g1 = tr.grads.clone()
        tr.update(1e-3)
        tr.step(dimg, dlab, 1e-3)
        g = tr.capture_step(dimg, dlab, 1e-3, warmup=0)
        g.replay()
        ctx.synchronize()
        results.append((g1, tr.params.clone(), launches))
        tr.close()
        ctx.close()
    g1, p, launches = results[1]
    assert torch.equal(g1, results[0][0])
    assert torch.equal(p, results[0][1])
    assert launches == results[0][2]
    for g1, p, launches in results[2:]:
        assert orc.max_err_norm(g1.cpu().numpy(), results[0][0].cpu().numpy()) <= 1e-5
        assert orc.max_err_norm(p.cpu().numpy(), results[0][1].cpu().numpy()) <= 1e-5
    assert results[2][2] == results[0][2]
    assert results[3][2] <= results[0][2]   # the default context adds into the gradient directly: no second kernel


def test_resnet56_loss_tracks_fp32_run(torch_cuda):
    """ResNet-56, batch 128 of N(0,1) CIFAR-shaped images, uniform labels, He init, momentum 0.9, lr 0.01/128, 200 steps
    on a repeated batch: the loss of the TF32 and of the 3xTF32 tensor-core run stays within 1 % (of the curve's largest
    value) of the CUDA-core fp32 run's, and all three decrease."""
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    steps = 200
    losses = {}
    _, _, dimg, dlab = make_batch(torch, 128, 32, 10, "r56")
    for math in ("fp32", "tf32", "3xtf32"):
        ctx = Context(0, math=math, sync=False)
        tr = ResNetTrainer(ctx, batch=128, blocks_per_stage=9, image_hw=32, classes=10)
        assert len([e for e in tr.entries if e["kind"] == "conv"]) == 57
        tr.init_params("r56")
        cur = []
        for _ in range(steps):
            tr.step(dimg, dlab, lr=0.01 / 128)
            cur.append(tr.loss())
        ctx.synchronize()
        losses[math] = cur
        tr.close()
        ctx.close()
    a = np.array(losses["fp32"])
    assert np.isfinite(a).all() and a[-1] < a[0]
    for math in ("tf32", "3xtf32"):
        b = np.array(losses[math])
        assert np.isfinite(b).all() and b[-1] < b[0]
        assert np.abs(a - b).max() / np.abs(a).max() <= 0.01, math


@pytest.mark.parametrize("math,tol", [("fp32", 2e-4), ("3xtf32", 2e-4), ("tf32", 5e-2)])
def test_small_densenet_step_matches_oracle(torch_cuda, math, tol):
    """DenseNet-BC with growth 4 and 2 layers per block on 16x16 inputs, batch 16: loss, logits, every gradient
    (fp32: 2e-4 per tensor; TF32: cosine >= 0.98 — fourteen small-batch BatchNorm layers amplify TF32 rounding)."""
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import DenseNetTrainer
    from tests.model_oracle import densenet_param_shapes, densenet_run
    growth, layers, hw, classes, batch = 4, 2, 16, 10, 16
    ctx = Context(0, math=math, sync=True)
    tr = DenseNetTrainer(ctx, batch=batch, growth=growth, layers=layers, image_hw=hw, classes=classes)
    shapes = densenet_param_shapes(growth, layers, hw, classes)
    assert [e["kind"] for e in tr.entries] == [k for k, _ in shapes]
    assert [e["size"] for e in tr.entries] == [int(np.prod(s)) for _, s in shapes]
    host = tr.init_params("dn")
    for i, e in enumerate(tr.entries):
        if e["kind"].startswith("bn"):
            host[e["offset"]:e["offset"] + e["size"]] += 0.1 * orc.uniform_pm1((e["size"],), "dn", "bnp", i)
    tr.set_params(host)
    P = [host[e["offset"]:e["offset"] + e["size"]].reshape(s) for e, (_, s) in zip(tr.entries, shapes)]
    images, onehot, dimg, dlab = make_batch(torch, batch, hw, classes, "dn")
    tr.forward(dimg, dlab)
    tr.backward()
    ctx.synchronize()
    loss_ref, G_ref, logits_ref = densenet_run(P, images, onehot, growth, layers)
    assert abs(tr.loss() - loss_ref) <= tol * max(1.0, abs(loss_ref))
    assert orc.max_err_norm(tr.tensor(-1, (batch, classes)).cpu().numpy(), logits_ref) <= tol
    g = tr.grads.cpu().numpy()
    for e, gr in zip(tr.entries, G_ref):
        got = g[e["offset"]:e["offset"] + e["size"]].astype(np.float64)
        want = np.asarray(gr, dtype=np.float64).ravel()
        if math != "tf32":
            assert orc.max_err_norm(got, want) <= tol, (e["kind"], e["dims"])
        else:
            cos = float(got @ want) / max(float(np.linalg.norm(got) * np.linalg.norm(want)), 1e-300)
            assert cos >= 0.98, (e["kind"], e["dims"], cos)
    tr.close()
    ctx.close()


def test_densenet_bc_100_forward_backward(torch_cuda):
    """Config 5: DenseNet-BC-100 (k = 12, 3 x 16 bottleneck layers, compression 0.5), batch 64 of 3x32x32 N(0,1)
    images: forward + backward run, the loss is finite and the TF32 loss agrees with the CUDA-core fp32 run."""
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import DenseNetTrainer
    _, _, dimg, dlab = make_batch(torch, 64, 32, 10, "dn100")
    losses = {}
    for math in ("fp32", "tf32"):
        ctx = Context(0, math=math, sync=False)
        tr = DenseNetTrainer(ctx, batch=64, growth=12, layers=16, image_hw=32, classes=10)
        assert len([e for e in tr.entries if e["kind"] == "conv"]) == 99
        tr.init_params("dn100")
        tr.forward(dimg, dlab)
        tr.backward()
        losses[math] = tr.loss()
        assert torch.isfinite(tr.grads).all()
        tr.close()
        ctx.close()
    assert np.isfinite(losses["fp32"]) and abs(losses["fp32"] - losses["tf32"]) <= 0.01 * abs(losses["fp32"])
