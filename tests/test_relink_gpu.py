"""The reference's own operand layer, relinked onto this library, against the training executor and the CPU oracle.

oracle/build_relink.sh compiles every seann source of the reference (operands, optimizers, Sequential) from the
reference tree against the header shim in crusaderbackend_b200/compat/ and links them with
tests/cpp/relink_driver.cu; the binary (oracle/_ref/relink_driver) builds a ResNet out of the reference's operand
classes and runs the reference's Sequential::forward / backward / learn. These tests check that
  * its losses, gradients and updated parameters equal the training executor's on the same seeded inputs
    (the executor set to the reference's BatchNorm gradient order, seann/operands/seblas/BatchNorm.cu:24) and the fp64
    oracle's,
  * over 200 steps of ResNet-56 at batch 128 the executor's TF32 loss stays within 1 % of the relinked reference graph's,
  * the reference's Sequential::train loop runs on the synthetic Dataset stand-in.
"""
import os
import subprocess
import tempfile

import numpy as np
import pytest

from oracle import oracle as orc
from tests.resnet_oracle import ResNetOracle

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
DRIVER = os.path.join(ROOT, "oracle", "_ref", "relink_driver")


def run_driver(*args, cwd=None, timeout=900):
    assert os.path.exists(DRIVER), "oracle/_ref/relink_driver is built by __graft_entry__.build() where the reference tree is mounted"
    env = dict(os.environ, CRUSADER_QUIET="1")
    r = subprocess.run([DRIVER, *map(str, args)], capture_output=True, text=True, timeout=timeout, cwd=cwd, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


def make_inputs(batch, hw, classes, key):
    images = orc.normal((batch, 3, hw, hw), key, "img")
    lab = orc.rng_for(key, "lab").integers(0, classes, batch)
    onehot = np.zeros((batch, classes), dtype=np.float32)
    onehot[np.arange(batch), lab] = 1
    return images, onehot


def relink_train(tr, host, images, onehot, blocks, steps, math, lr):
    """Runs the relinked reference graph; returns (losses, final params, gradients of step 1) in the executor's layout."""
    batch, hw, classes = images.shape[0], images.shape[2], onehot.shape[1]
    with tempfile.TemporaryDirectory() as tmp:
        fin, fout = os.path.join(tmp, "in.bin"), os.path.join(tmp, "out.bin")
        np.concatenate([host.astype(np.float32), images.ravel(), onehot.ravel()]).tofile(fin)
        run_driver("train", blocks, batch, hw, classes, steps, math, repr(float(lr)), fin, fout)
        out = np.fromfile(fout, dtype=np.float32)
    n = tr.n_params
    assert out.size == steps + 2 * n
    return out[:steps], out[steps:steps + n], out[steps + n:]


def executor_train(torch, tr, host, images, onehot, steps, lr):
    tr.set_params(host)
    dimg, dlab = torch.from_numpy(images).cuda(), torch.from_numpy(onehot).cuda()
    losses, g1 = [], None
    for s in range(steps):
        tr.forward(dimg, dlab)
        tr.backward()
        losses.append(tr.loss())
        if s == 0:
            g1 = tr.grads.cpu().numpy().copy()
        tr.update(lr, 0.9, 1e-4)
    tr.ctx.synchronize()
    return np.array(losses), tr.params.cpu().numpy(), g1


@pytest.mark.parametrize("math,tol", [("fp32", 2e-4), ("3xtf32", 2e-4), ("tf32", 5e-2)])
def test_relinked_reference_resnet8_matches_executor_and_oracle(math, tol):
    """ResNet-8, batch 8, three steps. fp32 and 3xTF32: every tensor within 2e-4 of the executor and (step-1 loss and
    gradients) of the fp64 oracle; TF32: loss and parameters within 5e-2 (batch-of-8 BatchNorm amplifies TF32 rounding)."""
    import torch
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    blocks, batch, hw, classes, steps, lr = 1, 8, 32, 10, 3, 0.01 / 8
    ctx = Context(0, math=math, sync=True)
    tr = ResNetTrainer(ctx, batch=batch, blocks_per_stage=blocks, image_hw=hw, classes=classes)
    tr.set_reference_bn_grad_order(True)
    host = tr.init_params("relink8")
    for i, e in enumerate(tr.entries):
        if e["kind"].startswith("bn"):
            host[e["offset"]:e["offset"] + e["size"]] += 0.1 * orc.uniform_pm1((e["size"],), "relink8", "bnp", i)
    images, onehot = make_inputs(batch, hw, classes, "relink8")
    r_loss, r_params, r_g1 = relink_train(tr, host, images, onehot, blocks, steps, math, lr)
    e_loss, e_params, e_g1 = executor_train(torch, tr, host, images, onehot, steps, lr)
    assert np.abs(r_loss - e_loss).max() <= tol * max(1.0, np.abs(e_loss).max())
    assert orc.max_err_norm(r_params, e_params) <= tol
    if math != "tf32":
        for e in tr.entries:
            sl = slice(e["offset"], e["offset"] + e["size"])
            assert orc.max_err_norm(r_g1[sl], e_g1[sl]) <= tol, (e["kind"], e["dims"])
        # the oracle, with BatchNorm's two gradients exchanged the way the reference's operand stores them
        oracle = ResNetOracle(blocks, hw, classes)
        shapes = oracle.param_shapes()
        P = [host[e["offset"]:e["offset"] + e["size"]].reshape(s) for e, (_, s) in zip(tr.entries, shapes)]
        loss_ref, G_ref, _ = oracle.run(P, images, onehot)
        assert abs(r_loss[0] - loss_ref) <= tol * max(1.0, abs(loss_ref))
        kinds = [e["kind"] for e in tr.entries]
        for i, (e, gr) in enumerate(zip(tr.entries, G_ref)):
            want = gr
            if kinds[i] == "bn_gamma":
                want = G_ref[i + 1]
            elif kinds[i] == "bn_beta":
                want = G_ref[i - 1]
            sl = slice(e["offset"], e["offset"] + e["size"])
            assert orc.max_err_norm(r_g1[sl], np.asarray(want).ravel()) <= tol, (e["kind"], e["dims"])
    tr.close()
    ctx.close()


def test_resnet56_loss_tracks_relinked_reference_over_200_steps():
    """ResNet-56, batch 128, 200 steps on a repeated seeded batch (momentum 0.9, lr 0.01/128, L2 1e-4): the loss curve of
    the executor in TF32 and in 3xTF32 stays within 1 % (of the curve's largest value) of the relinked reference
    operand graph's curve computed in 3xTF32, the shim's default mode."""
    import torch
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    blocks, batch, hw, classes, steps, lr = 9, 128, 32, 10, 200, 0.01 / 128
    images, onehot = make_inputs(batch, hw, classes, "relink56")
    curves = {}
    for math in ("tf32", "3xtf32"):
        ctx = Context(0, math=math, sync=False)
        tr = ResNetTrainer(ctx, batch=batch, blocks_per_stage=blocks, image_hw=hw, classes=classes)
        tr.set_reference_bn_grad_order(True)
        host = tr.init_params("relink56")
        if "ref" not in curves:
            curves["ref"], _, _ = relink_train(tr, host, images, onehot, blocks, steps, "3xtf32", lr)
        curves[math], _, _ = executor_train(torch, tr, host, images, onehot, steps, lr)
        tr.close()
        ctx.close()
    ref = curves["ref"]
    assert np.isfinite(ref).all() and ref[-1] < ref[0]
    for math in ("tf32", "3xtf32"):
        assert np.isfinite(curves[math]).all()
        assert np.abs(curves[math] - ref).max() <= 0.01 * np.abs(ref).max(), math


def test_reference_train_loop_runs_on_the_synthetic_dataset():
    """The reference's Sequential::train (seann/containers/Sequential.cu:107-163), compiled unchanged, drives two batches
    from the in-memory Dataset stand-in; it writes its log under the working directory, so it runs in a scratch one."""
    with tempfile.TemporaryDirectory() as tmp:
        out = run_driver("loop", 8, 32, cwd=tmp)
    assert "relink loop ok" in out
