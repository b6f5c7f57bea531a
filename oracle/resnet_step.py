"""fp32 CPU implementation of the ResNet-(6n+2) training step, composed from the OpenMP fp32 kernels of cpu_ref.c.

This is the timed CPU baseline of bench.py (`cpu_baseline` and `--impl reference`): the reference has no CPU
implementation of this path, so the arm is a port — the same operations in the same order as the reference's operand
graph (archive/Resnet56 topology with the GlobalAvgPool + Linear head; seann/containers/Sequential.cu:43-104 for the step).
Test infrastructure: the parity tests use the fp64 composition in tests/resnet_oracle.py, not this file."""
import numpy as np

from . import oracle as orc


class ResNetStepF32:
    def __init__(self, blocks, image_hw, classes, key="cpu"):
        self.blocks, self.hw, self.classes = blocks, image_hw, classes
        self.P = []
        ch, hw = 3, image_hw
        self.spec = []  # (kind, ...) in forward order

        def conv(oc, ic, f, stride, pad):
            self.P.append(orc.he_normal_filter(oc, ic, f, f, key, len(self.P)))
            return len(self.P) - 1

        def bn(c, hw_):
            self.P.append(np.ones((c, hw_, hw_), dtype=np.float32))
            self.P.append(np.zeros((c, hw_, hw_), dtype=np.float32))
            return len(self.P) - 2

        self.stem = (conv(16, 3, 3, 1, 1), bn(16, hw))
        ch = 16
        self.layers = []
        for stage in range(3):
            oc = 16 << stage
            for b in range(blocks):
                stride = 2 if (stage > 0 and b == 0) else 1
                ohw = hw // stride
                c1, b1 = conv(oc, ch, 3, stride, 1), bn(oc, ohw)
                c2, b2 = conv(oc, oc, 3, 1, 1), bn(oc, ohw)
                proj = conv(oc, ch, 1, stride, 0) if (stride != 1 or ch != oc) else None
                self.layers.append((stride, c1, b1, c2, b2, proj))
                ch, hw = oc, ohw
        self.P.append(orc.normal((classes, ch), key, "fc", std=float(np.sqrt(2.0 / ch))))
        self.P.append(np.zeros((classes,), dtype=np.float32))
        self.M = [np.zeros_like(p) for p in self.P]

    def step(self, images, onehot, lr, beta=0.9, l2=1e-4):
        P = self.P
        G = [None] * len(P)
        f32 = dict(f32=True)
        ci, bi = self.stem
        a0 = orc.conv_fwd(P[ci], images, None, (1, 1), (1, 1), **f32)
        x = orc.bn_fwd_f32(a0, P[bi + 1], P[bi], relu=True)
        tape = [(images, a0, x)]
        for (stride, c1, b1, c2, b2, proj) in self.layers:
            u = orc.conv_fwd(P[c1], x, None, (stride, stride), (1, 1), **f32)
            v = orc.bn_fwd_f32(u, P[b1 + 1], P[b1], relu=True)
            w = orc.conv_fwd(P[c2], v, None, (1, 1), (1, 1), **f32)
            sc = x if proj is None else orc.conv_fwd(P[proj], x, None, (stride, stride), (0, 0), **f32)
            y = orc.bn_fwd_f32(w, P[b2 + 1], P[b2], res=sc, relu=True)
            tape.append((x, u, v, w, y))
            x = y
        pooled = x.mean(axis=(2, 3), dtype=np.float32)
        logits = pooled @ P[-2].T + P[-1]
        z = logits - logits.max(axis=1, keepdims=True)
        e = np.exp(z)
        probs = e / (e.sum(axis=1, keepdims=True) + 1e-10)
        loss = float(-(np.log(probs + 1e-10) * onehot).sum() / images.shape[0])
        d = (probs - onehot).astype(np.float32)
        G[-2] = d.T @ pooled
        G[-1] = d.sum(axis=0)
        dx = np.repeat((d @ P[-2])[:, :, None, None] / (x.shape[2] * x.shape[3]), x.shape[2], axis=2)
        dx = np.ascontiguousarray(np.repeat(dx, x.shape[3], axis=3), dtype=np.float32)
        for (stride, c1, b1, c2, b2, proj), (xin, u, v, w, y) in zip(reversed(self.layers), reversed(tape[1:])):
            g = np.where(y > 0, dx, 0).astype(np.float32)            # ReLU after the shortcut add
            dw_, G[b2], G[b2 + 1] = orc.bn_bwd_f32(g, P[b2], w)
            G[c2] = orc.conv_wgrad(dw_, v, P[c2].shape, (1, 1), (1, 1), **f32)
            dv = orc.conv_dgrad(P[c2], dw_, v.shape, (1, 1), (1, 1), **f32)
            dv = np.where(v > 0, dv, 0).astype(np.float32)
            du, G[b1], G[b1 + 1] = orc.bn_bwd_f32(dv, P[b1], u)
            G[c1] = orc.conv_wgrad(du, xin, P[c1].shape, (stride, stride), (1, 1), **f32)
            dmain = orc.conv_dgrad(P[c1], du, xin.shape, (stride, stride), (1, 1), **f32)
            if proj is None:
                dx = dmain + g
            else:
                G[proj] = orc.conv_wgrad(g, xin, P[proj].shape, (stride, stride), (0, 0), **f32)
                dx = dmain + orc.conv_dgrad(P[proj], g, xin.shape, (stride, stride), (0, 0), **f32)
            dx = np.ascontiguousarray(dx, dtype=np.float32)
        images_, a0, x0 = tape[0]
        g = np.where(x0 > 0, dx, 0).astype(np.float32)
        da, G[bi], G[bi + 1] = orc.bn_bwd_f32(g, P[bi], a0)
        G[ci] = orc.conv_wgrad(da, images_, P[ci].shape, (1, 1), (1, 1), **f32)
        for i, p in enumerate(P):
            is_w = p.ndim in (2, 4)
            P[i], self.M[i], _ = orc.momentum_f32(p, np.asarray(G[i], dtype=np.float32).reshape(p.shape), self.M[i], lr, beta, l2, is_w)
        return loss
