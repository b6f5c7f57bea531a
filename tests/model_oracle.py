"""A minimal tape over the per-op fp64 oracle (oracle/cpu_ref.c) for checking whole training steps of the executor in
crusaderbackend_b200/csrc/trainer.cu: values are rounded to fp32 between ops (as on the GPU), gradients are summed
over the batch, and a tensor consumed twice receives the sum of both gradients. Test infrastructure only."""
import numpy as np

from oracle import oracle as orc


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Tape:
    def __init__(self, params):
        self.P = params
        self.G = [None] * len(params)
        self.vals = []
        self.ops = []
        self.next_param = 0

    def _take(self):
        i = self.next_param
        self.next_param += 1
        return i

    def _new(self, v):
        self.vals.append(f32(v))
        return len(self.vals) - 1

    def input(self, v):
        return self._new(v)

    def conv(self, x, stride, pad):
        i = self._take()
        y = self._new(orc.conv_fwd(self.P[i], self.vals[x], None, (stride, stride), (pad, pad)))
        self.ops.append(("conv", x, y, i, stride, pad))
        return y

    def bn(self, x):
        ig, ib = self._take(), self._take()
        yv, xh, _, _ = orc.bn_fwd(self.vals[x], self.P[ib], self.P[ig])
        y = self._new(yv)
        self.ops.append(("bn", x, y, ig, ib, f32(xh)))
        return y

    def relu(self, x):
        y = self._new(orc.relu(self.vals[x]))
        self.ops.append(("relu", x, y))
        return y

    def add(self, a, b):
        y = self._new(self.vals[a].astype(np.float64) + self.vals[b])
        self.ops.append(("add", a, b, y))
        return y

    def concat(self, a, b):
        y = self._new(np.concatenate([self.vals[a], self.vals[b]], axis=1))
        self.ops.append(("concat", a, b, y))
        return y

    def avgpool(self, x):
        y = self._new(orc.avgpool(self.vals[x]))
        self.ops.append(("avgpool", x, y))
        return y

    def gap(self, x):
        y = self._new(orc.gap(self.vals[x]))
        self.ops.append(("gap", x, y))
        return y

    def linear(self, x):
        iw, ib = self._take(), self._take()
        xin = self.vals[x].reshape(self.vals[x].shape[0], -1)
        y = self._new(orc.linear(xin, self.P[iw], self.P[ib]))
        self.ops.append(("linear", x, y, iw, ib))
        return y

    def loss_and_backward(self, logits, labels):
        """softmax cross-entropy on `logits`; fills self.G; returns (mean loss, logits value)."""
        probs = f32(orc.softmax(self.vals[logits]))
        loss, dlog = orc.cross_entropy(probs, labels)
        D = {logits: np.asarray(dlog, dtype=np.float64)}

        def acc(t, g):
            D[t] = g if t not in D else D[t] + g

        for op in reversed(self.ops):
            k = op[0]
            if k == "linear":
                _, x, y, iw, ib = op
                xin = self.vals[x].reshape(self.vals[x].shape[0], -1)
                self.G[iw], self.G[ib] = orc.linear_paramgrad(f32(D[y]), xin)
                acc(x, orc.linear_xgrad(f32(D[y]), self.P[iw]).reshape(self.vals[x].shape))
            elif k == "gap":
                _, x, y = op
                acc(x, orc.gap_back(f32(D[y]), self.vals[x].shape))
            elif k == "avgpool":
                _, x, y = op
                acc(x, orc.avgpool_back(f32(D[y]), self.vals[x].shape))
            elif k == "relu":
                _, x, y = op
                acc(x, orc.relu_grad(self.vals[x], f32(D[y])))
            elif k == "add":
                _, a, b, y = op
                acc(a, D[y].copy())
                acc(b, D[y].copy())
            elif k == "concat":
                _, a, b, y = op
                ca = self.vals[a].shape[1]
                acc(a, D[y][:, :ca].copy())
                acc(b, D[y][:, ca:].copy())
            elif k == "bn":
                _, x, y, ig, ib, xh = op
                dg, db = orc.bn_paramgrad(f32(D[y]), xh)
                self.G[ig], self.G[ib] = dg.reshape(self.P[ig].shape), db.reshape(self.P[ib].shape)
                acc(x, orc.bn_bwd(f32(D[y]), self.P[ig], self.vals[x]))
            elif k == "conv":
                _, x, y, i, stride, pad = op
                self.G[i] = orc.conv_wgrad(f32(D[y]), self.vals[x], self.P[i].shape, (stride, stride), (pad, pad))
                if x != 0:
                    acc(x, orc.conv_dgrad(self.P[i], f32(D[y]), self.vals[x].shape, (stride, stride), (pad, pad)))
        return loss / self.vals[0].shape[0], self.vals[logits]


def densenet_param_shapes(growth, layers, hw, classes):
    out = [("conv", (2 * growth, 3, 3, 3))]
    ch = 2 * growth
    for block in range(3):
        for _ in range(layers):
            out += [("bn_gamma", (ch, hw, hw)), ("bn_beta", (ch, hw, hw)), ("conv", (4 * growth, ch, 1, 1)),
                    ("bn_gamma", (4 * growth, hw, hw)), ("bn_beta", (4 * growth, hw, hw)), ("conv", (growth, 4 * growth, 3, 3))]
            ch += growth
        if block < 2:
            out += [("bn_gamma", (ch, hw, hw)), ("bn_beta", (ch, hw, hw)), ("conv", (ch // 2, ch, 1, 1))]
            ch //= 2
            hw //= 2
    out += [("bn_gamma", (ch, hw, hw)), ("bn_beta", (ch, hw, hw)), ("fc_weight", (classes, ch)), ("fc_bias", (classes,))]
    return out


def densenet_run(P, images, labels, growth, layers):
    """Same topology as cbt_densenet_create. Returns (mean loss, gradients, logits)."""
    t = Tape(P)
    x = t.conv(t.input(images), 1, 1)
    for block in range(3):
        for _ in range(layers):
            y = t.conv(t.relu(t.bn(x)), 1, 0)
            y = t.conv(t.relu(t.bn(y)), 1, 1)
            x = t.concat(x, y)
        if block < 2:
            x = t.avgpool(t.conv(t.relu(t.bn(x)), 1, 0))
    x = t.relu(t.bn(x))
    logits = t.linear(t.gap(x))
    loss, lv = t.loss_and_backward(logits, labels)
    return loss, t.G, lv
