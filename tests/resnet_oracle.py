"""CPU oracle of the ResNet training step, composed from the per-op fp64 oracle (oracle/cpu_ref.c).

Mirrors the topology and the flat parameter order of cbt_resnet_create (crusaderbackend_b200/csrc/trainer.cu):
stem conv-BN-ReLU, 3 stages x `blocks` residual blocks (conv-BN-ReLU-conv-BN, + identity or bare 1x1 stride-2
projection, ReLU), global average pooling, dense head, softmax cross-entropy with gradients summed over the batch.
Test infrastructure only."""
import numpy as np

from oracle import oracle as orc


def f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class ResNetOracle:
    def __init__(self, blocks, image_hw, classes):
        self.blocks, self.hw, self.classes = blocks, image_hw, classes

    def param_shapes(self):
        """[(kind, shape)] in the order the executor lays them out."""
        out = [("conv", (16, 3, 3, 3)), ("bn_gamma", (16, self.hw, self.hw)), ("bn_beta", (16, self.hw, self.hw))]
        ch, hw = 16, self.hw
        for stage in range(3):
            oc = 16 << stage
            for b in range(self.blocks):
                stride = 2 if (stage > 0 and b == 0) else 1
                ohw = (hw - 3 + 2) // stride + 1
                out += [("conv", (oc, ch, 3, 3)), ("bn_gamma", (oc, ohw, ohw)), ("bn_beta", (oc, ohw, ohw)),
                        ("conv", (oc, oc, 3, 3)), ("bn_gamma", (oc, ohw, ohw)), ("bn_beta", (oc, ohw, ohw))]
                if stride != 1 or ch != oc:
                    out.append(("conv", (oc, ch, 1, 1)))
                ch, hw = oc, ohw
        out += [("fc_weight", (self.classes, ch)), ("fc_bias", (self.classes,))]
        return out

    def run(self, P, images, labels):
        """P: list of parameter arrays in param_shapes() order. Returns (mean loss, [gradients], logits)."""
        G = [None] * len(P)
        tape = []
        idx = [0]

        def take():
            i = idx[0]
            idx[0] += 1
            return i

        def conv(x, stride, pad):
            i = take()
            y = orc.conv_fwd(P[i], f32(x), None, (stride, stride), (pad, pad))
            tape.append(("conv", i, f32(x), stride, pad))
            return f32(y)

        def bn(x):
            ig, ib = take(), take()
            y, xh, _, _ = orc.bn_fwd(f32(x), P[ib], P[ig])
            tape.append(("bn", ig, ib, f32(x), f32(xh)))
            return f32(y)

        def relu(x):
            tape.append(("relu", f32(x)))
            return f32(orc.relu(f32(x)))

        x = relu(bn(conv(images, 1, 1)))
        ch = 16
        for stage in range(3):
            oc = 16 << stage
            for b in range(self.blocks):
                stride = 2 if (stage > 0 and b == 0) else 1
                tape.append(("fork",))
                y = relu(bn(conv(x, stride, 1)))
                y = bn(conv(y, 1, 1))
                if stride != 1 or ch != oc:
                    tape.append(("swap_to_shortcut",))
                    sc = conv(x, stride, 0)
                    tape.append(("join_proj",))
                else:
                    sc = x
                    tape.append(("join_identity",))
                x = relu(f32(y.astype(np.float64) + sc))
                ch = oc
        shape_before_gap = x.shape
        pooled = f32(orc.gap(x))
        iw, ib = take(), take()
        logits = f32(orc.linear(pooled, P[iw], P[ib]))
        probs = f32(orc.softmax(logits))
        loss, dlogits = orc.cross_entropy(probs, labels)
        # ---- backward
        dW, db = orc.linear_paramgrad(f32(dlogits), pooled)
        G[iw], G[ib] = dW, db
        d = orc.linear_xgrad(f32(dlogits), P[iw])
        d = orc.gap_back(f32(d), shape_before_gap)
        stack = []  # (gradient waiting for the block input)
        for item in reversed(tape):
            k = item[0]
            if k == "relu":
                d = orc.relu_grad(item[1], f32(d))
            elif k == "bn":
                _, ig, ib_, xin, xh = item
                G[ig], G[ib_] = (g.reshape(P[ig].shape) for g in orc.bn_paramgrad(f32(d), xh))
                d = orc.bn_bwd(f32(d), P[ig], xin)
            elif k == "conv":
                _, i, xin, stride, pad = item
                G[i] = orc.conv_wgrad(f32(d), xin, P[i].shape, (stride, stride), (pad, pad))
                d = orc.conv_dgrad(P[i], f32(d), xin.shape, (stride, stride), (pad, pad))
            elif k == "join_identity":
                stack.append(np.array(d, dtype=np.float64))      # identity shortcut gets dOut; main path continues with dOut
            elif k == "join_proj":
                stack.append(np.array(d, dtype=np.float64))      # main path gradient saved; d now flows through the 1x1 conv
            elif k == "swap_to_shortcut":
                d_short = d                                       # gradient of the block input through the projection
                d = stack.pop()                                   # resume the main path with dOut
                stack.append(np.array(d_short, dtype=np.float64))
            elif k == "fork":
                d = np.array(d, dtype=np.float64) + stack.pop()   # block input: main path + shortcut
        return loss / images.shape[0], G, logits
