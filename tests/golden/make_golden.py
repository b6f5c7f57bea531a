"""Records golden vectors from the REFERENCE's own seblas kernels (oracle/_ref/libseblas_ref.so, built by
oracle/build_ref.sh from the reference tree and run on a B200).

Usage (on a GPU box):  python tests/golden/make_golden.py <out_dir>
Writes <out_dir>/ref_seblas_golden.npz; the committed copy lives beside this script. Inputs are not stored:
they are regenerated from the seeded generators in oracle/oracle.py under the key recorded in CASES, so the
file only holds the reference's outputs (a few hundred KB).
"""
from __future__ import annotations

import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), "..", ".."))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

# name -> parameters. Shapes are small so the fp64 oracle replays them in milliseconds on CPU.
CASES = {
    "gemm_nn_f4": dict(op="gemm", form=0, M=96, N=80, K=72, batch=2),
    "gemm_nn_scalar": dict(op="gemm", form=0, M=50, N=37, K=29, batch=1),
    "gemm_tn_f4": dict(op="gemm", form=1, M=96, N=80, K=72, batch=2),
    "gemm_tn_scalar": dict(op="gemm", form=1, M=50, N=37, K=29, batch=1),
    "gemm_nt_f4_m96": dict(op="gemm", form=2, M=96, N=80, K=72, batch=1),
    "gemm_nt_scalar_m150": dict(op="gemm", form=2, M=150, N=37, K=29, batch=1),
    "gemm_nt_f4_m256": dict(op="gemm", form=2, M=256, N=64, K=64, batch=1),  # float4 NT kernel, M > 128
    # sgemmNTA: C += sum_n A[n] B[n]^T; M <= 128 (its float4 kernel shares the NT kernel's row-block defect)
    "gemm_nta_f4": dict(op="gemm_nta", M=96, N=80, K=72, batch=3),
    "gemm_nta_scalar": dict(op="gemm_nta", M=50, N=37, K=29, batch=2),
    "conv_s1_bias": dict(op="conv", N=2, IC=5, IH=9, IW=9, OC=7, F=3, s=1, p=1, bias=True),
    "conv_s2": dict(op="conv", N=2, IC=5, IH=10, IW=10, OC=7, F=3, s=2, p=1, bias=False),
    "conv_1x1": dict(op="conv", N=3, IC=6, IH=8, IW=8, OC=4, F=1, s=1, p=0, bias=False),
    "conv_wide": dict(op="conv", N=2, IC=16, IH=32, IW=32, OC=16, F=3, s=1, p=1, bias=False),
    "linear": dict(op="linear", batch=12, IN=20, OUT=10),
    "linear_scalar": dict(op="linear", batch=7, IN=13, OUT=5),
    "bn": dict(op="bn", N=8, C=3, H=5, W=5),
    "eltwise": dict(op="eltwise", n=1000),
    "pool": dict(op="pool", N=2, C=3, H=8, W=8),
    "softmax": dict(op="softmax", rows=6, step=10),
    "momentum": dict(op="momentum", n=1001, lr=0.01, beta=0.9, l2=1e-4),
}


def inputs(name: str, c: dict) -> dict:
    """The seeded inputs of a case (shared by this recorder and the tests that replay the oracle)."""
    if c["op"] == "gemm":
        M, N, K, b = c["M"], c["N"], c["K"], c["batch"]
        A = orc.uniform_pm1((K, M) if c["form"] == 1 else (M, K), name, "A")
        B = orc.uniform_pm1((N, K) if c["form"] == 2 else (b, K, N), name, "B")
        return dict(A=A, B=B)
    if c["op"] == "gemm_nta":
        M, N, K, b = c["M"], c["N"], c["K"], c["batch"]
        return dict(A=orc.uniform_pm1((b, M, K), name, "A"), B=orc.uniform_pm1((b, N, K), name, "B"),
                    C0=orc.uniform_pm1((M, N), name, "C0"))
    if c["op"] == "conv":
        OH, OW = orc.conv_out_hw(c["IH"], c["IW"], c["F"], c["F"], c["s"], c["s"], c["p"], c["p"])
        return dict(W=orc.he_normal_filter(c["OC"], c["IC"], c["F"], c["F"], name),
                    X=orc.normal((c["N"], c["IC"], c["IH"], c["IW"]), name, "X"),
                    dY=orc.normal((c["N"], c["OC"], OH, OW), name, "dY"),
                    bias=orc.normal((c["OC"],), name, "bias") if c["bias"] else None,
                    dW0=orc.normal((c["OC"], c["IC"], c["F"], c["F"]), name, "dW0"))
    if c["op"] == "linear":
        return dict(X=orc.normal((c["batch"], c["IN"]), name, "X"), W=orc.normal((c["OUT"], c["IN"]), name, "W"),
                    b=orc.normal((c["OUT"],), name, "b"), dY=orc.normal((c["batch"], c["OUT"]), name, "dY"),
                    dW0=orc.normal((c["OUT"], c["IN"]), name, "dW0"))
    if c["op"] == "bn":
        shp = (c["N"], c["C"], c["H"], c["W"])
        return dict(X=orc.normal(shp, name, "X") * 2 + 0.5, dY=orc.normal(shp, name, "dY"),
                    gamma=orc.uniform_pm1(shp[1:], name, "g") + 1.5, beta=orc.uniform_pm1(shp[1:], name, "b"))
    if c["op"] == "eltwise":
        return dict(X=orc.normal((c["n"],), name, "X"), dY=orc.normal((c["n"],), name, "dY"))
    if c["op"] == "pool":
        shp = (c["N"], c["C"], c["H"], c["W"])
        return dict(X=orc.normal(shp, name, "X"), dYp=orc.normal((c["N"], c["C"], c["H"] // 2, c["W"] // 2), name, "dYp"),
                    dYg=orc.normal((c["N"], c["C"]), name, "dYg"))
    if c["op"] == "softmax":
        return dict(X=orc.normal((c["rows"], c["step"]), name, "X") * 3)
    if c["op"] == "momentum":
        return dict(w=orc.normal((c["n"],), name, "w"), g=orc.normal((c["n"],), name, "g"),
                    m=orc.normal((c["n"],), name, "m"))
    raise KeyError(c["op"])


def main(out_dir: str) -> None:
    import torch
    lib = C.CDLL(os.path.join(ROOT, "oracle", "_ref", "libseblas_ref.so"))
    dev = "cuda:0"
    out = {}

    def d(a):
        return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(dev)

    def p(t):
        return C.c_void_p(0 if t is None else t.data_ptr())

    def ok(rc, what):
        if rc != 0:
            raise RuntimeError(f"reference call failed: {what} rc={rc}")

    for name, c in CASES.items():
        x = inputs(name, c)
        if c["op"] == "gemm":
            A, B = d(x["A"]), d(x["B"])
            Cc = torch.zeros((c["batch"], c["M"], c["N"]), device=dev)
            ok(lib.ref_gemm(c["form"], p(A), p(B), p(Cc), c["M"], c["N"], c["K"], c["batch"]), name)
            out[name + "/C"] = Cc.cpu().numpy()
        elif c["op"] == "gemm_nta":
            A, B, Cc = d(x["A"]), d(x["B"]), d(x["C0"])
            ok(lib.ref_gemm_nta(p(A), p(B), p(Cc), c["M"], c["N"], c["K"], c["batch"]), name)
            out[name + "/C"] = Cc.cpu().numpy()
        elif c["op"] == "conv":
            W, X, dY, bias = d(x["W"]), d(x["X"]), d(x["dY"]), d(x["bias"])
            geo = (c["N"], c["IC"], c["IH"], c["IW"], c["OC"], c["F"], c["F"], c["s"], c["s"], c["p"], c["p"])
            Y = torch.zeros_like(dY)
            ok(lib.ref_conv(p(W), p(X), p(Y), p(bias), *geo), name)
            dX = torch.zeros_like(X)
            ok(lib.ref_conv_derive(p(W), p(dY), p(dX), *geo), name)
            dW = d(x["dW0"])
            ok(lib.ref_conv_error(p(dY), p(X), p(dW), *geo), name)
            out[name + "/Y"], out[name + "/dX"], out[name + "/dW"] = Y.cpu().numpy(), dX.cpu().numpy(), dW.cpu().numpy()
        elif c["op"] == "linear":
            X, W, b, dY, dW = d(x["X"]), d(x["W"]), d(x["b"]), d(x["dY"]), d(x["dW0"])
            Y = torch.zeros((c["batch"], c["OUT"]), device=dev)
            ok(lib.ref_linear(p(X), p(W), p(b), p(Y), c["batch"], c["IN"], c["OUT"]), name)
            dX = torch.zeros_like(X)
            ok(lib.ref_linear_xgrad(p(dY), p(W), p(dX), c["batch"], c["IN"], c["OUT"]), name)
            dB = torch.zeros(c["OUT"], device=dev)
            ok(lib.ref_linear_paramgrad(p(dY), p(X), p(dW), p(dB), c["batch"], c["IN"], c["OUT"]), name)
            out[name + "/Y"], out[name + "/dX"], out[name + "/dW"], out[name + "/dB_racy"] = (
                Y.cpu().numpy(), dX.cpu().numpy(), dW.cpu().numpy(), dB.cpu().numpy())
        elif c["op"] == "bn":
            X, dY, g, b = d(x["X"]), d(x["dY"]), d(x["gamma"]), d(x["beta"])
            dims = (c["N"], c["C"], c["H"], c["W"])
            Y, xh, dX = torch.zeros_like(X), torch.zeros_like(X), torch.zeros_like(X)
            mean, var, dg, db = (torch.zeros_like(g) for _ in range(4))
            ok(lib.ref_batchnorm(p(X), p(b), p(g), p(mean), p(var), p(Y), p(xh), *dims), name)
            ok(lib.ref_batchnorm_grad(p(dY), p(g), p(X), p(dX), *dims), name)
            ok(lib.ref_batchnorm_paramgrads(p(dY), p(xh), p(dg), p(db), *dims), name)
            for k, v in dict(Y=Y, xhat=xh, mean=mean, var=var, dX=dX, dgamma=dg, dbeta=db).items():
                out[f"{name}/{k}"] = v.cpu().numpy()
        elif c["op"] == "eltwise":
            X, dY = d(x["X"]), d(x["dY"])
            Y, dX = torch.zeros_like(X), torch.zeros_like(X)
            ok(lib.ref_relu(p(X), p(Y), c["n"]), name)
            ok(lib.ref_relu_grad(p(X), p(dY), p(dX), c["n"]), name)
            out[name + "/Y"], out[name + "/dX"] = Y.cpu().numpy(), dX.cpu().numpy()
        elif c["op"] == "pool":
            X, dYp, dYg = d(x["X"]), d(x["dYp"]), d(x["dYg"])
            dims = (c["N"], c["C"], c["H"], c["W"])
            Yp, Yg = torch.zeros_like(dYp), torch.zeros_like(dYg)
            dXp, dXg = torch.zeros_like(X), torch.zeros_like(X)
            ok(lib.ref_avgpool(p(X), p(Yp), *dims, 2), name)
            ok(lib.ref_avgpool_back(p(dXp), p(dYp), *dims, 2), name)
            ok(lib.ref_global_avgpool(p(X), p(Yg), *dims), name)
            ok(lib.ref_global_avgpool_back(p(dXg), p(dYg), *dims), name)
            for k, v in dict(Yp=Yp, dXp=dXp, Yg=Yg, dXg=dXg).items():
                out[f"{name}/{k}"] = v.cpu().numpy()
        elif c["op"] == "softmax":
            X = d(x["X"])
            Y = torch.zeros_like(X)
            ok(lib.ref_softmax(p(X), p(Y), c["rows"], c["step"]), name)
            out[name + "/Y"] = Y.cpu().numpy()
        elif c["op"] == "momentum":
            w, g, m = d(x["w"]), d(x["g"]), d(x["m"])
            ok(lib.ref_scale(p(w), c["n"], C.c_float(1.0 - c["l2"])), name)
            ok(lib.ref_momentum(p(w), p(g), p(m), c["n"], C.c_float(c["lr"]), C.c_float(c["beta"])), name)
            out[name + "/w"], out[name + "/g"], out[name + "/m"] = w.cpu().numpy(), g.cpu().numpy(), m.cpu().numpy()
        torch.cuda.synchronize()
        print("recorded", name, flush=True)
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "ref_seblas_golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.dirname(os.path.abspath(__file__)))
