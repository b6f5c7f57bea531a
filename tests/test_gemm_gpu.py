"""GEMM parity on a B200: the tcgen05 kernels (through the C ABI) against the fp64 CPU oracle.

Tolerances are the ones the specification states for `max|c - c64| / max|c64|`:
  TF32 mode <= 2e-3, 3xTF32 mode <= 1e-5; the CUDA-core fp32 path is held to 2e-6.
"""
import ctypes

import numpy as np
import pytest

from oracle import oracle as orc

pytestmark = pytest.mark.gpu

TOL = {"tf32": 2e-3, "3xtf32": 1e-5, "fp32": 2e-6}
FORMS = {"NN": (False, False), "NT": (False, True), "TN": (True, False)}


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


def make_operands(M, N, K, form, key):
    tA, tB = FORMS[form]
    A = orc.uniform_pm1((K, M) if tA else (M, K), key, "A")
    B = orc.uniform_pm1((N, K) if tB else (K, N), key, "B")
    return A, B


def run_gemm(torch, ctx, A, B, M, N, form, C0=None, accumulate=False):
    tA, tB = FORMS[form]
    dA, dB = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    dC = torch.full((M, N), float("nan"), device="cuda") if C0 is None else torch.from_numpy(C0).cuda()
    ctx.gemm(dA, dB, dC, transA=tA, transB=tB, accumulate=accumulate)
    return dC.cpu().numpy()


@pytest.mark.parametrize("math", ["tf32", "3xtf32"])
def test_config1_512_cubed_nn_seed0(torch_cuda, ctxs, math):
    """fp32 GEMM C = A B, M = N = K = 512, U(-1,1): full comparison with the fp64 triple loop."""
    A, B = make_operands(512, 512, 512, "NN", 0)
    got = run_gemm(torch_cuda, ctxs[math], A, B, 512, 512, "NN")
    assert ctxs[math].last_kernel == ("umma_tf32" if math == "tf32" else "umma_3xtf32")
    assert orc.max_err_norm(got, orc.gemm_f64(A, B)) <= TOL[math]


@pytest.mark.parametrize("math", ["tf32", "3xtf32"])
@pytest.mark.parametrize("form", list(FORMS))
@pytest.mark.parametrize("n", [1024, 2048, 4096, 8192])
def test_config2_sweep(torch_cuda, ctxs, n, form, math):
    """Square sweep in NN / NT / TN form. n = 1024 is checked in full, larger sizes on 48 seeded rows and 48
    seeded columns of the product (each still a full-length fp64 dot product)."""
    tA, tB = FORMS[form]
    A, B = make_operands(n, n, n, form, ("sweep", n, form))
    got = run_gemm(torch_cuda, ctxs[math], A, B, n, n, form)
    assert np.isfinite(got).all()
    if n <= 1024:
        ref = orc.gemm_f64(A, B, tA, tB)
        assert orc.max_err_norm(got, ref) <= TOL[math]
        return
    rng = orc.rng_for("sample", n, form)
    rows = np.sort(rng.choice(n, 48, replace=False))
    cols = np.sort(rng.choice(n, 48, replace=False))
    Asub = np.ascontiguousarray(A[:, rows] if tA else A[rows])
    Bsub = np.ascontiguousarray(B[cols] if tB else B[:, cols])
    ref_rows = orc.gemm_f64(Asub, B, tA, tB)
    ref_cols = orc.gemm_f64(A, Bsub, tA, tB)
    scale = max(np.abs(ref_rows).max(), np.abs(ref_cols).max())
    err = max(np.abs(got[rows] - ref_rows).max(), np.abs(got[:, cols] - ref_cols).max())
    assert err / scale <= TOL[math]


@pytest.mark.parametrize("math", ["tf32", "3xtf32"])
@pytest.mark.parametrize("form", ["NN", "NT"])
def test_config2_skinny_dense_layer_shape(torch_cuda, ctxs, form, math):
    """M = 128, N = 10, K = 4096. In NN form B's rows are 40 bytes apart, which TMA cannot address, so the call is
    served by the CUDA-core fp32 kernel; NT is served by the tensor-core kernel with split K."""
    A, B = make_operands(128, 10, 4096, form, ("skinny", form))
    got = run_gemm(torch_cuda, ctxs[math], A, B, 128, 10, form)
    kern = ctxs[math].last_kernel
    tol = TOL["fp32"] if kern == "simt_fp32" else TOL[math]
    assert orc.max_err_norm(got, orc.gemm_f64(A, B, *FORMS[form])) <= tol
    if form == "NN":
        assert kern == "simt_fp32"


@pytest.mark.parametrize("math", ["tf32", "3xtf32", "fp32"])
@pytest.mark.parametrize("form", list(FORMS))
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (5, 3, 2), (127, 129, 31), (128, 256, 32), (200, 100, 72), (300, 260, 100),
                                   (257, 513, 1000), (64, 1000, 8)])
def test_ragged_shapes(torch_cuda, ctxs, M, N, K, form, math):
    A, B = make_operands(M, N, K, form, ("ragged", M, N, K, form))
    got = run_gemm(torch_cuda, ctxs[math], A, B, M, N, form)
    kern = ctxs[math].last_kernel
    tol = TOL["fp32"] if kern == "simt_fp32" else TOL[math]
    assert orc.max_err_norm(got, orc.gemm_f64(A, B, *FORMS[form])) <= tol


@pytest.mark.parametrize("math", ["tf32", "3xtf32", "fp32"])
def test_accumulate_and_batched_shared_a(torch_cuda, ctxs, math):
    """accumulate adds onto C (sgemmNTA's C += ..., seblas/operations/cuGEMM.cu:1701); a 2-D A is shared by every
    batch of B as in sgemm's loop over B.n (seblas/operations/cuGEMM.cu:79)."""
    torch = torch_cuda
    M, N, K, nb = 96, 80, 72, 3
    A = orc.uniform_pm1((M, K), "acc", "A")
    B = orc.uniform_pm1((nb, K, N), "acc", "B")
    C0 = orc.uniform_pm1((nb, M, N), "acc", "C")
    dC = torch.from_numpy(C0).cuda()
    ctxs[math].gemm(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), dC, accumulate=True)
    ref = np.stack([orc.gemm_f64(A, B[b]) for b in range(nb)]) + C0
    assert orc.max_err_norm(dC.cpu().numpy(), ref) <= TOL[math]
    dC2 = torch.full((nb, M, N), float("nan"), device="cuda")
    ctxs[math].gemm(torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), dC2)
    assert orc.max_err_norm(dC2.cpu().numpy(), ref - C0) <= TOL[math]


def test_leading_dimensions_and_guard_bands(torch_cuda, ctxs):
    """Operands that are windows of larger buffers (ld > row length); canaries around C stay untouched."""
    torch = torch_cuda
    M, N, K = 150, 70, 90
    bufA = torch.from_numpy(orc.uniform_pm1((M, K + 14), "ld", "A")).cuda()
    bufB = torch.from_numpy(orc.uniform_pm1((K, N + 10), "ld", "B")).cuda()
    bufC = torch.full((M + 2, N + 6), 123.0, device="cuda")
    A, B, Cv = bufA[:, 4:4 + K], bufB[:, 4:4 + N], bufC[1:1 + M, 3:3 + N]  # 16-byte aligned windows
    for math in TOL:
        bufC.fill_(123.0)
        ctxs[math].gemm(A, B, Cv)
        ref = orc.gemm_f64(A.cpu().numpy(), B.cpu().numpy())
        assert orc.max_err_norm(Cv.cpu().numpy(), ref) <= TOL[math]
        full = bufC.cpu().numpy().copy()
        full[1:1 + M, 3:3 + N] = 123.0
        assert (full == 123.0).all(), "writes outside the C window"


def test_tf32_identity_is_bit_exact_truncation(torch_cuda, ctxs):
    """A * I returns A with the 13 low mantissa bits cleared in TF32 mode (the tensor core reads the 19 high bits
    of each fp32 word) and A itself to ~2^-21 in 3xTF32 mode. Size-independent, run at n = 4096."""
    torch = torch_cuda
    n = 4096
    A = torch.from_numpy(orc.uniform_pm1((n, n), "ident")).cuda()
    eye = torch.eye(n, device="cuda")
    out = torch.empty_like(A)
    ctxs["tf32"].gemm(A, eye, out)
    trunc = (A.view(torch.int32) & -8192).view(torch.float32)
    assert torch.equal(out, trunc)
    ctxs["3xtf32"].gemm(A, eye, out)
    assert ((out - A).abs().max() / A.abs().max()).item() < 1e-6


def test_deterministic_mode_is_bitwise_reproducible(torch_cuda):
    torch = torch_cuda
    from crusaderbackend_b200.api import Context
    ctx = Context(0, math="tf32", sync=True)
    ctx.set_deterministic(True)
    A = torch.from_numpy(orc.uniform_pm1((128, 4096), "det", "A")).cuda()
    B = torch.from_numpy(orc.uniform_pm1((16, 4096), "det", "B")).cuda()
    outs = []
    for _ in range(3):
        Cc = torch.empty(128, 16, device="cuda")
        ctx.gemm(A, B, Cc, transB=True)
        outs.append(Cc.clone())
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    ctx.close()


def test_empty_and_degenerate_extents(torch_cuda, ctxs):
    torch = torch_cuda
    ctx = ctxs["tf32"]
    lib, h = ctx.lib, ctx.h
    buf = torch.full((16,), 5.0, device="cuda")
    p = ctypes.c_void_p(buf.data_ptr())
    # M == 0 / N == 0 / batch == 0: nothing to do, nothing written
    assert lib.cb_gemm(h, 0, 0, 0, 4, 4, p, 4, p, 4, p, 4, 1, 0, 0, 0, 0) == 0
    assert lib.cb_gemm(h, 0, 0, 4, 0, 4, p, 4, p, 4, p, 4, 1, 0, 0, 0, 0) == 0
    assert lib.cb_gemm(h, 0, 0, 4, 4, 4, p, 4, p, 4, p, 4, 0, 0, 0, 0, 0) == 0
    assert (buf == 5.0).all()
    # K == 0: C = 0, or C unchanged when accumulating
    Cc = torch.full((4, 4), 9.0, device="cuda")
    pc = ctypes.c_void_p(Cc.data_ptr())
    assert lib.cb_gemm(h, 0, 0, 4, 4, 0, p, 4, p, 4, pc, 4, 1, 0, 0, 0, 1) == 0
    assert (Cc == 9.0).all()
    assert lib.cb_gemm(h, 0, 0, 4, 4, 0, p, 4, p, 4, pc, 4, 1, 0, 0, 0, 0) == 0
    ctx.synchronize()
    assert (Cc == 0.0).all()


def test_argument_errors_are_reported(torch_cuda, ctxs):
    from crusaderbackend_b200._lib import CB_EINVAL
    torch = torch_cuda
    ctx = ctxs["tf32"]
    lib, h = ctx.lib, ctx.h
    buf = torch.zeros(64, device="cuda")
    p = ctypes.c_void_p(buf.data_ptr())
    assert lib.cb_gemm(h, 0, 0, 4, 4, 4, None, 4, p, 4, p, 4, 1, 0, 0, 0, 0) == CB_EINVAL
    assert lib.cb_gemm(h, 0, 0, 4, 4, 4, p, 3, p, 4, p, 4, 1, 0, 0, 0, 0) == CB_EINVAL  # lda < K
    assert lib.cb_gemm(h, 0, 0, -1, 4, 4, p, 4, p, 4, p, 4, 1, 0, 0, 0, 0) == CB_EINVAL
    assert b"cb_gemm" in lib.cb_last_error(h)


def test_misaligned_operands_take_the_cuda_core_path(torch_cuda, ctxs):
    """A pointer that is not 16-byte aligned cannot be a TMA base: the call is served by the fp32 kernel."""
    torch = torch_cuda
    M, N, K = 64, 64, 64
    buf = torch.from_numpy(orc.uniform_pm1((M * K + 1,), "mis")).cuda()
    A = buf[1:].view(M, K)
    B = torch.from_numpy(orc.uniform_pm1((K, N), "mis", "B")).cuda()
    Cc = torch.empty(M, N, device="cuda")
    ctxs["tf32"].gemm(A, B, Cc)
    assert ctxs["tf32"].last_kernel == "simt_fp32"
    assert orc.max_err_norm(Cc.cpu().numpy(), orc.gemm_f64(A.cpu().numpy(), B.cpu().numpy())) <= TOL["fp32"]


def test_golden_reference_gemm_cases(torch_cuda, ctxs, golden):
    """Same seeded inputs as the recorded runs of the reference's sgemm / sgemmTN / sgemmNT kernels."""
    from tests.golden.make_golden import CASES, inputs
    torch = torch_cuda
    for name, c in CASES.items():
        if c["op"] != "gemm" or name == "gemm_nt_f4_m256":
            continue
        x = inputs(name, c)
        A, B = torch.from_numpy(x["A"]).cuda(), torch.from_numpy(x["B"]).cuda()
        out = torch.empty((c["batch"], c["M"], c["N"]), device="cuda")
        if c["form"] == 2:
            ctxs["3xtf32"].sgemmNT(A, B, out[0])
        elif c["form"] == 1:
            ctxs["3xtf32"].sgemmTN(A, B, out)
        else:
            ctxs["3xtf32"].sgemm(A, B, out)
        assert orc.max_err_norm(out.cpu().numpy(), golden[name + "/C"]) <= 2e-5, name


@pytest.mark.parametrize("math", ["tf32", "3xtf32", "fp32"])
@pytest.mark.parametrize("n,M,N,K", [(3, 96, 80, 72), (2, 50, 37, 29), (128, 10, 64, 64), (16, 64, 576, 40), (5, 130, 300, 100)])
def test_sgemm_nta_batch_folded_into_k(torch_cuda, ctxs, math, n, M, N, K):
    """seblas::sgemmNTA (seblas/operations/cuGEMM.cu:1701): C += sum over n of A[n] B[n]^T, against the fp64 oracle;
    on the tensor-core paths the whole batch is ONE launch (the k-blocks walk the samples; K need not be a multiple of
    the 32-element k-block: the tail of every sample is zero-filled)."""
    torch = torch_cuda
    A = orc.uniform_pm1((n, M, K), "nta", n, M, "A")
    B = orc.uniform_pm1((n, N, K), "nta", n, N, "B")
    C0 = orc.uniform_pm1((M, N), "nta", n, "C0")
    want = C0.astype(np.float64)
    for b in range(n):
        want = want + orc.gemm_f64(A[b], B[b], False, True)
    ctx = ctxs[math]
    dA, dB, dC = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), torch.from_numpy(C0).cuda()
    l0 = ctx.launches
    ctx.sgemmNTA(dA, dB, dC)
    launches = ctx.launches - l0
    ctx.synchronize()
    assert orc.max_err_norm(dC.cpu().numpy(), want) <= TOL[math]
    if math != "fp32" and K % 4 == 0:
        assert ctx.last_kernel.startswith("umma") and launches <= 2   # the GEMM, plus a clear only for split-K outputs


def test_golden_reference_sgemm_nta(torch_cuda, ctxs, golden):
    """Same seeded inputs as the recorded runs of the reference's sgemmNTA kernels."""
    from tests.golden.make_golden import CASES, inputs
    torch = torch_cuda
    for name, c in CASES.items():
        if c["op"] != "gemm_nta":
            continue
        x = inputs(name, c)
        A, B, Cc = (torch.from_numpy(x[k]).cuda() for k in ("A", "B", "C0"))
        ctxs["3xtf32"].sgemmNTA(A, B, Cc)
        assert orc.max_err_norm(Cc.cpu().numpy(), golden[name + "/C"]) <= 2e-5, name
