#!/usr/bin/env python
"""Benchmark of the dense-contraction path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--math tf32|3xtf32]

A "step" is one pass over the GEMM sweep of the specification (M=N=K in {1024,2048,4096,8192} in NN, NT and TN
form, plus the skinny dense-layer shape 128x10x4096), synthetic U(-1,1) operands from fixed seeds.

  value  whole-job TFLOP/s (algorithmic flops 2MNK of the sweep x ranks / device time, max over ranks) with the
         operands resident in HBM; every GEMM is timed with CUDA events on the launching stream and the L2 is
         flushed (a 256 MiB write, outside the timed events) before each call.
  e2e    the same sweep through the C ABI from pinned HOST buffers: the host->device copies of both operands and
         the device->host copy of the product are inside the timed region.
  --impl reference   the CPU arm: the OpenMP fp32 loops of oracle/ (a port: the reference has no CPU
         implementation of this path) on a bounded sample of the sweep, all host threads.

With N > 1 (torchrun, one rank per GPU) every rank runs the whole sweep on its own GPU: the GEMM micro-benchmarks
do not shard ("replicas only"), so scaling is weak and there is no data-path collective.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FORMS = {"NN": (False, False), "NT": (False, True), "TN": (True, False)}
SWEEP = [(n, n, n, f) for n in (1024, 2048, 4096, 8192) for f in FORMS] + [(128, 10, 4096, "NN")]
CPU_SAMPLE = [(n, n, n, f) for n in (1024, 2048) for f in FORMS] + [(4096, 4096, 4096, "NN"), (128, 10, 4096, "NN")]
WORKLOAD = ("configs[1]: fp32 GEMM sweep M=N=K in {1024,2048,4096,8192} x {NN,NT,TN} + skinny 128x10x4096, "
            "U(-1,1) seeded")


def flops(shapes):
    return sum(2.0 * m * n * k for m, n, k, _ in shapes)


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"tf32_tflops": d["bf16_tflops"] / 2.0, "hbm_gbs": d["hbm_gbs"],
                "source": "measured: MEASURED_PEAKS.json bf16 burst / 2 (no TF32 figure was measured)"}
    except Exception:
        return {"tf32_tflops": 1590.0 / 2.0, "hbm_gbs": 6650.0, "source": "fallback: 1.59 PFLOP/s bf16 / 2"}


def profiled_traffic(kernel: str):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get(kernel)
    except Exception:
        return None


class ClockSampler(threading.Thread):
    """Samples nvidia-smi clocks and throttle reasons of one GPU every 200 ms while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()

    def run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        mhz = sorted(float(s[0]) for s in self.samples if s[0].replace(".", "").isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower() == "active" for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": float(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples)}


def visible_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# ------------------------------------------------------------------------------------------ our arm
def bench_ours(args):
    import torch
    import torch.distributed as dist
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200 import seeds as orc

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ctx = Context(local, math=args.math, sync=False)

    # operands: one pair of seeded square buffers per size, shared by the three forms
    bufs = {}
    sizes = sorted({(m, n, k) for m, n, k, _ in SWEEP})
    host = {}
    for (m, n, k) in sizes:
        if m == n == k:
            a = orc.uniform_pm1((m, k), "bench", m, "A")
            b = orc.uniform_pm1((k, n), "bench", m, "B")
        else:
            a = orc.uniform_pm1((m, k), "bench", "skinnyA")
            b = orc.uniform_pm1((k, n), "bench", "skinnyB")
        host[(m, n, k)] = (torch.from_numpy(a).pin_memory(), torch.from_numpy(b).pin_memory(),
                           torch.empty((m, n), dtype=torch.float32).pin_memory())
        bufs[(m, n, k)] = (host[(m, n, k)][0].to(dev), host[(m, n, k)][1].to(dev),
                           torch.empty((m, n), device=dev, dtype=torch.float32))
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev, dtype=torch.float32)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_gemm(shape):
        m, n, k, form = shape
        A, B, Cc = bufs[(m, n, k)]
        tA, tB = FORMS[form]
        # a square buffer read as K x M (TN) or N x K (NT) is a different, equally valid problem
        ctx.gemm(A, B, Cc, transA=tA, transB=tB)

    def timed_step(record):
        for shape in SWEEP:
            flush.fill_(1.0)  # evict L2 (126 MB) outside the timed events
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            one_gemm(shape)
            e1.record()
            record.append((shape, e0, e1))

    for _ in range(args.warmup):
        timed_step([])
    barrier()
    sampler = ClockSampler(visible_gpu_index(local))
    sampler.start()
    launches0 = ctx.launches
    rec = []
    barrier()
    t_wall0 = time.perf_counter()
    for _ in range(args.steps):
        timed_step(rec)
    barrier()
    wall_ms = (time.perf_counter() - t_wall0) * 1e3 / args.steps
    launches = ctx.launches - launches0
    ctx.synchronize()
    per_shape = {}
    for shape, e0, e1 in rec:
        per_shape.setdefault(shape, []).append(e0.elapsed_time(e1))
    step_ms = sum(sum(v) / len(v) for v in per_shape.values())

    # ---- end to end from host buffers (copies inside the timed region)
    def e2e_step():
        for shape in SWEEP:
            m, n, k, form = shape
            hA, hB, hC = host[(m, n, k)]
            A, B, Cc = bufs[(m, n, k)]
            A.copy_(hA, non_blocking=True)
            B.copy_(hB, non_blocking=True)
            one_gemm(shape)
            hC.copy_(Cc, non_blocking=True)

    e2e_step()
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.steps):
        e2e_step()
    s1.record()
    barrier()
    e2e_ms = s0.elapsed_time(s1) / args.steps
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    ctx.synchronize()

    times = torch.tensor([step_ms, e2e_ms, wall_ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    step_ms_max, e2e_ms_max, wall_ms_max = times.tolist()

    h2d = sum(4 * (m * k + k * n) for m, n, k, _ in SWEEP)
    d2h = sum(4 * m * n for m, n, k, _ in SWEEP)
    peaks = measured_peaks()
    dom = (8192, 8192, 8192, "NN") if (8192, 8192, 8192, "NN") in per_shape else max(per_shape, key=lambda q: q[0] * q[1] * q[2])
    dom_ms = sum(per_shape[dom]) / len(per_shape[dom])
    dom_tflops = 2.0 * dom[0] * dom[1] * dom[2] / dom_ms / 1e9
    detail = {f"{m}x{n}x{k}_{f}": round(2.0 * m * n * k / (sum(v) / len(v)) / 1e9, 2)
              for (m, n, k, f), v in per_shape.items()}

    line = None
    if rank == 0:
        line = {
            "metric": "gemm_sweep_tflops", "value": round(flops(SWEEP) * world / step_ms_max / 1e9, 2),
            "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(step_ms_max, 4), "wall_ms_per_step": round(wall_ms_max, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32" if args.math == "tf32" else "3xtf32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "math": args.math, "parallelism": f"replicas x{world}",
                       "l2": "flushed by a 256 MiB write before every GEMM, outside the timed CUDA events"},
            "e2e": {"value": round(flops(SWEEP) * world / e2e_ms_max / 1e9, 2), "unit": "TFLOP/s",
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": round(e2e_ms_max, 3)},
            "gpu_launches": int(launches),
            "clocks": sampler.summary(),
            "roofline": {"bound": "tensor", "kernel": f"umma_gemm_kernel ({dom[0]}x{dom[1]}x{dom[2]} {dom[3]})",
                         "achieved": round(dom_tflops, 1), "peak": round(peaks["tf32_tflops"], 1),
                         "unit": "TFLOP/s", "frac": round(dom_tflops / peaks["tf32_tflops"], 4),
                         "traffic": profiled_traffic("umma_gemm_8192_nn"), "peak_source": peaks["source"],
                         "nominal_tf32_tflops": 1100.0},
            "tflops_by_shape": detail,
        }
        line["cpu_baseline"] = None if (args.no_cpu or world > 1) else cpu_baseline_leg()  # rank 0 at N = 1 only
        if not args.no_cpu and world == 1:
            try:
                line["reference_cuda"] = reference_cuda_leg()
            except Exception as exc:
                line["reference_cuda"] = {"error": str(exc)[:200]}
    extra_conv = None
    if not args.shapes or args.conv_shapes:
        only = set(args.conv_shapes.split(",")) if args.conv_shapes else None
        extra_conv = conv_section(ctx, torch, dev, flush, only)
    ctx.close()
    extra_resnet = None
    if (not args.shapes or args.resnet) and not args.no_resnet:
        try:
            extra_resnet = resnet56_section(torch, local, world, max(args.steps, 5), args.warmup)
            if world > 1:
                extra_resnet["weak_scaling_128_per_gpu"] = resnet56_section(torch, local, world, max(args.steps, 5),
                                                                            args.warmup, weak=True)
        except Exception as exc:  # keep the headline line even if the training section fails
            extra_resnet = {"error": str(exc)[:300]}
    if rank == 0:
        line["conv"] = extra_conv
        line["resnet56_train"] = extra_resnet
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------ conv shapes / ResNet-56
CONV_SHAPES = [  # (name, N, IC, H, OC, F, stride, pad): config 3 and the ResNet-56 layer shapes
    ("c3_64to64_3x3_s1_32x32", 128, 64, 32, 64, 3, 1, 1),
    ("c3_32to64_3x3_s2_32x32", 128, 32, 32, 64, 3, 2, 1),
    ("r56_16to16_3x3_s1_32x32", 128, 16, 32, 16, 3, 1, 1),
    ("r56_32to32_3x3_s1_16x16", 128, 32, 16, 32, 3, 1, 1),
    ("r56_64to64_3x3_s1_8x8", 128, 64, 8, 64, 3, 1, 1),
]


def conv_section(ctx, torch, dev, flush, only=None):
    """Forward / data-gradient / weight-gradient of the convolution shapes: per-call CUDA-event time with the L2
    flushed before each call, TFLOP/s on 2*N*OC*OH*OW*IC*FH*FW and GB/s on 4*(|X|+|W|+|Y|)."""
    out = {}
    for (name, N, IC, H, OC, F, s, p) in CONV_SHAPES:
        if only and name not in only:
            continue
        OH = (H - F + 2 * p) // s + 1
        X = torch.randn(N, IC, H, H, device=dev)
        W = torch.randn(OC, IC, F, F, device=dev) * (2.0 / (IC * F * F)) ** 0.5
        Y = torch.empty(N, OC, OH, OH, device=dev)
        dY = torch.randn(N, OC, OH, OH, device=dev)
        dX = torch.empty_like(X)
        dW = torch.zeros_like(W)
        fl = 2.0 * N * OC * OH * OH * IC * F * F
        by = 4.0 * (X.numel() + W.numel() + Y.numel())
        calls = {"fwd": lambda: ctx.conv(W, X, Y, s, s, p, p), "dgrad": lambda: ctx.convDerive(W, dY, dX, s, s, p, p),
                 "wgrad": lambda: ctx.convError(dY, X, dW, s, s, p, p)}
        for pname, fn in calls.items():
            for _ in range(2):
                fn()
            ts = []
            for _ in range(5):
                flush.fill_(1.0)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            ms = sorted(ts)[len(ts) // 2]
            out[f"{name}_{pname}"] = {"us": round(ms * 1e3, 1), "tflops": round(fl / ms / 1e9, 1),
                                      "gbs": round(by / ms / 1e6, 1), "kernel": ctx.last_kernel}
    return out


def resnet56_section(torch, local, world, steps, warmup, weak=False):
    """ResNet-56 training step (forward + backward + gradient allreduce + Momentum), global batch 128 split over the
    ranks (strong scaling, the configuration of the specification), replayed as one CUDA graph. Each timed step
    includes the host->device copy of that step's images and labels from pinned memory and ends with a device->host
    read of the loss."""
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    from crusaderbackend_b200 import dp
    from crusaderbackend_b200 import seeds as orc
    gb = 128 * world if weak else 128   # weak: 128 images per GPU; strong (the spec's configuration): 128 in total
    rank = int(os.environ.get("RANK", "0"))
    start, count = dp.shard_batch(gb, world, rank)
    ctx = Context(local, math="tf32", sync=False)
    tr = ResNetTrainer(ctx, batch=count, blocks_per_stage=9, image_hw=32, classes=10, distributed=world > 1)
    tr.init_params("bench")
    h_img = torch.from_numpy(orc.normal((gb, 3, 32, 32), "bench", "img")[start:start + count].copy()).pin_memory()
    lab = orc.rng_for("bench", "lab").integers(0, 10, gb)[start:start + count]
    onehot = torch.zeros(count, 10)
    onehot[torch.arange(count), torch.from_numpy(lab)] = 1
    h_lab = onehot.pin_memory()
    d_img = torch.empty(count, 3, 32, 32, device="cuda")
    d_lab = torch.empty(count, 10, device="cuda")
    d_img.copy_(h_img)
    d_lab.copy_(h_lab)
    lr = 0.01 / gb
    launches0 = ctx.launches
    tr.step(d_img, d_lab, lr)
    launches = ctx.launches - launches0
    graph = tr.capture_step(d_img, d_lab, lr, warmup=2)
    loss_dev = torch.empty(1, device="cuda")
    h_loss = torch.empty(1).pin_memory()

    def one_step():
        d_img.copy_(h_img, non_blocking=True)
        d_lab.copy_(h_lab, non_blocking=True)
        graph.replay()
        tr.lib.cbt_copy_loss(tr.h, loss_dev.data_ptr())
        h_loss.copy_(loss_dev, non_blocking=True)

    for _ in range(max(3, warmup)):
        one_step()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        one_step()
    e1.record()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    if world > 1:
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    ms = float(t.item())
    res = {"images_per_s": round(gb / ms * 1e3, 1), "ms_per_step": round(ms, 3), "global_batch": gb,
           "per_gpu_batch": count, "scaling": "weak" if weak else "strong", "math": "tf32", "kernels_per_step": int(launches),
           "cuda_graph": True, "loss_mean_last": round(float(h_loss.item()) / count, 5),
           "h2d_bytes_per_step": int(h_img.numel() * 4 + h_lab.numel() * 4), "d2h_bytes_per_step": 4,
           "flops_per_step": 96.5e9 * gb / 128,
           "note": "forward+backward+allreduce+Momentum; BatchNorm statistics are per GPU shard"}
    tr.close()
    ctx.close()
    return res


# ------------------------------------------------------------------------------------------ CPU legs
def cpu_pass(orc, ops):
    t0 = time.perf_counter()
    for (m, n, k, f), (a, b) in ops:
        orc.gemm_f32(a, b, *FORMS[f])
    return time.perf_counter() - t0


def cpu_operands(orc):
    ops = []
    for (m, n, k, f) in CPU_SAMPLE:
        tA, tB = FORMS[f]
        a = orc.uniform_pm1((k, m) if tA else (m, k), "cpu", m, n, k, "A")
        b = orc.uniform_pm1((n, k) if tB else (k, n), "cpu", m, n, k, "B")
        ops.append(((m, n, k, f), (a, b)))
    return ops


SAMPLE_TEXT = "sweep subset: {1024,2048}^3 x {NN,NT,TN} + 4096^3 NN + 128x10x4096 NN (195 GFLOP per pass)"


def cpu_baseline_leg():
    """OpenMP fp32 port of the same GEMMs on the host cores, bounded to roughly ten seconds."""
    from oracle import oracle as orc
    orc.use_all_cores()
    ops = cpu_operands(orc)
    cpu_pass(orc, ops[:3])  # warm the thread pool
    total, reps = 0.0, 0
    while total < 10.0 and reps < 6:
        total += cpu_pass(orc, ops)
        reps += 1
    return {"value": round(flops(CPU_SAMPLE) * reps / total / 1e12, 4), "unit": "TFLOP/s",
            "cores": orc.num_threads(), "kind": "port", "sample": f"{SAMPLE_TEXT}, {reps} passes"}


def reference_cuda_leg():
    """The reference's OWN CUDA kernels (seblas sgemm / conv / convDerive / convError, rebuilt for sm_100a into
    oracle/_ref/libseblas_ref.so) timed on the same GPU, as a second baseline beside the CPU port. Each seblas call
    ends in its own cudaDeviceSynchronize, so host wall-clock around the call is the reference's latency as its
    operands see it. Returns None when the library was not built (the reference tree was not mounted at build time)."""
    import ctypes
    path = os.path.join(ROOT, "oracle", "_ref", "libseblas_ref.so")
    if not os.path.exists(path):
        return None
    import torch
    try:
        lib = ctypes.CDLL(path)
    except OSError as exc:
        return {"error": str(exc)[:200]}
    out = {}

    def timed(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            t0 = time.perf_counter()
            fn()
            ts.append(time.perf_counter() - t0)
        return sorted(ts)[len(ts) // 2]

    p = lambda t: ctypes.c_void_p(t.data_ptr())
    for n in (1024, 2048, 4096):
        A = torch.rand(n, n, device="cuda") * 2 - 1
        B = torch.rand(1, n, n, device="cuda") * 2 - 1
        Cc = torch.zeros(1, n, n, device="cuda")
        for form, name in ((0, "NN"), (1, "TN")):
            dt = timed(lambda: lib.ref_gemm(form, p(A), p(B), p(Cc), n, n, n, 1))
            out[f"sgemm_{n}_{name}_tflops"] = round(2.0 * n ** 3 / dt / 1e12, 2)
    N, IC, H, OC = 128, 64, 32, 64
    X = torch.randn(N, IC, H, H, device="cuda")
    W = torch.randn(OC, IC, 3, 3, device="cuda") * 0.06
    Y = torch.zeros(N, OC, H, H, device="cuda")
    dX = torch.zeros_like(X)
    dW = torch.zeros_like(W)
    geo = (N, IC, H, H, OC, 3, 3, 1, 1, 1, 1)
    fl = 2.0 * N * OC * H * H * IC * 9
    out["conv_c3_fwd_us"] = round(timed(lambda: lib.ref_conv(p(W), p(X), p(Y), None, *geo)) * 1e6, 1)
    out["conv_c3_dgrad_us"] = round(timed(lambda: lib.ref_conv_derive(p(W), p(Y), p(dX), *geo)) * 1e6, 1)
    out["conv_c3_wgrad_us"] = round(timed(lambda: lib.ref_conv_error(p(Y), p(X), p(dW), *geo), reps=3) * 1e6, 1)
    out["conv_c3_fwd_tflops"] = round(fl / out["conv_c3_fwd_us"] / 1e6, 2)
    out["note"] = "reference seblas kernels (fp32 FFMA, sm_86 design) rebuilt for sm_100a; times include their own device sync"
    return out


def bench_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    orc.use_all_cores()
    ops = cpu_operands(orc)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_pass(orc, ops)
    t = 0.0
    for _ in range(args.steps):
        t += cpu_pass(orc, ops)
    ms = t * 1e3 / args.steps
    val = round(flops(CPU_SAMPLE) / (ms / 1e3) / 1e12, 4)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    print(json.dumps({
        "impl": "reference", "metric": "gemm_sweep_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 2), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": SAMPLE_TEXT,
                   "note": "the reference has no CPU implementation of this path; this is the OpenMP fp32 port in "
                           "oracle/cpu_ref.c on the host cores"},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": orc.num_threads(), "kind": "port",
                         "sample": SAMPLE_TEXT + " per step"},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--math", default="tf32", choices=["tf32", "3xtf32"])
    ap.add_argument("--shapes", default="", help="comma list like 4096x4096x4096_NN: restrict the sweep (profiling runs)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--conv-shapes", default="", help="comma list of CONV_SHAPES names: restrict the convolution section")
    ap.add_argument("--no-resnet", action="store_true", help="skip the ResNet-56 training section")
    ap.add_argument("--resnet", action="store_true", help="run the ResNet-56 section even with --shapes (profiling runs)")
    args = ap.parse_args()
    if args.shapes == "none":
        SWEEP[:] = [(128, 10, 4096, "NN")]
    elif args.shapes:
        keep = set(args.shapes.split(","))
        SWEEP[:] = [s for s in SWEEP if f"{s[0]}x{s[1]}x{s[2]}_{s[3]}" in keep]
        if not SWEEP:
            raise SystemExit("--shapes matched nothing")
    if args.warmup < 3 and not args.shapes:
        args.warmup = 3
    if args.impl == "reference":
        bench_reference(args)
    else:
        bench_ours(args)


if __name__ == "__main__":
    main()
