#!/usr/bin/env python
"""Benchmark of the dense-contraction path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Headline (every N, also N = 1): the ResNet-56 training step of the specification — 3 stages x 9 basic blocks, 16/32/64
channels, per-position BatchNorm, global average pooling, 10-way dense head, softmax cross-entropy, Momentum 0.9 —
on a GLOBAL batch of 128 synthetic 3x32x32 images (N(0,1), uniform labels, He-random weights from fixed seeds), sharded
over the ranks (strong scaling; one process per GPU, one sum-allreduce of the gradients per step). A step is forward +
backward + allreduce + update, replayed as one CUDA graph.

  value  images/s of the whole job with the batch already resident in HBM (CUDA events around K graph replays,
         max over ranks).
  e2e    the same step fed from pinned HOST memory: each step's images and labels are copied host->device on a copy
         stream while the previous step computes (two device batch buffers), and the step's loss is read back
         device->host, all inside the timed region.
  roofline   of the dominant kernel of the step, umma_conv_kernel (its convolution forward / data-gradient launches):
         algorithmic bytes 4(|X|+|W|+|Y|) of the step's stride-1 3x3 launches over their measured time (each distinct
         layer shape timed live under graph replay), against the measured HBM copy bandwidth.
  roofline_wgrad   the same object for umma_wgrad_kernel (the step's stride-1 3x3 weight gradients, which run on
         streams of their own beside the critical chain).
  cpu_baseline / --impl reference   the OpenMP fp32 port of the same step (oracle/resnet_step.py; the reference has
         no CPU implementation of this path) on a bounded sample of the batch, all host threads.

Extra keys on the same line (N = 1 only): `gemm` (the GEMM sweep of config 2 in TF32 and 3xTF32 against the measured
tensor peak), `conv` (config 3 and the ResNet-56 layer shapes), `densenet_bc100` (config 5), the measured UMMA-only TF32
peak, the reference's own CUDA kernels rebuilt for sm_100a timed on the same GPU; at N > 1 `weak_scaling_128_per_gpu`.
"""
from __future__ import annotations

import argparse
import ctypes as C
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
WORKLOAD = ("configs[3]: ResNet-56 training step (forward + backward + gradient allreduce + Momentum 0.9), global "
            "batch 128 of 3x32x32 fp32 N(0,1) images, uniform labels, He-random init")
GLOBAL_BATCH = 128
# Work model of the step: 0.754 GFLOP per image forward + backward; six activation passes per convolution layer
# (X read + Y write forward, dY read + dX write and dY + X read backward) plus BatchNorm / ReLU traffic, ~1.6 GB per
# 128-image step.
STEP_FLOPS = 96.5e9
STEP_MODEL_BYTES = 1.6e9


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured: MEASURED_PEAKS.json"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback: 6.65 TB/s, 1.59 PFLOP/s bf16"}


def profiled_traffic(key: str):
    """DRAM bytes per launch from the committed ncu summaries (profiles/traffic.json), or None."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get(key)
    except Exception:
        return None


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU while the timed region runs: NVML queries in this process every
    5 ms, or one nvidia-smi query (~50 ms) after the other when NVML cannot be loaded. Read-only."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.stop_flag = threading.Event()

    def _nvml_loop(self) -> bool:
        """In-process NVML reads (read-only queries), one sample every 5 ms; False when NVML is not usable."""
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons")
            max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            reasons_fn(h)
        except Exception:
            return False
        bits = (0x8, 0x40, 0x20, 0x4)   # hw_slowdown, hw_thermal_slowdown, sw_thermal_slowdown, sw_power_cap
        while not self.stop_flag.is_set():
            try:
                mask = int(reasons_fn(h))
                mhz = pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)
                self.samples.append([str(mhz), str(max_mhz)] + ["Active" if mask & b else "Not Active" for b in bits])
            except Exception:
                pass
            self.stop_flag.wait(0.005)
        return True

    def run(self):
        if self._nvml_loop():
            return
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self.stop_flag.wait(0.02)

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


# ------------------------------------------------------------------------------------------ ResNet-56 step (headline)
def resnet56_step(torch, local, world, rank, steps, warmup, weak=False, sampler=None):
    """Measurements of the ResNet-56 training step on this job (all ranks call it)."""
    import torch.distributed as dist
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    from crusaderbackend_b200 import dp, seeds
    gb = GLOBAL_BATCH * world if weak else GLOBAL_BATCH
    start, count = dp.shard_batch(gb, world, rank)
    ctx = Context(local, math="tf32", sync=False)
    tr = ResNetTrainer(ctx, batch=count, blocks_per_stage=9, image_hw=32, classes=10, distributed=world > 1)
    tr.init_params("bench")
    img_all = seeds.normal((gb, 3, 32, 32), "bench", "img")
    lab_all = seeds.rng_for("bench", "lab").integers(0, 10, gb)
    h_img = torch.from_numpy(img_all[start:start + count].copy()).pin_memory()
    onehot = torch.zeros(count, 10)
    onehot[torch.arange(count), torch.from_numpy(lab_all[start:start + count])] = 1
    h_lab = onehot.pin_memory()
    # two device batch buffers: the step reads one while the copy stream fills the other
    d_img = [torch.empty(count, 3, 32, 32, device="cuda") for _ in range(2)]
    d_lab = [torch.empty(count, 10, device="cuda") for _ in range(2)]
    for b in range(2):
        d_img[b].copy_(h_img)
        d_lab[b].copy_(h_lab)
    lr = 0.01 / gb
    tr.step(d_img[0], d_lab[0], lr)                      # first use: scratch, packed filters, NCCL set-up
    l0 = tr.launches
    tr.step(d_img[0], d_lab[0], lr)
    kernels_per_step = tr.launches - l0                  # steady state, all of the executor's streams
    graphs = [tr.capture_step(d_img[b], d_lab[b], lr, warmup=1 if b == 0 else 0) for b in range(2)]
    loss_dev = torch.empty(1, device="cuda")
    h_loss = torch.empty(1).pin_memory()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- value: batch resident in HBM
    for _ in range(max(3, warmup)):
        graphs[0].replay()
    barrier()
    if sampler is not None:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        graphs[0].replay()
    e1.record()
    barrier()
    ms_dev = e0.elapsed_time(e1) / steps

    # ---- e2e: host batches through a copy stream, loss read back every step
    compute = torch.cuda.current_stream()
    copy = torch.cuda.Stream()
    filled = [torch.cuda.Event() for _ in range(2)]
    consumed = [torch.cuda.Event() for _ in range(2)]

    def prefetch(b):
        with torch.cuda.stream(copy):
            copy.wait_event(consumed[b])                # the step that read this buffer has finished
            d_img[b].copy_(h_img, non_blocking=True)
            d_lab[b].copy_(h_lab, non_blocking=True)
            filled[b].record(copy)

    def e2e_steps(n):
        for b in range(2):
            consumed[b].record(compute)
        prefetch(0)
        for i in range(n):
            b = i & 1
            if i + 1 < n:
                prefetch(b ^ 1)
            compute.wait_event(filled[b])
            graphs[b].replay()
            consumed[b].record(compute)
            tr.lib.cbt_copy_loss(tr.h, loss_dev.data_ptr())
            h_loss.copy_(loss_dev, non_blocking=True)

    e2e_steps(max(3, warmup))
    barrier()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    e2e_steps(steps)
    s1.record()
    barrier()
    ms_e2e = s0.elapsed_time(s1) / steps
    if sampler is not None:
        sampler.stop_flag.set()
        sampler.join(timeout=2)
    ctx.synchronize()
    identical = dp.replicas_identical(tr.params)
    t = torch.tensor([ms_dev, ms_e2e], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_dev, ms_e2e = t.tolist()
    res = {"ms_per_step": ms_dev, "ms_per_step_e2e": ms_e2e, "global_batch": gb, "per_gpu_batch": count,
           "kernels_per_step": int(kernels_per_step), "replicas_identical": bool(identical),
           "loss_mean_last": round(float(h_loss.item()) / count, 5),
           "h2d_bytes_per_step": int(h_img.numel() * 4 + h_lab.numel() * 4) * world, "d2h_bytes_per_step": 4 * world}
    tr.close()
    ctx.close()
    return res


# ------------------------------------------------------------------------------------------ per-kernel sections (N = 1)
def graph_time_us(torch, ctx, fn, reps=20):
    """Device time per call of `fn` (a sequence of cb_* calls on ctx) under CUDA-graph replay, back to back."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    old = ctx._stream
    with torch.cuda.graph(g):
        cap = torch.cuda.current_stream(ctx.device)
        ctx.lib.cb_set_stream(ctx.h, C.c_void_p(cap.cuda_stream))
        for _ in range(reps):
            fn()
    ctx.lib.cb_set_stream(ctx.h, C.c_void_p(old.cuda_stream))
    torch.cuda.synchronize()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


# (name, N, IC, H, OC, F, stride, pad, launches of this shape in one ResNet-56 step: forward, data gradient)
CONV_SHAPES = [
    ("c3_64to64_3x3_s1_32x32", 128, 64, 32, 64, 3, 1, 1, 0, 0),
    ("c3_32to64_3x3_s2_32x32", 128, 32, 32, 64, 3, 2, 1, 0, 0),
    ("r56_16to16_3x3_s1_32x32", 128, 16, 32, 16, 3, 1, 1, 18, 18),
    ("r56_32to32_3x3_s1_16x16", 128, 32, 16, 32, 3, 1, 1, 17, 17),
    ("r56_64to64_3x3_s1_8x8", 128, 64, 8, 64, 3, 1, 1, 17, 17),
]


def conv_section(torch, local, peak_tflops, hbm_gbs):
    """Forward / data-gradient / weight-gradient of config 3 and the ResNet-56 layer shapes, per call under graph
    replay with the filters cached (as the executor runs them): TFLOP/s on 2*N*OC*OH*OW*IC*FH*FW against the measured
    tensor peak and GB/s on 4*(|X|+|W|+|Y|) against the measured HBM bandwidth. Also returns the aggregate over the
    stride-1 convolution forward / data-gradient launches of one ResNet-56 step (roofline of the dominant kernel)."""
    from crusaderbackend_b200.api import Context
    ctx = Context(local, math="tf32", sync=False)
    ctx.lib.cb_conv_cache_filters(ctx.h, 1)
    out = {}
    agg_bytes = agg_us = 0.0
    wg_bytes = wg_us = 0.0
    for (name, N, IC, H, OC, F, s, p, nf, nd) in CONV_SHAPES:
        OH = (H - F + 2 * p) // s + 1
        X = torch.randn(N, IC, H, H, device="cuda")
        W = torch.randn(OC, IC, F, F, device="cuda") * (2.0 / (IC * F * F)) ** 0.5
        Y = torch.empty(N, OC, OH, OH, device="cuda")
        dY = torch.randn(N, OC, OH, OH, device="cuda")
        dX = torch.empty_like(X)
        dW = torch.zeros_like(W)
        fl = 2.0 * N * OC * OH * OH * IC * F * F
        by = 4.0 * (X.numel() + W.numel() + Y.numel())
        calls = {"fwd": lambda: ctx.conv(W, X, Y, s, s, p, p), "dgrad": lambda: ctx.convDerive(W, dY, dX, s, s, p, p),
                 "wgrad": lambda: ctx.convError(dY, X, dW, s, s, p, p)}
        for pname, fn in calls.items():
            us = graph_time_us(torch, ctx, fn)
            out[f"{name}_{pname}"] = {"us": round(us, 1), "tflops": round(fl / us / 1e6, 1),
                                      "frac_tensor": round(fl / us / 1e6 / peak_tflops, 3),
                                      "gbs": round(by / us / 1e3, 1), "frac_hbm": round(by / us / 1e3 / hbm_gbs, 3),
                                      "kernel": ctx.last_kernel}
            if pname == "fwd":
                agg_bytes += nf * by
                agg_us += nf * us
            elif pname == "dgrad":
                agg_bytes += nd * by
                agg_us += nd * us
            else:  # one weight gradient per forward launch of the shape
                wg_bytes += nf * by
                wg_us += nf * us
    ctx.close()
    out["_wgrad_aggregate"] = (wg_bytes, wg_us)
    return out, agg_bytes, agg_us


def gemm_section(torch, local, peak_tflops):
    """GEMM sweep of config 2: every shape timed with CUDA events, L2 flushed by a 256 MiB write before each call; TF32
    for the whole sweep, 3xTF32 for the square NN shapes from 2048 up."""
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200 import seeds
    out = {}
    flush = torch.empty(256 * 1024 * 1024 // 4, device="cuda", dtype=torch.float32)
    bufs = {}
    for (m, n, k) in sorted({(m, n, k) for m, n, k, _ in SWEEP} | {(512, 512, 512)}):
        a = seeds.uniform_pm1((m, k), "bench", m, "A")
        b = seeds.uniform_pm1((k, n), "bench", m, "B")
        bufs[(m, n, k)] = (torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda(), torch.empty((m, n), device="cuda"))
    for math in ("tf32", "3xtf32"):
        ctx = Context(local, math=math, sync=False)
        # config 0 (512^3) rides along in both modes; it is not part of the sweep aggregate of config 1
        shapes = [(512, 512, 512, "NN")] + (SWEEP if math == "tf32" else
                                            [s for s in SWEEP if s[0] >= 2048 and s[3] == "NN" and s[0] == s[1]])
        total_fl = total_ms = 0.0
        for (m, n, k, form) in shapes:
            A, B, Cc = bufs[(m, n, k)]
            tA, tB = FORMS[form]
            ts = []
            for it in range(5):
                flush.fill_(1.0)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                ctx.gemm(A, B, Cc, transA=tA, transB=tB)
                e1.record()
                torch.cuda.synchronize()
                if it >= 2:
                    ts.append(e0.elapsed_time(e1))
            ms = sum(ts) / len(ts)
            tf = 2.0 * m * n * k / ms / 1e9
            key = f"{m}x{n}x{k}_{form}" + ("" if math == "tf32" else "_3xtf32")
            out[key] = {"tflops": round(tf, 1), "frac_tensor": round(tf / peak_tflops, 3), "us": round(ms * 1e3, 1)}
            if math == "3xtf32":
                out[key]["executed_tflops"] = round(3 * tf, 1)
                out[key]["frac_tensor_executed"] = round(3 * tf / peak_tflops, 3)
            if m != 512:
                total_fl += 2.0 * m * n * k
                total_ms += ms
        out["sweep_tflops" + ("" if math == "tf32" else "_3xtf32")] = round(total_fl / total_ms / 1e9, 1)
        ctx.close()
    return out


def resnet56_3xtf32_section(torch, local):
    """The ResNet-56 step of the headline in 3xTF32 mode (fp32-class accuracy), batch 128, one CUDA-graph replay per step."""
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import ResNetTrainer
    from crusaderbackend_b200 import seeds
    ctx = Context(local, math="3xtf32", sync=False)
    tr = ResNetTrainer(ctx, batch=GLOBAL_BATCH, blocks_per_stage=9, image_hw=32, classes=10)
    tr.init_params("bench")
    img = torch.from_numpy(seeds.normal((GLOBAL_BATCH, 3, 32, 32), "bench", "img")).cuda()
    lab = torch.zeros(GLOBAL_BATCH, 10, device="cuda")
    lab[torch.arange(GLOBAL_BATCH), torch.from_numpy(seeds.rng_for("bench", "lab").integers(0, 10, GLOBAL_BATCH)).cuda()] = 1
    g = tr.capture_step(img, lab, 0.01 / GLOBAL_BATCH, warmup=2)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    tr.close()
    ctx.close()
    return {"ms_per_step": round(ms, 3), "images_per_s": round(GLOBAL_BATCH / ms * 1e3, 1),
            "note": "3xTF32: convolutions of up to 32 channels (and 64 channels on 8x8 maps) in one tensor-core pass over "
                    "[x; x_lo; x] x [w; w; w_lo], the others as three passes"}


def densenet_section(torch, local):
    """Config 5: DenseNet-BC-100 (k = 12), batch 64, forward + backward + Momentum as one CUDA graph."""
    from crusaderbackend_b200.api import Context
    from crusaderbackend_b200.train import DenseNetTrainer
    from crusaderbackend_b200 import seeds
    ctx = Context(local, math="tf32", sync=False)
    tr = DenseNetTrainer(ctx, batch=64, growth=12, layers=16, image_hw=32, classes=10)
    tr.init_params("dn100")
    img = torch.from_numpy(seeds.normal((64, 3, 32, 32), "dn100", "img")).cuda()
    lab = torch.zeros(64, 10, device="cuda")
    lab[torch.arange(64), torch.from_numpy(seeds.rng_for("dn100", "lab").integers(0, 10, 64)).cuda()] = 1
    tr.step(img, lab, 0.01 / 64)
    l0 = tr.launches
    tr.step(img, lab, 0.01 / 64)
    kernels = tr.launches - l0
    g = tr.capture_step(img, lab, 0.01 / 64, warmup=1)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    tr.close()
    ctx.close()
    return {"ms_per_step": round(ms, 3), "images_per_s": round(64 / ms * 1e3, 1), "batch": 64, "kernels_per_step": int(kernels),
            "note": "forward + backward + Momentum, one CUDA-graph replay per step"}


def reference_cuda_leg(torch):
    """The reference's OWN CUDA kernels (seblas sgemm / conv / convDerive / convError, rebuilt for sm_100a into
    oracle/_ref/libseblas_ref.so) timed on the same GPU, as a second baseline beside the CPU port. Each seblas call
    ends in its own cudaDeviceSynchronize, so host wall-clock around the call is the reference's latency as its
    operands see it. Returns None when the library was not built (the reference tree was not mounted at build time)."""
    path = os.path.join(ROOT, "oracle", "_ref", "libseblas_ref.so")
    if not os.path.exists(path):
        return None
    try:
        lib = C.CDLL(path)
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

    p = lambda t: C.c_void_p(t.data_ptr())
    for n in (2048, 4096):
        A = torch.rand(n, n, device="cuda") * 2 - 1
        B = torch.rand(1, n, n, device="cuda") * 2 - 1
        Cc = torch.zeros(1, n, n, device="cuda")
        dt = timed(lambda: lib.ref_gemm(0, p(A), p(B), p(Cc), n, n, n, 1))
        out[f"sgemm_{n}_NN_tflops"] = round(2.0 * n ** 3 / dt / 1e12, 2)
    for (name, N, IC, H, OC) in (("c3_64to64", 128, 64, 32, 64), ("r56_16to16", 96, 16, 32, 16), ("r56_64to64_8x8", 96, 64, 8, 64)):
        X = torch.randn(N, IC, H, H, device="cuda")
        W = torch.randn(OC, IC, 3, 3, device="cuda") * 0.06
        Y = torch.zeros(N, OC, H, H, device="cuda")
        dX = torch.zeros_like(X)
        dW = torch.zeros_like(W)
        geo = (N, IC, H, H, OC, 3, 3, 1, 1, 1, 1)
        out[f"conv_{name}_fwd_us"] = round(timed(lambda: lib.ref_conv(p(W), p(X), p(Y), None, *geo)) * 1e6, 1)
        out[f"conv_{name}_dgrad_us"] = round(timed(lambda: lib.ref_conv_derive(p(W), p(Y), p(dX), *geo)) * 1e6, 1)
        out[f"conv_{name}_wgrad_us"] = round(timed(lambda: lib.ref_conv_error(p(Y), p(X), p(dW), *geo), reps=3) * 1e6, 1)
    out["note"] = ("reference seblas kernels (fp32 FFMA) rebuilt for sm_100a; times include their own device sync; the "
                   "ResNet-56 layer shapes use batch 96")
    return out


# ------------------------------------------------------------------------------------------ CPU legs
def cpu_step_rate(batch, steps, warmup):
    """images/s of the OpenMP fp32 port of the ResNet-56 step on `batch` images per step."""
    import numpy as np
    from oracle import oracle as orc
    from oracle.resnet_step import ResNetStepF32
    orc.use_all_cores()
    model = ResNetStepF32(9, 32, 10, key="bench")
    img = orc.normal((batch, 3, 32, 32), "bench", "img")
    lab = np.eye(10, dtype=np.float32)[orc.rng_for("bench", "lab").integers(0, 10, batch)]
    for _ in range(warmup):
        model.step(img, lab, 0.01 / GLOBAL_BATCH)
    t0 = time.perf_counter()
    for _ in range(steps):
        model.step(img, lab, 0.01 / GLOBAL_BATCH)
    dt = (time.perf_counter() - t0) / steps
    return batch / dt, dt, orc.num_threads()


def cpu_baseline_leg():
    """Bounded sample: two steps on 16 of the 128 images (after one warm-up step)."""
    rate, dt, cores = cpu_step_rate(16, 2, 1)
    return {"value": round(rate, 2), "unit": "images/s", "cores": cores, "kind": "port",
            "sample": f"ResNet-56 step on 16 of the 128 images, 2 steps after 1 warm-up ({dt:.2f} s per step)"}


def bench_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # bounded sample: 16 images per step; at most 6 timed steps so that the run ends within a few minutes
    steps = max(1, min(args.steps, 6))
    warm = 1
    rate, dt, cores = cpu_step_rate(16, steps, warm)
    sample = (f"ResNet-56 step on 16 of the 128 images per step, {steps} timed steps after {warm} warm-up "
              f"({dt:.2f} s per step)")
    print(json.dumps({
        "impl": "reference", "metric": "resnet56_train_images_per_s", "value": round(rate, 2), "unit": "images/s",
        "n_gpus": world, "steps": steps, "warmup": warm, "ms_per_step": round(dt * 1e3, 1), "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample,
                   "note": "the reference has no CPU implementation of this path; this is the OpenMP fp32 port in "
                           "oracle/ (cpu_ref.c + resnet_step.py) on the host cores"},
        "cpu_baseline": {"value": round(rate, 2), "unit": "images/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(rate, 2), "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }), flush=True)


# ------------------------------------------------------------------------------------------ single-kernel cases
def run_case(args):
    """`--case NAME`: a few launches of ONE kernel on a small, larger-than-L2-irrelevant case, for profiler captures of
    that kernel (prints a one-line summary, not the benchmark line). NAME is conv_fwd | conv_dgrad | conv_wgrad
    (with --shape N,IC,H,OC,F,stride), bn_fwd | bn_bwd (--shape N,C,H), momentum, head, gemm (--shape M,N,K,form)."""
    import torch
    from crusaderbackend_b200.api import Context
    torch.cuda.set_device(0)
    ctx = Context(0, math="tf32", sync=False)
    name = args.case
    shp = args.shape.split(",") if args.shape else []
    reps = max(1, args.steps)
    if name.startswith("conv_"):
        N, IC, H, OC, F, st = (int(v) for v in (shp or ["128", "16", "32", "16", "3", "1"]))
        p = 1 if F == 3 else 0
        OH = (H - F + 2 * p) // st + 1
        X = torch.randn(N, IC, H, H, device="cuda")
        W = torch.randn(OC, IC, F, F, device="cuda") * (2.0 / (IC * F * F)) ** 0.5
        Y = torch.empty(N, OC, OH, OH, device="cuda")
        dY = torch.randn(N, OC, OH, OH, device="cuda")
        dX = torch.empty_like(X)
        dW = torch.zeros_like(W)
        ctx.lib.cb_conv_cache_filters(ctx.h, 1)
        fn = {"conv_fwd": lambda: ctx.conv(W, X, Y, st, st, p, p), "conv_dgrad": lambda: ctx.convDerive(W, dY, dX, st, st, p, p),
              "conv_wgrad": lambda: ctx.convError(dY, X, dW, st, st, p, p)}[name]
    elif name in ("bn_fwd", "bn_bwd"):
        N, Cc, H = (int(v) for v in (shp or ["128", "16", "32"]))
        P = Cc * H * H
        X = torch.randn(N, P, device="cuda")
        Y = torch.empty_like(X)
        R = torch.randn(N, P, device="cuda")
        dY = torch.randn(N, P, device="cuda")
        dX, dR = torch.empty_like(X), torch.empty_like(X)
        g, b = torch.ones(P, device="cuda"), torch.zeros(P, device="cuda")
        dg, db = torch.empty(P, device="cuda"), torch.empty(P, device="cuda")
        pt = lambda t: C.c_void_p(t.data_ptr())
        if name == "bn_fwd":
            fn = lambda: ctx._check(ctx.lib.cb_bn_fwd_add_relu(ctx.h, pt(X), pt(b), pt(g), pt(R), pt(Y), N, P))
        else:
            ctx._check(ctx.lib.cb_bn_fwd_add_relu(ctx.h, pt(X), pt(b), pt(g), pt(R), pt(Y), N, P))
            fn = lambda: ctx._check(ctx.lib.cb_bn_bwd_fused_res(ctx.h, pt(dY), pt(g), pt(X), pt(dX), pt(dg), pt(db), pt(Y), pt(dR), 0, N, P))
    elif name == "gemm":
        M, N, K, form = (shp or ["4096", "4096", "4096", "NN"])
        M, N, K = int(M), int(N), int(K)
        tA, tB = FORMS[form]
        A = torch.randn((K, M) if tA else (M, K), device="cuda")
        B = torch.randn((N, K) if tB else (K, N), device="cuda")
        Cc = torch.empty(M, N, device="cuda")
        fn = lambda: ctx.gemm(A, B, Cc, transA=tA, transB=tB)
    elif name in ("momentum", "head"):
        from crusaderbackend_b200.train import ResNetTrainer
        tr = ResNetTrainer(ctx, batch=128, blocks_per_stage=9, image_hw=32, classes=10)
        tr.init_params("bench")
        img = torch.randn(128, 3, 32, 32, device="cuda")
        lab = torch.zeros(128, 10, device="cuda")
        lab[:, 0] = 1
        fn = lambda: tr.step(img, lab, 1e-4)
        reps = 1
    else:
        raise SystemExit(f"unknown case {name}")
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"case": name, "shape": args.shape, "launch_us_with_host_gaps": round(e0.elapsed_time(e1) / reps * 1e3, 1),
                      "kernel": ctx.last_kernel}), flush=True)


# ------------------------------------------------------------------------------------------ our arm
def bench_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    peaks = measured_peaks()

    sampler = ClockSampler(visible_gpu_index(local)) if rank == 0 else None
    head = resnet56_step(torch, local, world, rank, args.steps, args.warmup, sampler=sampler)
    weak = None
    if world > 1 and not args.quick:
        weak = resnet56_step(torch, local, world, rank, max(5, args.steps // 2), args.warmup, weak=True)

    line = None
    if rank == 0:
        gb = head["global_batch"]
        ms = head["ms_per_step"]
        floor_ms = STEP_MODEL_BYTES / world / peaks["hbm_gbs"] / 1e6
        line = {
            "metric": "resnet56_train_images_per_s", "value": round(gb / ms * 1e3, 1), "unit": "images/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
            "config": {"workload": WORKLOAD, "global_batch": gb, "per_gpu_batch": head["per_gpu_batch"],
                       "parallelism": f"dp{world}", "math": "tf32 tensor-core products, fp32 accumulate",
                       "l2": "one step touches ~1.6 GB of activations and gradients, far more than the 126 MB L2"},
            "e2e": {"value": round(gb / head["ms_per_step_e2e"] * 1e3, 1), "unit": "images/s",
                    "h2d_bytes_per_step": head["h2d_bytes_per_step"], "d2h_bytes_per_step": head["d2h_bytes_per_step"],
                    "ms_per_step": round(head["ms_per_step_e2e"], 4)},
            "gpu_launches": int(head["kernels_per_step"]) * args.steps,
            "kernels_per_step": head["kernels_per_step"],
            "replicas_identical": head["replicas_identical"],
            "loss_mean_last": head["loss_mean_last"],
            "clocks": sampler.summary(),
            "step_roofline": {"flops_per_step": STEP_FLOPS, "tflops": round(STEP_FLOPS / ms / 1e9, 1),
                              "model_bytes_per_step": STEP_MODEL_BYTES, "floor_ms_at_measured_hbm": round(floor_ms, 4),
                              "frac_of_byte_floor": round(floor_ms / ms, 4)},
            "roofline": None, "cpu_baseline": None,
        }
        if weak is not None:
            line["weak_scaling_128_per_gpu"] = {"images_per_s": round(weak["global_batch"] / weak["ms_per_step"] * 1e3, 1),
                                                "ms_per_step": round(weak["ms_per_step"], 4),
                                                "global_batch": weak["global_batch"],
                                                "replicas_identical": weak["replicas_identical"]}
    if rank == 0:
        # per-kernel sections on rank 0 (the other ranks wait at the closing barrier); everything beyond the roofline
        # of the dominant kernel only on single-GPU runs
        from crusaderbackend_b200.api import Context
        ctx = Context(local, math="tf32", sync=False)
        umma_peak = ctx.measure_umma_peak(256, False, False, 20000)
        ctx.close()
        conv, agg_bytes, agg_us = conv_section(torch, local, umma_peak, peaks["hbm_gbs"])
        achieved = agg_bytes / agg_us / 1e3 if agg_us else 0.0
        line["roofline"] = {"bound": "hbm", "kernel": "umma_conv_kernel (the 104 stride-1 3x3 forward / data-gradient "
                            "launches of one step; each layer shape timed under graph replay)",
                            "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": round(achieved / peaks["hbm_gbs"], 4),
                            "traffic": profiled_traffic("umma_conv_r56_16to16_fwd"), "peak_source": peaks["source"]}
        wg_bytes, wg_us = conv.pop("_wgrad_aggregate")
        wg = wg_bytes / wg_us / 1e3 if wg_us else 0.0
        # the second tensor-core kernel of the step (off the critical chain, on the weight-gradient streams)
        line["roofline_wgrad"] = {"bound": "hbm", "kernel": "umma_wgrad_kernel (the stride-1 3x3 weight-gradient launches of one "
                                  "step, one launch each; each layer shape timed under graph replay)",
                                  "achieved": round(wg, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                  "frac": round(wg / peaks["hbm_gbs"], 4),
                                  "traffic": profiled_traffic("umma_wgrad_r56_16to16"), "peak_source": peaks["source"]}
        line["tensor_peak"] = {"tf32_tflops_measured": round(umma_peak, 1),
                               "how": "cb_measure_umma_peak: resident-operand tcgen05.mma.kind::tf32 loop, M=128 N=256 K=8, every SM",
                               "bf16_tflops_measured_cublas": peaks["bf16_tflops"], "nominal_tf32_tflops": 1100.0}
        line["conv"] = conv
        if not args.quick and world == 1:
            line["gemm"] = gemm_section(torch, local, umma_peak)
            try:
                line["resnet56_3xtf32"] = resnet56_3xtf32_section(torch, local)
            except Exception as exc:
                line["resnet56_3xtf32"] = {"error": str(exc)[:300]}
            try:
                line["densenet_bc100"] = densenet_section(torch, local)
            except Exception as exc:
                line["densenet_bc100"] = {"error": str(exc)[:300]}
            if not args.no_cpu:
                try:
                    line["reference_cuda"] = reference_cuda_leg(torch)
                except Exception as exc:
                    line["reference_cuda"] = {"error": str(exc)[:200]}
                line["cpu_baseline"] = cpu_baseline_leg()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline and reference-CUDA legs (profiling runs)")
    ap.add_argument("--quick", action="store_true", help="headline and convolution table only (profiling runs)")
    ap.add_argument("--case", default=None, help="run a few launches of one kernel instead of the benchmark (profiler captures)")
    ap.add_argument("--shape", default=None, help="comma-separated extents of --case")
    args = ap.parse_args()
    if args.case:
        run_case(args)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        bench_reference(args)
    else:
        bench_ours(args)


if __name__ == "__main__":
    main()
