"""Python face of the training-step executor (include/crusader_b200_train.h) for tests and bench.py.

torch owns the flat parameter / gradient / momentum buffers. Under torchrun the executor itself performs the
collective of a data-parallel step (cbt_dp_init: bucketed NCCL sum-allreduce of the gradients on a communication
stream, overlapped with the backward pass); torch.distributed only carries the 128-byte rendezvous id."""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from .api import Context, CrusaderError

_i, _ll, _f, _fl = C.c_int, C.c_longlong, C.c_void_p, C.c_float
TRAIN_SIGNATURES = {
    "cbt_resnet_create": (_i, [C.POINTER(C.c_void_p), C.c_void_p, _i, _i, _i, _i]),
    "cbt_densenet_create": (_i, [C.POINTER(C.c_void_p), C.c_void_p, _i, _i, _i, _i, _i]),
    "cbt_destroy": (_i, [C.c_void_p]),
    "cbt_last_error": (C.c_char_p, [C.c_void_p]),
    "cbt_param_count": (_ll, [C.c_void_p]),
    "cbt_param_entries": (_i, [C.c_void_p]),
    "cbt_param_entry": (_i, [C.c_void_p, _i, C.POINTER(_ll), C.POINTER(_ll), C.POINTER(_i), C.POINTER(_i), C.POINTER(_i)]),
    "cbt_op_count": (_i, [C.c_void_p]),
    "cbt_bind": (_i, [C.c_void_p, _f, _f, _f]),
    "cbt_forward": (_i, [C.c_void_p, _f, _f]),
    "cbt_backward": (_i, [C.c_void_p]),
    "cbt_update": (_i, [C.c_void_p, _fl, _fl, _fl]),
    "cbt_loss": (_i, [C.c_void_p, C.POINTER(_fl)]),
    "cbt_tensor_ptr": (C.c_void_p, [C.c_void_p, _i, _i]),
    "cbt_loss_ptr": (C.c_void_p, [C.c_void_p]),
    "cbt_copy_tensor": (_i, [C.c_void_p, _i, _i, _f, _ll]),
    "cbt_copy_loss": (_i, [C.c_void_p, _f]),
    "cbt_set_reference_bn_grad_order": (_i, [C.c_void_p, _i]),
    "cbt_params_changed": (_i, [C.c_void_p]),
    "cbt_set_bn_groups": (_i, [C.c_void_p, _i]),
    "cbt_dp_unique_id": (_i, [C.c_char_p]),
    "cbt_dp_init": (_i, [C.c_void_p, C.c_char_p, _i, _i, _i]),
    "cbt_dp_world": (_i, [C.c_void_p]),
    "cbt_set_wgrad_streams": (_i, [C.c_void_p, _i]),
    "cbt_side_launches": (_ll, [C.c_void_p]),
    "cbt_save_crseq": (_i, [C.c_void_p, C.c_char_p, C.c_uint]),
    "cbt_load_crseq": (_i, [C.c_void_p, C.c_char_p, C.POINTER(C.c_uint)]),
}
KINDS = {0: "conv", 1: "bn_gamma", 2: "bn_beta", 3: "fc_weight", 4: "fc_bias"}


def seeded_params(entries, n_params, seed_key="init") -> np.ndarray:
    """The flat parameter vector init_params binds: entry i of `entries` (dicts with kind, offset, size, dims) drawn
    from the generator keyed by (seed_key, i)."""
    from . import seeds
    host = np.zeros(n_params, dtype=np.float32)
    for i, e in enumerate(entries):
        sl = slice(e["offset"], e["offset"] + e["size"])
        if e["kind"] == "conv":
            oc, ic, fh, fw = e["dims"]
            host[sl] = seeds.normal((e["size"],), seed_key, i, std=float(np.sqrt(2.0 / (ic * fh * fw))))
        elif e["kind"] == "fc_weight":
            host[sl] = seeds.normal((e["size"],), seed_key, i, std=float(np.sqrt(2.0 / e["dims"][1])))
        elif e["kind"] == "fc_bias":
            host[sl] = seeds.normal((e["size"],), seed_key, i, std=float(np.sqrt(2.0 / e["size"])))
        elif e["kind"] == "bn_gamma":
            host[sl] = 1.0
    return host


def _load():
    lib = _lib.load()
    for name, (res, args) in TRAIN_SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    return lib


class ResNetTrainer:
    """ResNet-(6*blocks+2) training step on one GPU; `group` (a torch.distributed group or True) enables the
    gradient allreduce."""

    def __init__(self, ctx: Context, batch: int, blocks_per_stage: int = 9, image_hw: int = 32, classes: int = 10,
                 distributed: bool = False, _create=None):
        self.lib = _load()
        self.ctx = ctx
        self.batch, self.classes, self.image_hw = batch, classes, image_hw
        self.distributed = distributed
        h = C.c_void_p()
        if _create is None:
            rc = self.lib.cbt_resnet_create(C.byref(h), ctx.h, batch, blocks_per_stage, image_hw, classes)
        else:
            rc = _create(self.lib, h)
        self.h = h
        if rc != 0:
            raise CrusaderError(rc, self.lib.cbt_last_error(h).decode() if h else "model creation failed")
        self.n_params = int(self.lib.cbt_param_count(h))
        dev = torch.device("cuda", ctx.device)
        self.params = torch.zeros(self.n_params, device=dev)
        self.grads = torch.zeros(self.n_params, device=dev)
        self.momentum = torch.zeros(self.n_params, device=dev)
        self._check(self.lib.cbt_bind(h, self.params.data_ptr(), self.grads.data_ptr(), self.momentum.data_ptr()))
        if distributed:
            self._dp_init()
        self.entries = []
        for i in range(self.lib.cbt_param_entries(h)):
            off, size, isw, kind = _ll(), _ll(), _i(), _i()
            dims = (_i * 4)()
            self._check(self.lib.cbt_param_entry(h, i, C.byref(off), C.byref(size), C.byref(isw), C.byref(kind), dims))
            self.entries.append(dict(offset=off.value, size=size.value, is_weight=bool(isw.value), kind=KINDS[kind.value],
                                     dims=tuple(dims)))

    def _check(self, rc):
        if rc != 0:
            raise CrusaderError(rc, self.lib.cbt_last_error(self.h).decode())

    def close(self):
        if getattr(self, "h", None):
            # NCCL does not release a communicator while a CUDA graph that captured one of its collectives is alive
            # (ncclCommDestroy waits for the graph), so the graphs of capture_step go first
            for g in getattr(self, "_graphs", []):
                g.reset()
            self._graphs = []
            self.lib.cbt_destroy(self.h)
            self.h = None

    # ---- parameters
    def init_params(self, seed_key="init") -> np.ndarray:
        """He-normal filters and dense weights, gamma = 1, beta = 0 — the reference's randFillNetParams
        (seann/operands/seblas/Conv2D.cu:45-50, Linear.cu:42-46, BatchNorm.cu:8-11) with seeded draws."""
        host = seeded_params(self.entries, self.n_params, seed_key)
        self.set_params(host)
        return host

    def set_params(self, host: np.ndarray):
        self.params.copy_(torch.from_numpy(np.ascontiguousarray(host, dtype=np.float32)))
        self.grads.zero_()
        self.momentum.zero_()
        self.params_changed()

    def params_changed(self):
        """Call after writing to self.params directly: the executor re-packs its cached convolution filters."""
        self._check(self.lib.cbt_params_changed(self.h))

    def save_crseq(self, path: str, epoch: int = 0):
        """Write the parameters as a .crseq file the reference's loadSequence reads (seio/modelcache/codec.cu:41-97)."""
        self._check(self.lib.cbt_save_crseq(self.h, str(path).encode(), int(epoch)))

    def load_crseq(self, path: str) -> int:
        """Load the parameters of a .crseq file written by the reference's saveSequence (seio/modelcache/codec.cu:8-39)
        or by save_crseq; returns the file's epoch id."""
        epoch = C.c_uint(0)
        self._check(self.lib.cbt_load_crseq(self.h, str(path).encode(), C.byref(epoch)))
        return int(epoch.value)

    def set_reference_bn_grad_order(self, on: bool):
        """Store BatchNorm's d(gamma) / d(beta) in each other's slot, as the reference's operand does
        (seann/operands/seblas/BatchNorm.cu:24)."""
        self._check(self.lib.cbt_set_reference_bn_grad_order(self.h, int(on)))

    # ---- step
    def forward(self, images: torch.Tensor, labels_onehot: torch.Tensor):
        self._check(self.lib.cbt_forward(self.h, images.data_ptr(), labels_onehot.data_ptr()))

    def backward(self):
        self._check(self.lib.cbt_backward(self.h))

    def _dp_init(self, buckets: int = 3):
        """Joins the executor's own NCCL communicator: rank 0's rendezvous id travels over torch.distributed."""
        import torch.distributed as dist
        world, rank = dist.get_world_size(), dist.get_rank()
        buf = C.create_string_buffer(128)
        if rank == 0:
            self._check(self.lib.cbt_dp_unique_id(buf))
        t = torch.tensor(list(buf.raw), dtype=torch.uint8, device=self.params.device)
        dist.broadcast(t, 0)
        ident = bytes(t.cpu().tolist())
        self._check(self.lib.cbt_dp_init(self.h, ident, world, rank, buckets))

    def set_wgrad_streams(self, n: int):
        """Run the convolution weight gradients of the backward pass on n streams of their own (0 = inline)."""
        self._check(self.lib.cbt_set_wgrad_streams(self.h, int(n)))

    @property
    def launches(self) -> int:
        """Kernel launches so far: the context's stream plus the weight-gradient streams."""
        return int(self.ctx.launches) + int(self.lib.cbt_side_launches(self.h))

    def set_bn_groups(self, groups: int):
        """BatchNorm statistics per group of batch/groups consecutive samples (what `groups` data-parallel ranks compute)."""
        self._check(self.lib.cbt_set_bn_groups(self.h, groups))

    def allreduce_grads(self):
        """Kept for callers of the three-call form: with a distributed trainer cbt_backward has already summed the
        gradients over the ranks."""

    def update(self, lr: float, beta: float = 0.9, l2: float = 1e-4):
        self._check(self.lib.cbt_update(self.h, lr, beta, l2))

    def step(self, images, labels_onehot, lr, beta=0.9, l2=1e-4):
        self.forward(images, labels_onehot)
        self.backward()
        self.allreduce_grads()
        self.update(lr, beta, l2)

    # ---- whole step as one CUDA graph (launch-bound otherwise: ~700 kernels per ResNet-56 step)
    def capture_step(self, images, labels_onehot, lr, beta=0.9, l2=1e-4, warmup=2, include_allreduce=True):
        """Runs `warmup` eager steps (workspace growth, packed filters, NCCL set-up), then records forward + backward
        (with the gradient allreduce of a distributed trainer) + update into a torch.cuda.CUDAGraph that reads the
        given static input tensors, and freezes the context's workspace (a later call on the same context that needed a
        larger scratch block would otherwise free memory the graph still uses). Returns the graph; call .replay()
        after refreshing images / labels in place."""
        for _ in range(warmup):
            self.step(images, labels_onehot, lr, beta, l2)
        torch.cuda.synchronize()
        # the graph keeps the addresses of the context's scratch blocks: no reallocation from here on
        self.ctx._check(self.ctx.lib.cb_freeze_workspace(self.ctx.h, 1))
        graph = torch.cuda.CUDAGraph()
        old = self.ctx._stream
        with torch.cuda.graph(graph):
            cap = torch.cuda.current_stream(self.ctx.device)
            self.ctx._check(self.ctx.lib.cb_set_stream(self.ctx.h, C.c_void_p(cap.cuda_stream)))
            self.forward(images, labels_onehot)
            self.backward()
            if include_allreduce:
                self.allreduce_grads()
            self.update(lr, beta, l2)
        self.ctx._check(self.ctx.lib.cb_set_stream(self.ctx.h, C.c_void_p(old.cuda_stream)))
        torch.cuda.synchronize()
        if not hasattr(self, "_graphs"):
            self._graphs = []
        self._graphs.append(graph)   # close() resets them before the executor (and its communicator) goes
        return graph

    def loss_tensor(self) -> torch.Tensor:
        """One-element device tensor holding a copy of the summed loss of the last forward pass."""
        out = torch.empty(1, device=self.params.device)
        self._check(self.lib.cbt_copy_loss(self.h, out.data_ptr()))
        return out

    def loss(self) -> float:
        v = _fl()
        self._check(self.lib.cbt_loss(self.h, C.byref(v)))
        return float(v.value)

    def tensor(self, tid: int, shape, grad=False) -> torch.Tensor:
        """Copy of an internal activation (or its gradient) for tests."""
        n = int(np.prod(shape))
        out = torch.empty(n, device=self.params.device)
        self._check(self.lib.cbt_copy_tensor(self.h, tid, int(grad), out.data_ptr(), n))
        self.ctx.synchronize()
        return out.view(*shape)


class DenseNetTrainer(ResNetTrainer):
    """DenseNet-BC (growth k, `layers` bottleneck layers per block; k = 12, layers = 16 is DenseNet-BC-100)."""

    def __init__(self, ctx: Context, batch: int, growth: int = 12, layers: int = 16, image_hw: int = 32, classes: int = 10,
                 distributed: bool = False):
        super().__init__(ctx, batch, image_hw=image_hw, classes=classes, distributed=distributed,
                         _create=lambda lib, h: lib.cbt_densenet_create(C.byref(h), ctx.h, batch, growth, layers, image_hw,
                                                                        classes))
