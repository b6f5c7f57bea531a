"""Host-side plumbing of the data-parallel training step: one process per GPU, the batch sharded by rank, one
sum-allreduce of the flat gradient buffer per step (gradients are sums over samples in the reference's convention,
seblas/operations/cuLoss.cu:231-234, so a SUM over ranks reproduces the single-process gradient of the full batch),
then the identical Momentum update on every rank — no parameter broadcast is needed after the first one."""
from __future__ import annotations

import os

import torch
import torch.distributed as dist


def shard_batch(global_batch: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous (start, count) of this rank's samples; the first global_batch % world ranks get one more."""
    if world < 1 or not 0 <= rank < world or global_batch < 0:
        raise ValueError("bad shard request")
    base, rem = divmod(global_batch, world)
    count = base + (1 if rank < rem else 0)
    start = rank * base + min(rank, rem)
    return start, count


def init_from_env(backend: str | None = None) -> tuple[int, int, int]:
    """(rank, world, local_rank) from the torchrun environment; initialises the default process group when
    WORLD_SIZE > 1 (NCCL on GPUs, gloo on CPU)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        kw = {}
        if backend == "nccl":
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, **kw)
    return rank, world, local


def allreduce_sum_(flat: torch.Tensor) -> torch.Tensor:
    """In-place sum over ranks of the flat gradient buffer (a no-op without a process group)."""
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
    return flat


def broadcast_(flat: torch.Tensor, src: int = 0) -> torch.Tensor:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.broadcast(flat, src)
    return flat


def replicas_identical(flat: torch.Tensor) -> bool:
    """True when every rank holds bit-identical values (compares an exact integer checksum of the bit patterns)."""
    if not (dist.is_initialized() and dist.get_world_size() > 1):
        return True
    bits = flat.detach().contiguous().view(torch.int32).to(torch.int64)
    w = torch.arange(1, bits.numel() + 1, device=bits.device, dtype=torch.int64) % 1000003
    cs = torch.stack([bits.sum(), (bits * w).sum()])
    lo, hi = cs.clone(), cs.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    return bool(torch.equal(lo, hi))
