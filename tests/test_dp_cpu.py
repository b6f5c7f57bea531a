"""Data-parallel plumbing with two gloo ranks on CPU: sharding, sum-allreduce of the flat gradient buffer and
replica consistency after the Momentum update (the oracle's fp32 update stands in for the GPU kernel)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from crusaderbackend_b200 import dp
from oracle import oracle as orc


def test_shard_batch_partitions_exactly():
    for gb in (0, 1, 7, 128, 130):
        for world in (1, 2, 3, 4, 8):
            spans = [dp.shard_batch(gb, world, r) for r in range(world)]
            covered = []
            for s, c in spans:
                covered += list(range(s, s + c))
            assert covered == list(range(gb))
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1
    with pytest.raises(ValueError):
        dp.shard_batch(8, 2, 2)


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    r, w, _ = dp.init_from_env("gloo")
    n = 1003
    params = torch.from_numpy(orc.normal((n,), "dp", "w")) if r == 0 else torch.zeros(n)
    dp.broadcast_(params)
    mom = torch.zeros(n)
    ok = True
    for step in range(3):
        start, count = dp.shard_batch(10, w, r)
        # per-sample gradients; this rank sums its shard (the reference sums gradients over the batch)
        per_sample = np.stack([orc.normal((n,), "dp", "g", step, s) for s in range(start, start + count)])
        grads = torch.from_numpy(per_sample.sum(0).astype(np.float32))
        dp.allreduce_sum_(grads)
        wn, mn, _ = orc.momentum_f32(params.numpy(), grads.numpy(), mom.numpy(), 0.01, 0.9, 1e-4, True)
        params, mom = torch.from_numpy(wn), torch.from_numpy(mn)
        ok = ok and dp.replicas_identical(params)
    # a diverged replica must be detected
    bad = params.clone()
    if r == 1:
        bad[5] += 1e-3
    detected = not dp.replicas_identical(bad)
    if r == 0:
        torch.save(dict(params=params, ok=ok, detected=detected), out)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gloo_step_matches_single_process(tmp_path):
    out = str(tmp_path / "dp.pt")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    res = torch.load(out)
    assert res["ok"] and res["detected"]
    # single process, full batch
    n = 1003
    params, mom = orc.normal((n,), "dp", "w"), np.zeros(n, np.float32)
    for step in range(3):
        g = np.stack([orc.normal((n,), "dp", "g", step, s) for s in range(10)])
        # same association as the two-rank run: shard sums first, then their sum
        g2 = g[:5].sum(0).astype(np.float32) + g[5:].sum(0).astype(np.float32)
        params, mom, _ = orc.momentum_f32(params, g2, mom, 0.01, 0.9, 1e-4, True)
    assert np.array_equal(res["params"].numpy(), params)
