"""Multi-process logic on CPU ranks (gloo, world_size 2): the batch shards without a
data-path collective, and the weight-gradient exchange is one flat all-reduce whose result
equals the single-process gradient.  The arithmetic on each rank is the CPU oracle (this
test exercises the sharding and reduction plumbing, not the kernels)."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from oracle.oracle import Oracle, module_backward, module_forward, round_robin_angles
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(0)                # same global batch on every rank
        N, C, H, W, K = 4, 16, 12, 12, 15
        x = rng.standard_normal((N, H, W, C)).astype(np.float32)
        dy = rng.standard_normal((N, H, W, C)).astype(np.float32)
        w = (0.02 * rng.standard_normal((C, 1, 1, K))).astype(np.float32)
        bias = rng.standard_normal(C).astype(np.float32)
        th = round_robin_angles(C)
        oracle = Oracle()
        lo, hi = rank * N // world, (rank + 1) * N // world          # batch shard of this rank
        y = module_forward(oracle, x[lo:hi], w, th, bias, 1, True, False)
        dx, dw, db = module_backward(oracle, x[lo:hi], w, th, dy[lo:hi], bias, 1, True, False)
        flat = torch.from_numpy(np.concatenate([dw.reshape(-1), db]))  # one flat gradient buffer
        dist.all_reduce(flat)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), y=y, dx=dx, flat=flat.numpy(), lo=lo, hi=hi)
    finally:
        dist.destroy_process_group()


def test_batch_sharding_and_gradient_allreduce(tmp_path):
    from oracle.oracle import Oracle, module_backward, module_forward, round_robin_angles
    world, port = 2, 29611 + os.getpid() % 500
    mp.start_processes(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True, start_method="spawn")
    rng = np.random.default_rng(0)
    N, C, H, W, K = 4, 16, 12, 12, 15
    x = rng.standard_normal((N, H, W, C)).astype(np.float32)
    dy = rng.standard_normal((N, H, W, C)).astype(np.float32)
    w = (0.02 * rng.standard_normal((C, 1, 1, K))).astype(np.float32)
    bias = rng.standard_normal(C).astype(np.float32)
    th = round_robin_angles(C)
    oracle = Oracle()
    y = module_forward(oracle, x, w, th, bias, 1, True, False)
    dx, dw, db = module_backward(oracle, x, w, th, dy, bias, 1, True, False)
    ref_flat = np.concatenate([dw.reshape(-1), db])
    for rank in range(world):
        r = np.load(os.path.join(str(tmp_path), f"rank{rank}.npz"))
        lo, hi = int(r["lo"]), int(r["hi"])
        assert np.array_equal(r["y"], y[lo:hi]) and np.array_equal(r["dx"], dx[lo:hi])   # no exchange needed
        err = np.abs(r["flat"] - ref_flat).max() / np.abs(ref_flat).max()
        assert err <= 1e-4, err                                                           # sum over ranks
