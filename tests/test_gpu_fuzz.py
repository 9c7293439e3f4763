"""Seeded random shapes: every fast route (tiled, direct, chunk ranges, stride-2 input gradient)
against the general kernels on the same device inputs.  The general kernels are pinned to the
oracle by tests/test_gpu_parity.py; this file hunts for configuration corner cases (tile sizes,
halos, ragged edges, channel-chunk ranges)."""
import os

import numpy as np
import pytest
import torch

import oriented1d_b200 as o1d
from tests.util import angle_list

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _case(seed):
    rng = np.random.default_rng(seed)
    dtype = torch.float32 if rng.random() < 0.6 else torch.bfloat16
    ve = 8 if dtype == torch.float32 else 16
    C = int(rng.choice([1, 2, 3, 4, 6, 12])) * ve
    if rng.random() < 0.35:                       # sizes the tiled kernels take
        hw = int(rng.choice([7, 14, 21, 28, 8, 16, 24, 32, 56]))
        H, W = hw, hw
    else:
        H, W = int(rng.integers(1, 90)), int(rng.integers(1, 90))
    if rng.random() < 0.15:
        H, W = int(rng.integers(90, 260)), int(rng.integers(90, 330))
    K = int(rng.choice([1, 3, 7, 13, 15, 27, 31]))
    stride = int(rng.choice([1, 1, 2]))
    mode = str(rng.choice(["rr", "model", "model+", "random"]))
    N = int(rng.integers(1, 5))
    return N, C, H, W, K, stride, mode, dtype


@pytest.mark.parametrize("seed", range(int(os.environ.get("O1D_FUZZ_CASES", "48"))))
def test_fast_routes_equal_general_route(seed):
    N, C, H, W, K, s, mode, dtype = _case(seed)
    g = torch.Generator(device="cpu").manual_seed(seed)
    P, Q = -(-H // s), -(-W // s)
    x = torch.randn((N, H, W, C), generator=g).to(DEV).to(dtype)
    dy = torch.randn((N, P, Q, C), generator=g).to(DEV).to(dtype)
    w = (0.05 * torch.randn((C, 1, 1, K), generator=g)).to(DEV)
    bias = torch.randn((C,), generator=g).to(DEV)
    resid = bool(seed & 1)
    plan = o1d.Plan(angle_list(mode, C, seed), K)

    def run():
        y = o1d.fprop(x, w, bias, plan, s, True, resid).float()
        dx = o1d.dgrad(dy, w, plan, H, W, s, True, resid).float()
        dw, db = o1d.wgrad(dy, x, plan, s, True, True)
        return y, dx, dw, db

    try:
        o1d.ops.set_route(1)
        ref = run()
    finally:
        o1d.ops.set_route(0)
    for route in (0, 2, 3):
        try:
            o1d.ops.set_route(route)
            got = run()
        finally:
            o1d.ops.set_route(0)
        assert o1d.ops.device_status() == 0
        tag = (seed, route, N, C, H, W, K, s, mode, str(dtype))
        for name, a, b, tol32 in (("y", got[0], ref[0], 1e-5), ("dx", got[1], ref[1], 1e-5),
                                  ("dw", got[2], ref[2], 1e-4), ("db", got[3], ref[3], 1e-4)):
            assert a.shape == b.shape, (name, tag)
            if dtype == torch.float32 or name in ("dw", "db"):
                scale = float(b.abs().max().clamp_min(1e-20))
                assert float((a - b).abs().max()) <= tol32 * scale, (name, tag)
            else:           # both round an fp32 sum to bf16: at most one bf16 ulp apart
                assert float(((a - b).abs() / b.abs().clamp_min(1e-2)).max()) <= 2 ** -7, (name, tag)
