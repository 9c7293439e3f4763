"""Generate tests/golden/golden.npz from the REFERENCE's own CPU operator.

Needs a reference checkout (the script compiles models/dwoconv1d_reference/kernels/
kernels.cpp through oracle/build.py) and therefore only runs where that checkout
exists; the resulting fixture is committed and is what the tests read.

    python tests/golden/make_golden.py

Contents (all float32 unless noted):
  impulse_y        [1,8,33,33]  response to a unit impulse at (16,16) with w[c,k]=k+1 for
                                the 8 orientations i*pi/8, K=31: the tap table as the
                                reference rasterises it (colliding taps add up)
  caseNN_{x,w,theta,dy,y,dx,dw}  the three loops on seeded inputs (NCHW)
  modNN_{x,w,theta,bias,dy,y,dx,dw,db}  forward+backward through the reference's
                                autograd function with bias / resid / nhwc variations
  caseNN_meta / modNN_meta  int64 vectors (N,C,H,W,K,stride[,nhwc,resid])
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import build as obuild  # noqa: E402
from oracle.oracle import Reference, model_angles, round_robin_angles  # noqa: E402

# (N, C, H, W, K, stride, angle mode)
CASES = [
    (2, 16, 12, 10, 31, 1, "rr"),
    (1, 8, 16, 20, 15, 2, "rr"),
    (2, 24, 7, 7, 31, 1, "model"),
    (1, 16, 14, 14, 27, 1, "model+"),
    (1, 8, 8, 12, 7, 4, "rr"),
    (2, 8, 9, 11, 13, 1, "random"),
    (1, 16, 20, 28, 31, 2, "model+"),
    (1, 5, 6, 33, 3, 1, "random"),
    (1, 8, 36, 20, 31, 1, "rr"),
]
# (N, C, H, W, K, stride, nhwc, resid, angle mode)
MODULE_CASES = [
    (2, 8, 10, 12, 31, 1, 0, 0, "rr"),
    (2, 8, 10, 12, 31, 1, 1, 0, "rr"),
    (1, 16, 12, 8, 15, 1, 1, 1, "model"),
    (1, 8, 12, 16, 31, 2, 1, 0, "model+"),
    (1, 8, 12, 16, 15, 2, 0, 1, "random"),
]


def angles(mode, C, rng):
    if mode == "rr":
        return round_robin_angles(C)
    if mode == "model":
        return model_angles(C, 8, 0.0)
    if mode == "model+":
        return model_angles(C, 8, 0.5)
    return rng.uniform(-2 * np.pi, 2 * np.pi, C).astype(np.float32)


def main():
    obuild.build_ref()
    ref = Reference()
    out = {}
    # impulse response = tap table
    K = 31
    x = np.zeros((1, 8, 33, 33), np.float32)
    x[:, :, 16, 16] = 1
    w = np.tile(np.arange(1, K + 1, dtype=np.float32), (8, 1)).reshape(8, 1, 1, K)
    out["impulse_y"] = ref.fprop(x, w, round_robin_angles(8), 1)
    rng = np.random.default_rng(20231002)
    for i, (N, C, H, W, K, s, mode) in enumerate(CASES):
        x = rng.standard_normal((N, C, H, W)).astype(np.float32)
        w = (0.02 * rng.standard_normal((C, 1, 1, K))).astype(np.float32)
        th = angles(mode, C, rng)
        dy = rng.standard_normal((N, C, H // s, W // s)).astype(np.float32)
        p = f"case{i:02d}_"
        out[p + "meta"] = np.array([N, C, H, W, K, s], np.int64)
        out[p + "x"], out[p + "w"], out[p + "theta"], out[p + "dy"] = x, w, th, dy
        out[p + "y"] = ref.fprop(x, w, th, s)
        out[p + "dx"] = ref.dgrad(dy, w, th, s)
        out[p + "dw"] = ref.wgrad(dy, x, th, K, s)
    for i, (N, C, H, W, K, s, nhwc, resid, mode) in enumerate(MODULE_CASES):
        xs = (N, H, W, C) if nhwc else (N, C, H, W)
        ys = (N, H // s, W // s, C) if nhwc else (N, C, H // s, W // s)
        x = rng.standard_normal(xs).astype(np.float32)
        w = (0.02 * rng.standard_normal((C, 1, 1, K))).astype(np.float32)
        bias = rng.standard_normal(C).astype(np.float32)
        th = angles(mode, C, rng)
        dy = rng.standard_normal(ys).astype(np.float32)
        y, dx, dw, db = ref.module(x, w, th, bias, dy, s, bool(nhwc), bool(resid))
        p = f"mod{i:02d}_"
        out[p + "meta"] = np.array([N, C, H, W, K, s, nhwc, resid], np.int64)
        for k, v in dict(x=x, w=w, theta=th, bias=bias, dy=dy, y=y, dx=dx, dw=dw, db=db).items():
            out[p + k] = v
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
