"""Helpers shared by the tests: tolerances, seeded inputs, angle lists."""
import numpy as np

# fp32 tolerances of the operator: max|a-b| / max|b| with b the oracle
TOL_FPROP = 1e-5
TOL_DGRAD = 1e-5
TOL_WGRAD = 1e-4


def rel_err(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    den = np.abs(b).max()
    return np.abs(a - b).max() / (den if den > 0 else 1.0)


def bf16_round(a):
    """Round-to-nearest-even fp32 -> bf16 -> fp32, in numpy."""
    a = np.ascontiguousarray(a, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).reshape(a.shape)


def bf16_ulp(r, floor):
    """bf16 unit in the last place at |r| (8 significant bits), with |r| clamped from
    below by `floor` so that sums that cancel to ~0 are judged at the scale of the data."""
    m = np.maximum(np.abs(np.asarray(r, np.float64)), floor)
    return 2.0 ** (np.floor(np.log2(m)) - 7)


def assert_bf16_close(out, ref_fp32, what=""):
    """out (bf16 values as float) within 2 bf16 ulp of the fp32-accumulated reference."""
    ref = np.asarray(ref_fp32, np.float64)
    floor = 1e-3 * max(np.abs(ref).max(), 1e-30)
    bad = np.abs(np.asarray(out, np.float64) - ref) > 2.0 * bf16_ulp(ref, floor)
    assert not bad.any(), f"{what}: {bad.sum()} of {bad.size} outputs beyond 2 bf16 ulp"


def make_inputs(seed, N, C, H, W, K, stride=1):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((N, C, H, W)).astype(np.float32)
    w = (0.02 * rng.standard_normal((C, 1, 1, K))).astype(np.float32)
    dy = rng.standard_normal((N, C, -(-H // stride), -(-W // stride))).astype(np.float32)
    return x, w, dy


def angle_list(mode, C, seed=0):
    from oracle.oracle import model_angles, round_robin_angles
    if mode == "rr":
        return round_robin_angles(C)
    if mode == "model":
        return model_angles(C, 8, 0.0)
    if mode == "model+":
        return model_angles(C, 8, 0.5)
    if mode == "zero":
        return np.zeros(C, np.float32)
    return np.random.default_rng(seed).uniform(-2 * np.pi, 2 * np.pi, C).astype(np.float32)
