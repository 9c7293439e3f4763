"""The CPU oracle against the reference's own outputs (tests/golden/golden.npz, produced
by tests/golden/make_golden.py from models/dwoconv1d_reference/kernels/kernels.cpp) and
against known properties of the rasterised lines.  No GPU needed."""
import numpy as np
import pytest

from oracle import oracle as O
from tests.util import angle_list, make_inputs, rel_err


def _cases(golden, prefix):
    return sorted({k.split("_")[0] for k in golden.files if k.startswith(prefix)})


def test_loops_match_reference_bit_for_bit(oracle, golden):
    names = _cases(golden, "case")
    assert len(names) >= 8
    for name in names:
        N, C, H, W, K, s = golden[name + "_meta"]
        x, w, th, dy = (golden[f"{name}_{k}"] for k in ("x", "w", "theta", "dy"))
        assert np.array_equal(oracle.fprop(x, w, th, int(s)), golden[name + "_y"]), name
        assert np.array_equal(oracle.dgrad(dy, w, th, int(s)), golden[name + "_dx"]), name
        assert np.array_equal(oracle.wgrad(dy, x, th, int(K), int(s)), golden[name + "_dw"]), name


def test_module_semantics_match_reference(oracle, golden):
    """resid / bias / nhwc handling of the autograd function (kernels.cpp:141-203)."""
    for name in _cases(golden, "mod"):
        N, C, H, W, K, s, nhwc, resid = (int(v) for v in golden[name + "_meta"])
        g = {k: golden[f"{name}_{k}"] for k in ("x", "w", "theta", "bias", "dy", "y", "dx", "dw", "db")}
        y = O.module_forward(oracle, g["x"], g["w"], g["theta"], g["bias"], s, bool(nhwc), bool(resid))
        dx, dw, db = O.module_backward(oracle, g["x"], g["w"], g["theta"], g["dy"], g["bias"], s,
                                       bool(nhwc), bool(resid))
        assert np.array_equal(y, g["y"]) and np.array_equal(dx, g["dx"]) and np.array_equal(dw, g["dw"])
        assert np.allclose(db, g["db"], rtol=1e-5, atol=1e-5)


def test_impulse_response_is_the_tap_table(oracle, golden):
    """x = delta, w[k] = k+1: the output holds each tap's weight at minus its offset;
    colliding taps add.  Ties the offsets() helper to the reference's rasterisation."""
    y = golden["impulse_y"]
    dh, dw = oracle.offsets(O.round_robin_angles(8), 31)
    for c in range(8):
        expect = np.zeros((33, 33), np.float32)
        for k in range(31):
            # y[p,q] picks x[p+dh, q+dw] = delta(16,16)  ->  p = 16-dh, q = 16-dw
            expect[16 - dh[c, k], 16 - dw[c, k]] += k + 1
        assert np.array_equal(y[0, c], expect), c


def test_known_line_shapes(oracle):
    dh, dw = oracle.offsets(O.round_robin_angles(8), 31)
    uniq = [len(set(zip(dh[i].tolist(), dw[i].tolist()))) for i in range(8)]
    assert uniq == [31, 29, 21, 29, 31, 29, 21, 29]
    ext = [(int(abs(dh[i]).max()), int(abs(dw[i]).max())) for i in range(8)]
    assert ext == [(0, 15), (5, 13), (10, 10), (13, 5), (15, 0), (13, 5), (10, 10), (5, 13)]
    assert dh[1].tolist() == [5, 5, 4, 4, 4, 3, 3, 3, 2, 2, 1, 1, 1, 0, 0, 0, 0, 0, -1, -1, -1, -2, -2,
                              -3, -3, -3, -4, -4, -4, -5, -5]
    assert dw[1].tolist() == [-13, -12, -12, -11, -10, -9, -8, -7, -6, -5, -4, -3, -2, -1, 0, 0, 0, 1,
                              2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 12, 13]
    # lines are odd-symmetric, and a shorter kernel is the centre of a longer one
    assert np.array_equal(dh, -dh[:, ::-1]) and np.array_equal(dw, -dw[:, ::-1])
    for K in (7, 13, 15, 27):
        a, b = oracle.offsets(O.round_robin_angles(8), K)
        lo = 15 - K // 2
        assert np.array_equal(a, dh[:, lo:lo + K]) and np.array_equal(b, dw[:, lo:lo + K])


def test_layer_offset_permutes_the_same_eight_lines(oracle):
    """+90 degrees on odd layers (models/convnext.py:67-77) only re-orders the 8 lines."""
    a = oracle.offsets(O.model_angles(96, 8, 0.0), 31)
    b = oracle.offsets(O.model_angles(96, 8, 0.5), 31)
    lines = lambda t: {tuple(t[0][c]) + tuple(t[1][c]) for c in range(96)}
    assert lines(a) == lines(b) and len(lines(a)) == 8


@pytest.mark.parametrize("stride", [1, 2])
def test_f64_variants_agree(oracle, stride):
    x, w, dy = make_inputs(3, 2, 8, 12, 16, 31, stride)
    th = angle_list("random", 8, 5)
    assert rel_err(oracle.fprop(x, w, th, stride), oracle.fprop_f64(x, w, th, stride)) < 1e-6
    assert rel_err(oracle.dgrad(dy, w, th, stride), oracle.dgrad_f64(dy, w, th, stride)) < 1e-6
    assert rel_err(oracle.wgrad(dy, x, th, 31, stride), oracle.wgrad_f64(dy, x, th, 31, stride)) < 1e-5


def test_adjointness(oracle):
    """<fprop(x), dy> == <x, dgrad(dy)> == <w, wgrad(dy, x)> (exact in real arithmetic)."""
    for stride in (1, 2, 4):
        x, w, dy = make_inputs(11, 2, 8, 16, 12, 15, stride)
        th = angle_list("random", 8, 7)
        a = float((oracle.fprop_f64(x, w, th, stride) * dy).sum())
        b = float((oracle.dgrad_f64(dy, w, th, stride) * x).sum())
        c = float((oracle.wgrad_f64(dy, x, th, 15, stride) * w).sum())
        assert abs(a - b) <= 1e-9 * abs(a) + 1e-9 and abs(a - c) <= 1e-9 * abs(a) + 1e-9


def test_forward_safe_equals_unpadded_op(oracle):
    """Zero padding on the far side does not change the in-range outputs
    (dwoconv1d.py:154-187), for stride 1 on sizes that need padding."""
    x, w, _ = make_inputs(5, 1, 8, 25, 40, 13, 1)
    th = angle_list("model+", 8)
    bias = np.linspace(-1, 1, 8).astype(np.float32)
    a = O.forward_safe(oracle, x, w, th, bias, 1, False, False)
    b = O.module_forward(oracle, x, w, th, bias, 1, False, False)
    assert a.shape == b.shape and np.array_equal(a, b)
    # stride 2, odd size: output extents are ceil(H/2) x ceil(W/2)
    y = O.forward_safe(oracle, x, w, th, bias, 2, False, False)
    assert y.shape == (1, 8, 13, 20)


def test_dense_line_equals_conv2d(oracle):
    """The operator is a depthwise conv2d whose (2pad+1)^2 kernel holds w[c,k] scatter-added
    at the rasterised offsets — the CPU formulation used as a timed baseline."""
    torch = pytest.importorskip("torch")
    import torch.nn.functional as F
    x, w, _ = make_inputs(9, 2, 16, 14, 18, 31, 1)
    th = angle_list("rr", 16)
    dh, dw = oracle.offsets(th, 31)
    k2d = np.zeros((16, 1, 31, 31), np.float64)
    for c in range(16):
        for k in range(31):
            k2d[c, 0, dh[c, k] + 15, dw[c, k] + 15] += w[c, 0, 0, k]
    for stride in (1, 2):
        y = F.conv2d(torch.from_numpy(x).double(), torch.from_numpy(k2d), None, stride, 15, 1, 16).numpy()
        assert rel_err(oracle.fprop_f64(x, w, th, stride), y) < 1e-12
