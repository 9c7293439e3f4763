"""Parity of the CUDA path (called through the C ABI) with the CPU oracle and with the
reference's own golden outputs.  Needs a B200: run with `-m gpu`.

Tolerances: fp32  max|a-b|/max|b| <= 1e-5 (fprop, dgrad), 1e-4 (wgrad, reduction order
differs); bf16  every output within 2 bf16 ulp of the fp32-accumulated result computed
from the same bf16-rounded inputs."""
import numpy as np
import pytest
import torch

import oriented1d_b200 as o1d
from oracle import oracle as O
from tests.util import (TOL_DGRAD, TOL_FPROP, TOL_WGRAD, angle_list, assert_bf16_close, bf16_round,
                        make_inputs, rel_err)

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _seed(shape):
    return sum(int(v) * m for v, m in zip(shape[:6], (1000003, 1009, 31, 7, 3, 1)))


def _to_dev(a_nchw, nhwc, dtype=torch.float32):
    t = torch.from_numpy(np.ascontiguousarray(a_nchw))
    if nhwc:
        t = t.permute(0, 2, 3, 1).contiguous()
    return t.to(DEV).to(dtype)


def _to_nchw(t, nhwc):
    t = t.float().cpu()
    if nhwc:
        t = t.permute(0, 3, 1, 2)
    return t.contiguous().numpy()


def _golden_cases(golden, prefix):
    return sorted({k.split("_")[0] for k in golden.files if k.startswith(prefix)})


@pytest.mark.parametrize("nhwc", [False, True])
def test_golden_loops(golden, nhwc):
    """The reference's own outputs for fprop / dgrad / wgrad."""
    for name in _golden_cases(golden, "case"):
        N, C, H, W, K, s = (int(v) for v in golden[name + "_meta"])
        x, w, th, dy = (golden[f"{name}_{k}"] for k in ("x", "w", "theta", "dy"))
        plan = o1d.Plan(th, K)
        wd = torch.from_numpy(w).to(DEV)
        y = o1d.fprop(_to_dev(x, nhwc), wd, None, plan, s, nhwc)
        dx = o1d.dgrad(_to_dev(dy, nhwc), wd, plan, H, W, s, nhwc)
        dw, _ = o1d.wgrad(_to_dev(dy, nhwc), _to_dev(x, nhwc), plan, s, nhwc)
        assert rel_err(_to_nchw(y, nhwc), golden[name + "_y"]) <= TOL_FPROP, name
        assert rel_err(_to_nchw(dx, nhwc), golden[name + "_dx"]) <= TOL_DGRAD, name
        assert rel_err(dw.cpu().numpy(), golden[name + "_dw"]) <= TOL_WGRAD, name


def test_golden_module(golden):
    """Forward + backward of the nn.Module against the reference's autograd function."""
    for name in _golden_cases(golden, "mod"):
        N, C, H, W, K, s, nhwc, resid = (int(v) for v in golden[name + "_meta"])
        g = {k: golden[f"{name}_{k}"] for k in ("x", "w", "theta", "bias", "dy", "y", "dx", "dw", "db")}
        m = o1d.DepthwiseOrientedConv1d(C, C, K, groups=C, stride=s, padding=K // 2, bias=True,
                                        angle=[float(a) for a in g["theta"]], nhwc=bool(nhwc),
                                        resid=bool(resid)).to(DEV)
        with torch.no_grad():
            m.weight.copy_(torch.from_numpy(g["w"]))
            m.bias.copy_(torch.from_numpy(g["bias"]))
        x = torch.from_numpy(g["x"]).to(DEV).requires_grad_(True)
        y = m(x)
        y.backward(torch.from_numpy(g["dy"]).to(DEV))
        assert rel_err(y.detach().cpu().numpy(), g["y"]) <= TOL_FPROP, name
        assert rel_err(x.grad.cpu().numpy(), g["dx"]) <= TOL_DGRAD, name
        assert rel_err(m.weight.grad.cpu().numpy(), g["dw"]) <= TOL_WGRAD, name
        assert rel_err(m.bias.grad.cpu().numpy(), g["db"]) <= TOL_WGRAD, name
        assert m.theta.grad is None


def test_impulse_response(golden):
    """x = delta, w[k] = k+1 reproduces the reference's tap table exactly (small integers)."""
    x = np.zeros((1, 8, 33, 33), np.float32)
    x[:, :, 16, 16] = 1
    w = np.tile(np.arange(1, 32, dtype=np.float32), (8, 1)).reshape(8, 1, 1, 31)
    plan = o1d.Plan(angle_list("rr", 8), 31)
    for nhwc in (False, True):
        y = o1d.fprop(_to_dev(x, nhwc), torch.from_numpy(w).to(DEV), None, plan, 1, nhwc)
        assert np.array_equal(_to_nchw(y, nhwc), golden["impulse_y"])


SHAPES = [
    # N, C, H, W, K, stride, angles
    (2, 96, 56, 56, 31, 1, "rr"),          # the reference's CPU-runnable configuration
    (2, 96, 56, 56, 31, 1, "model"),
    (3, 192, 28, 28, 31, 1, "rr"),
    (3, 384, 14, 14, 31, 1, "model+"),
    (4, 768, 7, 7, 31, 1, "rr"),
    (35, 64, 7, 7, 13, 1, "model+"),       # 7x7 plane kernels: short kernel, a partly filled second tile of 32 images
    (2, 64, 32, 48, 31, 2, "model"),       # stem-like: stride 2
    (2, 64, 32, 48, 15, 2, "model+"),
    (2, 16, 21, 27, 31, 2, "random"),      # stride 2, odd sizes, arbitrary angles
    (2, 16, 20, 28, 15, 1, "random"),
    (1, 24, 25, 40, 13, 1, "model+"),      # odd sizes
    (2, 16, 14, 14, 27, 1, "model"),
    (1, 40, 9, 5, 7, 1, "random"),
    (1, 8, 16, 16, 5, 4, "rr"),
    (1, 3, 5, 70, 63, 1, "random"),        # K wider than the register tap chunk
    (1, 8, 1, 1, 31, 1, "rr"),             # single pixel
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s[:6])) + s[6])
@pytest.mark.parametrize("nhwc", [False, True], ids=["nchw", "nhwc"])
def test_fp32_parity(oracle, shape, nhwc):
    N, C, H, W, K, s, mode = shape
    x, w, dy = make_inputs(_seed(shape), N, C, H, W, K, s)
    th = angle_list(mode, C, seed=C)
    bias = np.linspace(-1, 1, C).astype(np.float32)
    plan = o1d.Plan(th, K)
    wd, bd = torch.from_numpy(w).to(DEV), torch.from_numpy(bias).to(DEV)
    for resid in (False, True):
        y = o1d.fprop(_to_dev(x, nhwc), wd, bd, plan, s, nhwc, resid)
        dx = o1d.dgrad(_to_dev(dy, nhwc), wd, plan, H, W, s, nhwc, resid)
        ry, (rdx, rdw, rdb) = _oracle_fwd_bwd(oracle, x, w, th, dy, bias, s, resid)
        assert rel_err(_to_nchw(y, nhwc), ry) <= TOL_FPROP
        assert rel_err(_to_nchw(dx, nhwc), rdx) <= TOL_DGRAD
    dw, db = o1d.wgrad(_to_dev(dy, nhwc), _to_dev(x, nhwc), plan, s, nhwc, with_bias=True)
    # anchor for the reduction: the same sum in double precision
    rdw64 = oracle.wgrad_f64(*_pad_for_stride(dy, x, s), th, K, s)
    assert rel_err(dw.cpu().numpy(), rdw64) <= TOL_WGRAD
    assert rel_err(dw.cpu().numpy(), rdw) <= 2 * TOL_WGRAD     # the fp32 loops carry their own error
    assert rel_err(db.cpu().numpy(), dy.sum(axis=(0, 2, 3), dtype=np.float64)) <= TOL_WGRAD


def _oracle_fwd_bwd(oracle, x, w, th, dy, bias, s, resid):
    """Oracle forward/backward in NCHW; sizes the stride does not divide go through the
    reference's pad-and-crop route (forward_safe)."""
    if x.shape[2] % s == 0 and x.shape[3] % s == 0:
        return (O.module_forward(oracle, x, w, th, bias, s, False, resid),
                O.module_backward(oracle, x, w, th, dy, bias, s, False, resid))
    return (O.forward_safe(oracle, x, w, th, bias, s, False, resid),
            O.backward_safe(oracle, x, w, th, dy, bias, s, False, resid))


def _pad_for_stride(dy, x, s):
    """Zero-extend x (and dy) so that H, W divide by s; contributes nothing to the sums."""
    H, W = x.shape[2], x.shape[3]
    ph, pw = (-H) % s, (-W) % s
    xp = np.pad(x, ((0, 0), (0, 0), (0, ph), (0, pw)))
    return dy, xp


BF16_SHAPES = [SHAPES[0], SHAPES[2], SHAPES[4], SHAPES[5], SHAPES[8],
               SHAPES[1],                              # 56x56, block-wise angles
               (3, 384, 14, 14, 31, 1, "model+"),
               (3, 384, 14, 14, 31, 1, "rr"),
               (3, 192, 28, 28, 31, 1, "model"),
               (2, 768, 7, 7, 31, 1, "model+"),
               (1, 96, 50, 80, 27, 1, "model+"),       # dense-prediction map (row/column tiles)
               (2, 64, 32, 48, 31, 2, "model"),        # stem: stride 2, even/odd channel pairs share a line
               (2, 64, 32, 48, 15, 2, "model+")]


@pytest.mark.parametrize("shape", BF16_SHAPES, ids=lambda s: "x".join(map(str, s[:6])) + s[6])
@pytest.mark.parametrize("nhwc", [False, True], ids=["nchw", "nhwc"])
def test_bf16_parity(oracle, shape, nhwc):
    N, C, H, W, K, s, mode = shape
    x, w, dy = make_inputs(_seed(shape) + 1, N, C, H, W, K, s)
    x, w, dy = bf16_round(x), bf16_round(w), bf16_round(dy)
    th = angle_list(mode, C, seed=C)
    plan = o1d.Plan(th, K)
    wd = torch.from_numpy(w).to(DEV)
    y = o1d.fprop(_to_dev(x, nhwc, torch.bfloat16), wd, None, plan, s, nhwc)
    dx = o1d.dgrad(_to_dev(dy, nhwc, torch.bfloat16), wd, plan, H, W, s, nhwc)
    dw, db = o1d.wgrad(_to_dev(dy, nhwc, torch.bfloat16), _to_dev(x, nhwc, torch.bfloat16), plan, s, nhwc,
                       with_bias=True)
    assert y.dtype == torch.bfloat16 and dx.dtype == torch.bfloat16 and dw.dtype == torch.float32
    ry, (rdx, _, _) = _oracle_fwd_bwd(oracle, x, w, th, dy, None, s, False)
    assert_bf16_close(_to_nchw(y, nhwc), ry, "fprop")
    assert_bf16_close(_to_nchw(dx, nhwc), rdx, "dgrad")
    rdw64 = oracle.wgrad_f64(*_pad_for_stride(dy, x, s), th, K, s)
    assert rel_err(dw.cpu().numpy(), rdw64) <= TOL_WGRAD      # dw is accumulated and emitted in fp32
    assert rel_err(db.cpu().numpy(), dy.sum(axis=(0, 2, 3), dtype=np.float64)) <= TOL_WGRAD


def test_wgrad_is_deterministic():
    x, w, dy = make_inputs(7, 8, 96, 56, 56, 31)
    plan = o1d.Plan(angle_list("rr", 96), 31)
    for nhwc in (False, True):
        xd, dyd = _to_dev(x, nhwc), _to_dev(dy, nhwc)
        a = o1d.wgrad(dyd, xd, plan, 1, nhwc, True)
        for _ in range(3):
            b = o1d.wgrad(dyd, xd, plan, 1, nhwc, True)
            assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_transposes(dtype):
    for shape in [(2, 56, 56, 96), (3, 7, 7, 768), (1, 5, 9, 3), (2, 13, 17, 40), (1, 1, 1, 1), (1, 64, 64, 64)]:
        x = torch.randn(shape, device=DEV).to(dtype)
        y = o1d.nhwc_to_nchw(x)
        assert y.is_contiguous() and torch.equal(y, x.permute(0, 3, 1, 2).contiguous())
        z = o1d.nchw_to_nhwc(y)
        assert z.is_contiguous() and torch.equal(z, x)


def test_five_callable_surface(oracle):
    """The reference loader's fprop/dgrad/wgrad/nhwc_to_nchw/nchw_to_nhwc contract."""
    fprop, dgrad, wgrad, to_nchw, to_nhwc = o1d.oriented_dwconv1d_get_module_from_params("float", 15, 2, 7, Sb=1)
    x, w, dy = make_inputs(21, 2, 16, 12, 20, 15, 2)
    th = angle_list("model", 16)
    xd, wd, dyd, thd = (torch.from_numpy(a).to(DEV) for a in (x, w, dy, th))
    assert rel_err(fprop(xd, wd, thd).cpu().numpy(), oracle.fprop(x, w, th, 2)) <= TOL_FPROP
    assert rel_err(dgrad(dyd, wd, thd).cpu().numpy(), oracle.dgrad(dy, w, th, 2)) <= TOL_DGRAD
    assert rel_err(wgrad(dyd, xd, thd).cpu().numpy(), oracle.wgrad_f64(dy, x, th, 15, 2)) <= TOL_WGRAD
    assert torch.equal(to_nhwc(to_nchw(xd.permute(0, 2, 3, 1).contiguous())), xd.permute(0, 2, 3, 1).contiguous())
    with pytest.raises(RuntimeError, match="divisible"):
        fprop(xd[:, :, :11], wd, thd)


def test_module_arbitrary_size_and_bf16_theta(oracle):
    """forward_safe on sizes the reference would pad (dwoconv1d.py:154-187), and a module
    cast to bfloat16 still rasterises from its fp32 angles."""
    C, K = 24, 13
    th = angle_list("model+", C)
    m = o1d.DepthwiseOrientedConv1d(C, C, K, groups=C, stride=2, padding=K // 2, angle=[float(a) for a in th],
                                    nhwc=True, arbitrary_size=True).to(DEV)
    x, w, _ = make_inputs(4, 1, C, 25, 40, K, 2)
    with torch.no_grad():
        m.weight.copy_(torch.from_numpy(w))
        m.bias.zero_()
    y = m(_to_dev(x, True))
    assert tuple(y.shape) == (1, 13, 20, C)
    ry = O.forward_safe(oracle, x, w, th, None, 2, False, False)
    assert rel_err(_to_nchw(y.detach(), True), ry) <= TOL_FPROP
    # bf16 module: theta is rounded by .bfloat16(), the plan must not be
    mb = o1d.DepthwiseOrientedConv1d(8, 8, 31, groups=8, padding=15, angle=[float(a) for a in angle_list("rr", 8)]
                                     ).to(DEV).bfloat16()
    xi = np.zeros((1, 8, 33, 33), np.float32)
    xi[:, :, 16, 16] = 1
    with torch.no_grad():
        mb.weight.copy_(torch.arange(1, 32).float().repeat(8, 1).reshape(8, 1, 1, 31))
        mb.bias.zero_()
    yi = mb(torch.from_numpy(xi).to(DEV).bfloat16()).detach().float().cpu().numpy()
    dh, dw = oracle.offsets(angle_list("rr", 8), 31)
    for c in range(8):
        expect = np.zeros((33, 33), np.float32)
        for k in range(31):
            expect[16 - dh[c, k], 16 - dw[c, k]] += k + 1
        assert np.array_equal(yi[0, c], expect), c


@pytest.mark.parametrize("hw,C", [(56, 96), (28, 192), (14, 384), (7, 768)])
def test_full_size_properties(oracle, hw, C):
    """Batch-128 stage shapes, where the CPU oracle would take minutes: size-independent
    properties instead — linearity in x, exact adjointness identities between the three
    kernels, agreement of a sampled sub-batch with the rest — and the oracle itself on two
    images cut out of the full-batch results."""
    N, K = 128, 31
    g = torch.Generator(device="cpu").manual_seed(hw)
    plan = o1d.Plan(angle_list("rr", C), K)
    x1 = torch.randn((N, hw, hw, C), generator=g).to(DEV)
    x2 = torch.randn((N, hw, hw, C), generator=g).to(DEV)
    dy = torch.randn((N, hw, hw, C), generator=g).to(DEV)
    w = (0.02 * torch.randn((C, 1, 1, K), generator=g)).to(DEV)
    y1 = o1d.fprop(x1, w, None, plan, 1, True)
    y2 = o1d.fprop(x2, w, None, plan, 1, True)
    y12 = o1d.fprop(x1 + 2 * x2, w, None, plan, 1, True)
    assert float((y12 - (y1 + 2 * y2)).abs().max()) <= 1e-5 * float(y12.abs().max())
    # <fprop(x), dy> = <x, dgrad(dy)> = <w, wgrad(dy, x)>
    dx = o1d.dgrad(dy, w, plan, hw, hw, 1, True)
    dw, db = o1d.wgrad(dy, x1, plan, 1, True, True)
    a = float((y1.double() * dy.double()).sum())
    b = float((x1.double() * dx.double()).sum())
    c = float((w.double() * dw.double()).sum())
    scale = float((y1.double() * dy.double()).abs().sum())
    assert abs(a - b) <= 1e-6 * scale and abs(a - c) <= 1e-6 * scale
    assert float((db.double() - dy.double().sum(dim=(0, 1, 2))).abs().max()) <= 1e-4 * float(db.abs().max())
    # the batch is independent per image: a 2-image slice reproduces its part bit for bit
    ys = o1d.fprop(x1[5:7].contiguous(), w, None, plan, 1, True)
    assert torch.equal(ys, y1[5:7])
    # ... and those two images of the full-batch run are what the oracle computes
    th = angle_list("rr", C)
    xs, dys, wn = _to_nchw(x1[5:7], True), _to_nchw(dy[5:7], True), w.cpu().numpy()
    assert rel_err(_to_nchw(y1[5:7], True), oracle.fprop(xs, wn, th, 1)) <= TOL_FPROP
    assert rel_err(_to_nchw(dx[5:7], True), oracle.dgrad(dys, wn, th, 1)) <= TOL_DGRAD
    dws, _ = o1d.wgrad(dy[5:7].contiguous(), x1[5:7].contiguous(), plan, 1, True, True)
    assert rel_err(dws.cpu().numpy(), oracle.wgrad_f64(dys, xs, th, K, 1)) <= TOL_WGRAD
    # the full-batch weight gradient is the sum over images: two slices of 64 add up to it
    dwa, _ = o1d.wgrad(dy[:64].contiguous(), x1[:64].contiguous(), plan, 1, True, True)
    dwb, _ = o1d.wgrad(dy[64:].contiguous(), x1[64:].contiguous(), plan, 1, True, True)
    assert float((dw - (dwa + dwb)).abs().max()) <= 1e-5 * float(dw.abs().max())


@pytest.mark.parametrize("hw,C,mode", [(56, 96, "rr"), (56, 96, "model"), (28, 192, "rr"), (28, 192, "model+"),
                                        (14, 384, "rr"), (14, 384, "model"), (7, 768, "rr"), (7, 768, "model+"),
                                        (32, 64, "model"), (16, 24, "rr")])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_tiled_route_equals_general_route(hw, C, mode, dtype):
    """The tiled kernels (TMA-staged planes, register windows) against the general kernels
    on identical device inputs, forward and input gradient, with bias / identity tap."""
    N, K = 5, 31
    g = torch.Generator(device="cpu").manual_seed(hw * C)
    x = torch.randn((N, hw, hw, C), generator=g).to(DEV).to(dtype)
    dy = torch.randn((N, hw, hw, C), generator=g).to(DEV).to(dtype)
    w = (0.02 * torch.randn((C, 1, 1, K), generator=g)).to(DEV)
    bias = torch.randn((C,), generator=g).to(DEV)
    plan = o1d.Plan(angle_list(mode, C), K)
    try:
        o1d.ops.set_route(True)
        y_ref = o1d.fprop(x, w, bias, plan, 1, True, True).float()
        assert o1d.ops.last_route() == "general"
        dx_ref = o1d.dgrad(x, w, plan, hw, hw, 1, True, False).float()
        assert o1d.ops.last_route() == "general"
        dw_ref, db_ref = o1d.wgrad(dy, x, plan, 1, True, True)
        assert o1d.ops.last_route() == "general"
    finally:
        o1d.ops.set_route(False)
    # which family must answer: a fast path that declines would otherwise compare the general
    # kernels with themselves
    esize = 4 if dtype == torch.float32 else 2
    want = {2: ("tiled",), 3: ("direct",) if (C * esize) % 32 == 0 else ("direct", "tiled"),   # direct kernels
            0: ("tiled", "direct", "plane7", "lines")}                  # take 32-byte channel groups
    for route in (2, 3, 0):          # tiled preferred, direct preferred, automatic
        try:
            o1d.ops.set_route(route)
            y = o1d.fprop(x, w, bias, plan, 1, True, True).float()
            assert o1d.ops.last_route() in want[route], (route, o1d.ops.last_route())
            dx = o1d.dgrad(x, w, plan, hw, hw, 1, True, False).float()
            assert o1d.ops.last_route() in want[route], (route, o1d.ops.last_route())
        finally:
            o1d.ops.set_route(0)
        assert o1d.ops.device_status() == 0
        if dtype == torch.float32:
            assert float((y - y_ref).abs().max()) <= 1e-5 * float(y_ref.abs().max()), route
            assert float((dx - dx_ref).abs().max()) <= 1e-5 * float(dx_ref.abs().max()), route
        else:
            assert float(((y - y_ref).abs() / y_ref.abs().clamp_min(1e-2)).max()) <= 2 ** -7, route
            assert float(((dx - dx_ref).abs() / dx_ref.abs().clamp_min(1e-2)).max()) <= 2 ** -7, route
    for route in (0, 3):             # automatic (tiled where it applies), direct preferred
        try:
            o1d.ops.set_route(route)
            dw, db = o1d.wgrad(dy, x, plan, 1, True, True)
            assert o1d.ops.last_route() in want[route], (route, o1d.ops.last_route())
            dw2, db2 = o1d.wgrad(dy, x, plan, 1, True, True)
        finally:
            o1d.ops.set_route(0)
        assert o1d.ops.device_status() == 0
        assert torch.equal(dw, dw2) and torch.equal(db, db2), route          # deterministic
        assert float((dw - dw_ref).abs().max()) <= 1e-4 * float(dw_ref.abs().max()), route
        assert float((db - db_ref).abs().max()) <= 1e-4 * float(db_ref.abs().max()), route
    if dtype == torch.float32:
        assert float((y - y_ref).abs().max()) <= 1e-5 * float(y_ref.abs().max())
        assert float((dx - dx_ref).abs().max()) <= 1e-5 * float(dx_ref.abs().max())
    else:   # both round an fp32 sum to bf16: at most one bf16 ulp apart
        assert float(((y - y_ref).abs() / y_ref.abs().clamp_min(1e-2)).max()) <= 2 ** -7
        assert float(((dx - dx_ref).abs() / dx_ref.abs().clamp_min(1e-2)).max()) <= 2 ** -7


@pytest.mark.parametrize("mode,K,N", [("rr", 31, 3), ("rr", 15, 2), ("rr", 7, 1)])
def test_whole_line_kernels(oracle, mode, K, N):
    """The whole-line family (route 4: 8-channel items, lines slid through register windows, packed
    fp32 arithmetic) against the oracle at the 56x56 stage shape, with bias and the identity tap,
    forward and input gradient."""
    C, hw = 96, 56
    x, w, dy = make_inputs(K * 7 + N, N, C, hw, hw, K)
    th = angle_list(mode, C)
    bias = np.linspace(-1, 1, C).astype(np.float32)
    plan = o1d.Plan(th, K)
    wd, bd = torch.from_numpy(w).to(DEV), torch.from_numpy(bias).to(DEV)
    try:
        o1d.ops.set_route(4)
        for resid in (False, True):
            y = o1d.fprop(_to_dev(x, True), wd, bd, plan, 1, True, resid)
            assert o1d.ops.last_route() == "lines"
            dx = o1d.dgrad(_to_dev(dy, True), wd, plan, hw, hw, 1, True, resid)
            assert o1d.ops.last_route() == "lines"
            ry, (rdx, _, _) = _oracle_fwd_bwd(oracle, x, w, th, dy, bias, 1, resid)
            assert rel_err(_to_nchw(y, True), ry) <= TOL_FPROP
            assert rel_err(_to_nchw(dx, True), rdx) <= TOL_DGRAD
    finally:
        o1d.ops.set_route(0)
    assert o1d.ops.device_status() == 0


def test_whole_line_kernels_full_batch():
    """Batch 128 through the whole-line family: every CTA walks several items (ring wrap-around,
    tables loaded one item ahead); bit-equal to the same images run two at a time."""
    C, hw, K, N = 96, 56, 31, 128
    g = torch.Generator(device="cpu").manual_seed(3)
    x = torch.randn((N, hw, hw, C), generator=g).to(DEV)
    w = (0.02 * torch.randn((C, 1, 1, K), generator=g)).to(DEV)
    plan = o1d.Plan(angle_list("rr", C), K)
    try:
        o1d.ops.set_route(4)
        y = o1d.fprop(x, w, None, plan, 1, True)
        assert o1d.ops.last_route() == "lines"
        for i in (0, 37, 126):
            assert torch.equal(o1d.fprop(x[i:i + 2].contiguous(), w, None, plan, 1, True), y[i:i + 2])
        o1d.ops.set_route(2)
        yt = o1d.fprop(x, w, None, plan, 1, True)
    finally:
        o1d.ops.set_route(0)
    assert float((y - yt).abs().max()) <= 1e-5 * float(yt.abs().max())
    assert o1d.ops.device_status() == 0


@pytest.mark.parametrize("mode,K,N,C,hw", [("rr", 31, 3, 96, 56), ("model+", 31, 2, 96, 56), ("zero", 31, 2, 32, 56),
                                           ("rr", 15, 2, 96, 56), ("rr", 7, 1, 32, 56), ("rr", 31, 3, 64, 28),
                                           ("model", 27, 2, 64, 28)])
def test_walker_kernels(oracle, mode, K, N, C, hw):
    """The walker family (route 5: items kept in their NHWC layout in shared memory and computed in
    place, TMA loads and stores on both sides) against the oracle, with bias and the identity tap,
    forward and input gradient, round-robin and block-wise angle assignment."""
    x, w, dy = make_inputs(K * 5 + N + hw, N, C, hw, hw, K)
    th = angle_list(mode, C)
    bias = np.linspace(-1, 1, C).astype(np.float32)
    plan = o1d.Plan(th, K)
    wd, bd = torch.from_numpy(w).to(DEV), torch.from_numpy(bias).to(DEV)
    try:
        o1d.ops.set_route(5)
        for resid in (False, True):
            y = o1d.fprop(_to_dev(x, True), wd, bd, plan, 1, True, resid)
            assert o1d.ops.last_route() == "walk"
            dx = o1d.dgrad(_to_dev(dy, True), wd, plan, hw, hw, 1, True, resid)
            assert o1d.ops.last_route() == "walk"
            ry, (rdx, _, _) = _oracle_fwd_bwd(oracle, x, w, th, dy, bias, 1, resid)
            assert rel_err(_to_nchw(y, True), ry) <= TOL_FPROP
            assert rel_err(_to_nchw(dx, True), rdx) <= TOL_DGRAD
    finally:
        o1d.ops.set_route(0)
    assert o1d.ops.device_status() == 0


def test_line_only_layers_take_the_walker_route(oracle):
    """A 56x56 fp32 layer whose channels are all rows, columns or diagonals (no slanted line) is served
    by the walker family on the automatic route (the reference module's default, angle = 0, is such a
    layer, dwoconv1d.py:93-107); results against the oracle, forward and input gradient."""
    C, hw, K, N = 32, 56, 31, 2
    x, w, dy = make_inputs(77, N, C, hw, hw, K)
    th = np.asarray([(i % 4) * np.pi / 4 for i in range(C)], np.float32)
    plan = o1d.Plan(th, K)
    wd = torch.from_numpy(w).to(DEV)
    y = o1d.fprop(_to_dev(x, True), wd, None, plan, 1, True)
    assert o1d.ops.last_route() == "walk"
    dx = o1d.dgrad(_to_dev(dy, True), wd, plan, hw, hw, 1, True)
    assert o1d.ops.last_route() == "walk"
    assert rel_err(_to_nchw(y, True), oracle.fprop(x, w, th, 1)) <= TOL_FPROP
    assert rel_err(_to_nchw(dx, True), oracle.dgrad(dy, w, th, 1)) <= TOL_DGRAD
    # a slanted channel anywhere in the layer keeps the tiled kernels
    th2 = th.copy(); th2[5] = np.float32(np.pi / 8)
    o1d.fprop(_to_dev(x, True), wd, None, o1d.Plan(th2, K), 1, True)
    assert o1d.ops.last_route() == "tiled"
    assert o1d.ops.device_status() == 0


def test_walker_kernels_full_batch():
    """Batch 128 through the walker family: every CTA streams about ten items through its two tiles;
    bit-equal to the same images run two at a time, and equal to the tiled kernels up to rounding."""
    C, hw, K, N = 96, 56, 31, 128
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn((N, hw, hw, C), generator=g).to(DEV)
    w = (0.02 * torch.randn((C, 1, 1, K), generator=g)).to(DEV)
    plan = o1d.Plan(angle_list("rr", C), K)
    try:
        o1d.ops.set_route(5)
        y = o1d.fprop(x, w, None, plan, 1, True)
        assert o1d.ops.last_route() == "walk"
        for i in (0, 37, 126):
            assert torch.equal(o1d.fprop(x[i:i + 2].contiguous(), w, None, plan, 1, True), y[i:i + 2])
        o1d.ops.set_route(2)
        yt = o1d.fprop(x, w, None, plan, 1, True)
    finally:
        o1d.ops.set_route(0)
    assert float((y - yt).abs().max()) <= 1e-5 * float(yt.abs().max())
    assert o1d.ops.device_status() == 0


@pytest.mark.parametrize("K", [7, 13, 15, 27])
def test_tiled_short_kernels(oracle, K):
    """K < 31 uses the centre of the 31-tap line."""
    N, C, hw = 2, 32, 28
    x, w, dy = make_inputs(K, N, C, hw, hw, K)
    th = angle_list("model+", C)
    plan = o1d.Plan(th, K)
    wd = torch.from_numpy(w).to(DEV)
    y = o1d.fprop(_to_dev(x, True), wd, None, plan, 1, True)
    dx = o1d.dgrad(_to_dev(dy, True), wd, plan, hw, hw, 1, True)
    dw, _ = o1d.wgrad(_to_dev(dy, True), _to_dev(x, True), plan, 1, True)
    assert rel_err(_to_nchw(y, True), oracle.fprop(x, w, th, 1)) <= TOL_FPROP
    assert rel_err(_to_nchw(dx, True), oracle.dgrad(dy, w, th, 1)) <= TOL_DGRAD
    assert rel_err(dw.cpu().numpy(), oracle.wgrad_f64(dy, x, th, K, 1)) <= TOL_WGRAD


def test_nchw_module_takes_the_tiled_route(oracle):
    """An NCHW module whose NHWC form qualifies for the tiled kernels converts layout on the
    way in and out; results and gradients still match the oracle (NCHW)."""
    N, C, hw, K = 3, 96, 28, 31
    x, w, dy = make_inputs(77, N, C, hw, hw, K)
    th = angle_list("model", C)
    bias = np.linspace(-0.5, 0.5, C).astype(np.float32)
    m = o1d.DepthwiseOrientedConv1d(C, C, K, groups=C, padding=K // 2, angle=[float(a) for a in th]).to(DEV)
    with torch.no_grad():
        m.weight.copy_(torch.from_numpy(w))
        m.bias.copy_(torch.from_numpy(bias))
    assert o1d.ops.uses_tiled(m._get_plan(), N, hw, hw, 1, True, torch.float32)
    assert not o1d.ops.uses_tiled(m._get_plan(), N, hw, hw, 1, False, torch.float32)
    xd = torch.from_numpy(x).to(DEV).requires_grad_(True)
    y = m(xd)
    assert y.shape == xd.shape and y.is_contiguous()
    y.backward(torch.from_numpy(dy).to(DEV))
    ry = O.module_forward(oracle, x, w, th, bias, 1, False, False)
    rdx, rdw, rdb = O.module_backward(oracle, x, w, th, dy, bias, 1, False, False)
    assert rel_err(y.detach().cpu().numpy(), ry) <= TOL_FPROP
    assert rel_err(xd.grad.cpu().numpy(), rdx) <= TOL_DGRAD
    assert rel_err(m.weight.grad.cpu().numpy(), oracle.wgrad_f64(dy, x, th, K, 1)) <= TOL_WGRAD
    assert rel_err(m.bias.grad.cpu().numpy(), rdb) <= TOL_WGRAD


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_module_forward_and_backward_stay_on_fast_kernels(dtype):
    """Forward and backward of the nn.Module at a stage shape: every one of the three kernels
    must come from a fast family.  Backward runs on autograd's own worker thread, so the route
    is recorded from inside a tensor hook on that thread."""
    N, C, hw, K = 2, 96, 56, 31
    m = o1d.DepthwiseOrientedConv1d(C, C, K, groups=C, padding=K // 2, nhwc=True,
                                    angle=[float(a) for a in angle_list("rr", C)]).to(DEV)
    x = torch.randn((N, hw, hw, C), device=DEV).to(dtype).requires_grad_(True)
    seen = {}
    orig_dgrad, orig_wgrad = o1d.ops.dgrad, o1d.ops.wgrad

    def dgrad(*a, **k):
        out = orig_dgrad(*a, **k)
        seen["dgrad"] = o1d.ops.last_route()
        return out

    def wgrad(*a, **k):
        out = orig_wgrad(*a, **k)
        seen["wgrad"] = o1d.ops.last_route()
        return out

    o1d.ops.dgrad, o1d.ops.wgrad = dgrad, wgrad
    try:
        y = m(x)
        seen["fprop"] = o1d.ops.last_route()
        y.backward(torch.randn_like(y))
        torch.cuda.synchronize()
    finally:
        o1d.ops.dgrad, o1d.ops.wgrad = orig_dgrad, orig_wgrad
    assert set(seen) == {"fprop", "dgrad", "wgrad"}
    assert all(v in ("tiled", "lines") for v in seen.values()), seen
    assert o1d.ops.device_status() == 0


@pytest.mark.parametrize("N,C,H,W,K,nhwc,mode,dtype", [
    (2, 96, 56, 56, 31, True, "rr", torch.float32),         # tiled kernels, segments of 8
    (2, 64, 28, 28, 31, True, "model+", torch.float32),     # tiled kernels, segments of 7, block-wise angles
    (2, 128, 7, 7, 31, True, "model", torch.float32),       # 7x7: tiled instead of the plane kernels
    (2, 16, 20, 28, 15, True, "random", torch.float32),     # general kernels (arbitrary angles)
    (2, 16, 12, 12, 7, False, "rr", torch.float32),         # general kernels, NCHW
    (2, 64, 28, 28, 31, True, "model", torch.bfloat16),
])
def test_gelu_on_load(N, C, H, W, K, nhwc, mode, dtype):
    """conv(GELU(x)) with the GELU applied inside the kernels (the 1D++ blocks' second conv,
    models/convnext.py:389-391): forward, gradient with respect to the pre-activation tensor and
    weight gradient against float64 autograd through F.gelu and the unfused operator's dense form."""
    import torch.nn.functional as F
    g = torch.Generator(device="cpu").manual_seed(H * C + K)
    shape = (N, H, W, C) if nhwc else (N, C, H, W)
    x = torch.randn(shape, generator=g).to(DEV).to(dtype)
    dy = torch.randn(shape, generator=g).to(DEV).to(dtype)
    th = angle_list(mode, C, seed=C)
    m = o1d.DepthwiseOrientedConv1d(C, C, K, groups=C, padding=K // 2, nhwc=nhwc, resid=True,
                                    angle=[float(a) for a in th]).to(DEV)
    with torch.no_grad():
        m.weight.copy_(0.05 * torch.randn(m.weight.shape, generator=g))
        m.bias.copy_(torch.randn((C,), generator=g))
    m.gelu_input = True
    xf = x.clone().requires_grad_(True)
    y = m(xf)
    y.backward(dy)
    assert o1d.ops.device_status() == 0
    # reference: float64, GELU by torch, the conv as a dense depthwise conv2d over the rasterised kernel
    dh, dw = o1d.offsets(th, K)
    pad = K // 2
    wd = m.weight.detach().double().reshape(C, K).clone().requires_grad_(True)
    xr = x.double().clone().requires_grad_(True)
    wfull = wd + torch.nn.functional.one_hot(torch.tensor(pad), K).double().to(DEV)
    k2d = torch.zeros((C, 1, K, K), dtype=torch.float64, device=DEV)
    ci = torch.arange(C, device=DEV).repeat_interleave(K)
    ri = torch.from_numpy(dh.astype(np.int64)).reshape(-1).to(DEV) + pad
    qi = torch.from_numpy(dw.astype(np.int64)).reshape(-1).to(DEV) + pad
    k2d = k2d.index_put((ci, torch.zeros_like(ci), ri, qi), wfull.reshape(-1), accumulate=True)
    gx = F.gelu(xr)
    gx_nchw = gx.permute(0, 3, 1, 2) if nhwc else gx
    yr = F.conv2d(gx_nchw, k2d, m.bias.detach().double(), 1, pad, 1, C)
    yr = yr.permute(0, 2, 3, 1) if nhwc else yr
    yr.backward(dy.double())
    if dtype == torch.float32:
        tol_y, tol_w = 2e-5, 1e-4
    else:                                   # one bf16 rounding of each output
        tol_y, tol_w = 2 ** -7, 2e-3
    rel = lambda a, b: float((a.double() - b).abs().max() / b.abs().max())
    assert rel(y.detach(), yr.detach()) <= tol_y
    assert rel(xf.grad, xr.grad) <= tol_y
    assert rel(m.weight.grad.reshape(C, K), wd.grad) <= tol_w
    assert rel(m.bias.grad, dy.double().sum(dim=(0, 1, 2) if nhwc else (0, 2, 3))) <= tol_w


def test_bounded_wait_runs_out_without_a_fault():
    """The kernels wait for TMA transfers with a poll limit.  Here a wait is made to run out (a
    barrier that nothing completes, a limit of about a thousand polls): the kernel must return, the
    device flag must read 1, clearing must work, and the context must stay usable."""
    from oriented1d_b200 import _lib
    assert o1d.ops.device_status(clear=True) in (0, 1)
    assert o1d.ops.device_status() == 0
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    rc = _lib.lib.o1d_selftest_wait_timeout(gave_up.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 1
    assert o1d.ops.device_status() == 1
    assert o1d.ops.device_status(clear=True) == 1
    assert o1d.ops.device_status() == 0
    # the context is intact: a normal call still works and raises nothing
    plan = o1d.Plan(angle_list("rr", 8), 7)
    x = torch.ones((1, 8, 8, 8), device=DEV)
    y = o1d.fprop(x, torch.ones((8, 1, 1, 7), device=DEV), None, plan, 1, True)
    assert torch.isfinite(y).all() and o1d.ops.device_status() == 0


DENSE = [
    # C, H, W, K, stride: the dense-prediction backbone at 800x1280 input — stage maps with the
    # kernel lengths that backbone crops to (semantic_segmentation/backbone/convnext.py:316-327)
    # and the second stem convolution (400x640 -> 200x320)
    (96, 200, 320, 31, 1),
    (192, 100, 160, 31, 1),
    (384, 50, 80, 27, 1),
    (768, 25, 40, 13, 1),
    (64, 400, 640, 31, 2),
]


@pytest.mark.parametrize("shape", DENSE, ids=lambda s: "x".join(map(str, s)))
def test_dense_prediction_shapes(oracle, shape):
    """Large-spatial / small-batch maps (row/column tiles with line halos), forward, input and
    weight gradients against the oracle, NHWC, through the module's arbitrary-size entry."""
    C, H, W, K, s = shape
    x, w, dy = make_inputs(H + W, 1, C, H, W, K, stride=s)
    th = angle_list("model+", C)
    m = o1d.DepthwiseOrientedConv1d(C, C, K, groups=C, stride=s, padding=K // 2, nhwc=True, bias=False,
                                    angle=[float(a) for a in th], arbitrary_size=True).to(DEV)
    with torch.no_grad():
        m.weight.copy_(torch.from_numpy(w))
    xd = _to_dev(x, True).requires_grad_(True)
    y = m(xd)
    y.backward(_to_dev(dy, True))
    assert o1d.ops.device_status() == 0
    assert rel_err(_to_nchw(y.detach(), True), oracle.fprop(x, w, th, s)) <= TOL_FPROP
    assert rel_err(_to_nchw(xd.grad, True), oracle.dgrad(dy, w, th, s)) <= TOL_DGRAD
    assert rel_err(m.weight.grad.cpu().numpy(), oracle.wgrad_f64(dy, x, th, K, s)) <= TOL_WGRAD


def test_first_stem_conv_at_detection_size():
    """800x1280x64, K=31, stride 2 (models/convnext.py:158-160 at the detection input size): the
    automatic route against the general kernels on the same device inputs."""
    C, H, W, K, s = 64, 800, 1280, 31, 2
    g = torch.Generator(device="cpu").manual_seed(5)
    x = torch.randn((1, H, W, C), generator=g).to(DEV)
    w = (0.02 * torch.randn((C, 1, 1, K), generator=g)).to(DEV)
    plan = o1d.Plan(angle_list("model", C), K)
    y = o1d.fprop(x, w, None, plan, s, True)
    try:
        o1d.ops.set_route(1)
        y_ref = o1d.fprop(x, w, None, plan, s, True)
    finally:
        o1d.ops.set_route(0)
    assert o1d.ops.device_status() == 0
    assert y.shape == (1, H // 2, W // 2, C)
    assert float((y - y_ref).abs().max()) <= 1e-5 * float(y_ref.abs().max())


@pytest.mark.skipif(not O.ReferenceGPU.available(), reason="reference CUDA kernels not built (oracle/build.py --gpu-reference)")
@pytest.mark.parametrize("hw,C", [(56, 16), (28, 16), (14, 24), (7, 32)])
def test_reference_cuda_kernels_agree_with_the_cpu_loops(oracle, hw, C):
    """The reference's own specialised CUDA kernels (device sincosf rasterisation, fp32
    atomics in wgrad) against its CPU loops: pins the GPU baseline that bench.py times, and
    shows the device rasterisation lands on the same pixels as the host one."""
    ref = O.ReferenceGPU()
    N, K = 2, 31
    x, w, dy = make_inputs(hw + C, N, C, hw, hw, K)
    th = angle_list("rr", C)
    xd, wd, dyd, thd = (torch.from_numpy(a).to(DEV) for a in (x, w, dy, th))
    assert rel_err(ref.fprop(xd, wd, thd).cpu().numpy(), oracle.fprop(x, w, th, 1)) <= TOL_FPROP
    assert rel_err(ref.dgrad(dyd, wd, thd).cpu().numpy(), oracle.dgrad(dy, w, th, 1)) <= TOL_DGRAD
    assert rel_err(ref.wgrad(dyd, xd, thd).cpu().numpy(), oracle.wgrad_f64(dy, x, th, K, 1)) <= TOL_WGRAD


@pytest.mark.parametrize("C", [64, 96, 192, 384, 768, 1024])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_layernorm_channels_last(C, dtype):
    """o1d_layernorm_cl against F.layer_norm (+ exact GELU) in float64 on the same inputs."""
    g = torch.Generator(device="cpu").manual_seed(C)
    x = (2.0 * torch.randn((3, 5, 7, C), generator=g) + 0.5).to(DEV).to(dtype)
    w = torch.randn((C,), generator=g).to(DEV)
    b = torch.randn((C,), generator=g).to(DEV)
    for gelu in (False, True):
        y = o1d.ops.layer_norm_cl(x, w, b, 1e-6, gelu).double()
        ref = torch.nn.functional.layer_norm(x.double(), (C,), w.double(), b.double(), 1e-6)
        if gelu:
            ref = torch.nn.functional.gelu(ref)
        tol = 1e-5 if dtype == torch.float32 else 2 ** -7        # bf16: one rounding of the output
        assert float(((y - ref).abs() / ref.abs().clamp_min(1.0)).max()) <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("C,rows", [(64, (3, 5, 7)), (96, (2, 56, 56)), (128, (1, 9, 11)), (384, (4, 14, 14)),
                                    (512, (2, 7, 7)), (768, (5, 7, 7)), (1024, (3, 7, 5))])
def test_layernorm_channels_last_backward(C, rows, dtype):
    """o1d_layernorm_cl_bwd (through the autograd function the caller model uses) against float64
    autograd of F.layer_norm on the same inputs: dx, dweight, dbias; the sums are reproducible."""
    if dtype == torch.float32 and C > 512:
        pytest.skip("fp32 rows of more than 512 channels stay on the library LayerNorm")
    g = torch.Generator(device="cpu").manual_seed(C + rows[0])
    x = (1.5 * torch.randn(rows + (C,), generator=g) + 0.25).to(DEV).to(dtype)
    dy = torch.randn(rows + (C,), generator=g).to(DEV).to(dtype)
    w = (1.0 + 0.5 * torch.randn((C,), generator=g)).to(DEV).requires_grad_(True)
    b = torch.randn((C,), generator=g).to(DEV).requires_grad_(True)
    rel = lambda a, r: float((a.double() - r).abs().max() / r.abs().max())
    tol = 2e-5 if dtype == torch.float32 else 2 ** -7            # bf16: one rounding of dx
    for gelu in (False, True):                                   # True: the stems' LayerNorm -> GELU
        xg = x.clone().requires_grad_(True)
        w.grad = b.grad = None
        y = o1d.ops.LayerNormCL.apply(xg, w, b, 1e-6, gelu)
        y.backward(dy)
        xr = x.double().requires_grad_(True)
        wr, br = w.detach().double().requires_grad_(True), b.detach().double().requires_grad_(True)
        ref = torch.nn.functional.layer_norm(xr, (C,), wr, br, 1e-6)
        (torch.nn.functional.gelu(ref) if gelu else ref).backward(dy.double())
        assert rel(xg.grad, xr.grad) <= tol
        assert rel(w.grad, wr.grad) <= 1e-4 and rel(b.grad, br.grad) <= 1e-4
        dx2, dg2, db2 = o1d.ops.layer_norm_cl_bwd(x, dy, w.detach(), 1e-6, b.detach(), gelu)
        assert torch.equal(dx2, xg.grad) and torch.equal(dg2, w.grad) and torch.equal(db2, b.grad)
    assert o1d.ops.device_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("rows,C", [((3, 5, 7), 64), ((2, 56, 56), 384), ((64, 14, 14), 2048), ((1, 1, 1), 8),
                                    ((5, 7, 7), 4096), ((2, 9), 1000)])
def test_colsum_and_linear_bias_gradient(rows, C, dtype):
    """o1d_colsum against a float64 sum, and the Linear wrapper's three gradients against
    autograd's on the same inputs."""
    g = torch.Generator(device="cpu").manual_seed(C + rows[0])
    dy = torch.randn(rows + (C,), generator=g).to(DEV).to(dtype)
    s = o1d.ops.colsum(dy)
    ref = dy.double().reshape(-1, C).sum(0)
    assert float((s.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max().clamp_min(1.0)) * (dy.numel() // C) ** 0.5
    assert torch.equal(s, o1d.ops.colsum(dy))                         # fixed order
    cin = 24
    lin = torch.nn.Linear(cin, C).to(DEV).to(dtype)
    x = torch.randn(rows + (cin,), generator=g).to(DEV).to(dtype)
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    o1d.ops.linear_cl(lin, xa).backward(dy)
    ga = [xa.grad.clone(), lin.weight.grad.clone(), lin.bias.grad.clone()]
    lin.zero_grad()
    lin(xb).backward(dy)
    tol = 1e-5 if dtype == torch.float32 else 2 ** -6
    for a, b in zip(ga, [xb.grad, lin.weight.grad, lin.bias.grad]):
        assert float((a.double() - b.double()).abs().max()) <= tol * float(b.double().abs().max().clamp_min(1e-6))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("cin,cout", [(3, 64), (1, 8), (4, 96)])
def test_pointwise_in(dtype, cin, cout):
    """Stem input projection (NCHW image -> channels-last, Linear over the input channels)
    against torch in float64 on the same (rounded) inputs."""
    g = torch.Generator(device="cpu").manual_seed(cin * 100 + cout)
    x = torch.randn((3, cin, 17, 23), generator=g).to(DEV).to(dtype)
    w = torch.randn((cout, cin), generator=g).to(DEV)
    b = torch.randn((cout,), generator=g).to(DEV)
    y = o1d.ops.pointwise_in(x, w, b)
    ref = torch.nn.functional.linear(x.double().permute(0, 2, 3, 1), w.double(), b.double())
    assert y.shape == ref.shape and y.is_contiguous()
    tol = 1e-6 if dtype == torch.float32 else 2 ** -8
    assert float(((y.double() - ref).abs() / ref.abs().clamp_min(1.0)).max()) <= tol
    y0 = o1d.ops.pointwise_in(x, w, None)
    ref0 = ref - b.double()
    assert float(((y0.double() - ref0).abs() / ref0.abs().clamp_min(1.0)).max()) <= tol
