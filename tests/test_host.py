"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol the
header declares, the host rasteriser and plan builder agree with the oracle, argument
validation returns status codes, and the Python module keeps the reference's surface."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import oriented1d_b200 as o1d
from oriented1d_b200 import _lib
from tests.util import angle_list

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "o1d.h")).read()
    declared = set(re.findall(r"\b(o1d_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    lib = ctypes.CDLL(_lib._build.LIB)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.o1d_abi_version() == _lib.ABI_VERSION


def test_strerror_and_status_codes():
    assert _lib.lib.o1d_strerror(0) == b"ok"
    for code in range(1, 6):
        assert _lib.lib.o1d_strerror(code) not in (b"ok", b"unknown status")
    assert _lib.lib.o1d_strerror(99) == b"unknown status"
    with pytest.raises(ValueError):
        _lib.check(1, "x")
    with pytest.raises(_lib.O1dError):
        _lib.check(2, "x")


@pytest.mark.parametrize("K", [3, 7, 13, 15, 27, 31, 63])
def test_offsets_equal_oracle(oracle, K):
    for mode in ("rr", "model", "model+", "random"):
        th = angle_list(mode, 96, seed=K)
        dh, dw = o1d.offsets(th, K)
        rh, rw = oracle.offsets(th, K)
        assert np.array_equal(dh.astype(np.int32), rh) and np.array_equal(dw.astype(np.int32), rw)


def test_offsets_rejects_bad_arguments():
    with pytest.raises(ValueError):
        o1d.offsets(np.zeros(4, np.float32), 4)       # even K


def _plan_fields(plan):
    hdr = plan.host[:64].view(torch.int32).tolist()
    C, K, ncls = hdr[1], hdr[2], hdr[3]
    cls = plan.host[hdr[7]:hdr[7] + 2 * C].view(torch.int16).numpy().astype(np.int64)
    taps = plan.host[hdr[8]:hdr[8] + ncls * K * 2].view(torch.int8).numpy().reshape(ncls, K, 2)
    canon = plan.host[hdr[9]:hdr[9] + ncls].view(torch.int8).numpy()
    return dict(C=C, K=K, ncls=ncls, max_dh=hdr[4], max_dw=hdr[5], all_canon=hdr[6], cls=cls, taps=taps,
                canon=canon)


@pytest.mark.parametrize("mode,expect_cls", [("rr", 8), ("model", 8), ("model+", 8), ("zero", 1)])
def test_plan_classes(oracle, mode, expect_cls):
    th = angle_list(mode, 96)
    plan = o1d.Plan(th, 31)
    f = _plan_fields(plan)
    assert plan.num_classes == f["ncls"] == expect_cls and f["all_canon"] == 1
    rh, rw = oracle.offsets(th, 31)
    for c in range(96):
        t = f["taps"][f["cls"][c]]
        assert np.array_equal(t[:, 0], rh[c]) and np.array_equal(t[:, 1], rw[c])
    assert f["max_dh"] == abs(rh).max() and f["max_dw"] == abs(rw).max()
    # canonical id i means "the line of angle i*pi/8"
    ch, cw = oracle.offsets(angle_list("rr", 8), 31)
    for i in range(f["ncls"]):
        o = f["canon"][i]
        assert np.array_equal(f["taps"][i][:, 0], ch[o]) and np.array_equal(f["taps"][i][:, 1], cw[o])


def test_plan_arbitrary_angles_get_their_own_classes(oracle):
    th = angle_list("random", 40, seed=3)
    f = _plan_fields(o1d.Plan(th, 15))
    rh, rw = oracle.offsets(th, 15)
    assert f["ncls"] == len({tuple(rh[c]) + tuple(rw[c]) for c in range(40)})
    for c in range(40):
        assert np.array_equal(f["taps"][f["cls"][c]][:, 0], rh[c])


def test_entry_points_reject_bad_arguments_without_a_gpu():
    """Validation happens before any CUDA call, so these run on a CPU-only host."""
    lib = _lib.lib
    plan = o1d.Plan(np.zeros(8, np.float32), 31)
    ph = plan.host.data_ptr()
    buf = torch.zeros(64)
    p = buf.data_ptr()
    # null x
    assert lib.o1d_fprop(None, p, None, ph, p, p, 1, 8, 8, 8, 31, 1, 0, 0, 0, None) == 1
    # even K
    assert lib.o1d_fprop(p, p, None, ph, p, p, 1, 8, 8, 8, 30, 1, 0, 0, 0, None) == 1
    # bad layout / dtype / stride
    assert lib.o1d_fprop(p, p, None, ph, p, p, 1, 8, 8, 8, 31, 1, 2, 0, 0, None) == 1
    assert lib.o1d_fprop(p, p, None, ph, p, p, 1, 8, 8, 8, 31, 1, 0, 5, 0, None) == 1
    assert lib.o1d_dgrad(p, p, ph, p, p, 1, 8, 8, 8, 31, 0, 0, 0, 0, None) == 1
    # plan built for another C / K
    assert lib.o1d_fprop(p, p, None, ph, p, p, 1, 8, 8, 16, 31, 1, 0, 0, 0, None) == 5
    assert lib.o1d_dgrad(p, p, ph, p, p, 1, 8, 8, 8, 15, 1, 0, 0, 0, None) == 5
    # corrupt plan
    assert lib.o1d_fprop(p, p, None, p, p, p, 1, 8, 8, 8, 31, 1, 0, 0, 0, None) == 5
    # workspace too small
    assert lib.o1d_wgrad(p, p, ph, p, p, None, p, 0, 1, 8, 8, 8, 31, 1, 0, 0, None) == 4
    assert lib.o1d_wgrad_workspace_bytes(1, 8, 8, 8, 31, 1, 0, 0) > 0
    assert lib.o1d_wgrad_workspace_bytes(1, 8, 8, 8, 30, 1, 0, 0) == 0
    assert lib.o1d_transpose(None, p, 1, 4, 4, 0, None) == 1


def test_module_surface_matches_reference():
    """Constructor, parameters and state dict as models/dwoconv1d/dwoconv1d.py:92-152."""
    angles = [float(a) for a in angle_list("model", 16)]
    m = o1d.DepthwiseOrientedConv1d(16, 16, 31, groups=16, stride=1, padding=15, bias=True, angle=angles,
                                    nhwc=True, resid=True)
    assert isinstance(m, torch.nn.Conv2d)
    sd = m.state_dict()
    assert list(sd) == ["weight", "bias", "theta"]
    assert sd["weight"].shape == (16, 1, 1, 31) and sd["bias"].shape == (16,) and sd["theta"].shape == (16,)
    assert sd["theta"].dtype == torch.float32 and m.theta.requires_grad
    assert m.resid.shape == (16, 1, 1, 31) and float(m.resid.sum()) == 16 and float(m.resid[0, 0, 0, 15]) == 1
    # scalar angle -> theta [C,1] (dwoconv1d.py:125-126)
    m2 = o1d.DepthwiseOrientedConv1d(8, 8, 7, groups=8, padding=3, angle=0.5, bias=False)
    assert m2.theta.shape == (8, 1) and m2.bias is None and m2.resid is None
    # Stem1D passes padding=(K-stride)//2; it only lands in nn.Conv2d.padding (convnext.py:149-150)
    m3 = o1d.DepthwiseOrientedConv1d(8, 8, 31, groups=8, stride=2, padding=14, angle=angles[:8])
    assert m3.padding == (0, 14) and m3.stride == (2, 2)
    with pytest.raises(AssertionError):
        o1d.DepthwiseOrientedConv1d(8, 8, 4, groups=8)          # even kernel
    with pytest.raises(AssertionError):
        o1d.DepthwiseOrientedConv1d(8, 16, 3, groups=8)         # not depthwise
    # state dict round trip, including a checkpoint whose theta is [C,1]
    m4 = o1d.DepthwiseOrientedConv1d(16, 16, 31, groups=16, padding=15, angle=[0.0] * 16)
    m4.load_state_dict(sd)
    assert torch.equal(m4.theta, m.theta)


def test_shape_mismatches_raise_before_any_launch():
    """A dy, weight or bias that does not match x would be read past its end on the device."""
    plan = o1d.Plan(np.zeros(8, np.float32), 7)
    x = torch.zeros(2, 8, 6, 6)
    w = torch.zeros(8, 1, 1, 7)
    with pytest.raises(ValueError, match="dy has shape"):
        o1d.wgrad(torch.zeros(2, 8, 6, 5), x, plan)
    with pytest.raises(ValueError, match="dy has shape"):
        o1d.wgrad(torch.zeros(1, 8, 6, 6), x, plan)
    with pytest.raises(ValueError, match="bias"):
        o1d.fprop(x, w, torch.zeros(7), plan)
    with pytest.raises(ValueError, match="weight"):
        o1d.fprop(x, torch.zeros(8, 1, 1, 5), None, plan)
    with pytest.raises(ValueError, match="channels"):
        o1d.fprop(torch.zeros(2, 4, 6, 6), w, None, plan)
    with pytest.raises(ValueError, match="dy extents"):
        o1d.dgrad(torch.zeros(2, 8, 3, 3), w, plan, 6, 6, 1)
    m = o1d.get_dwoconv1d_kernel("float", 7, 1, 3)
    with pytest.raises(ValueError, match="dy has shape"):
        m.wgrad(torch.zeros(2, 8, 6, 5), x, torch.zeros(8))


def test_plan_cache_does_not_outlive_its_angles():
    """The 5-callable module caches plans per theta tensor.  A second tensor with other angles
    must get its own plan even if the allocator reuses the first one's address."""
    m = o1d.get_dwoconv1d_kernel("float", 31, 1, 15)
    seen = []
    for angle in (0.0, np.pi / 4, np.pi / 2):
        th = torch.full((16,), angle, dtype=torch.float32)
        plan = m._plan(th)
        dh, dw = o1d.offsets(th.numpy(), 31)
        hdr = plan.host[:64].view(torch.int32).tolist()
        taps = plan.host[hdr[8]:hdr[8] + 31 * 2].view(torch.int8).numpy().reshape(31, 2)
        assert np.array_equal(taps[:, 0], dh[0]) and np.array_equal(taps[:, 1], dw[0]), angle
        assert m._plan(th) is plan                      # same tensor, same version: cached
        seen.append(th.data_ptr())
        del th
    # in-place change of the same tensor: version moves, the plan follows
    th = torch.zeros(16)
    p0 = m._plan(th)
    th.fill_(np.pi / 2)
    p1 = m._plan(th)
    assert p1 is not p0
    hdr = p1.host[:64].view(torch.int32).tolist()
    assert hdr[4] == 15 and hdr[5] == 0                   # vertical line: max |dh| 15, max |dw| 0
    # the nn.Module: swapping theta.data rebuilds the plan
    mod = o1d.DepthwiseOrientedConv1d(8, 8, 31, groups=8, padding=15, angle=[0.0] * 8)
    a = mod._get_plan()
    mod.theta.data = torch.full((8,), float(np.pi / 2))
    b = mod._get_plan()
    assert b is not a and b.host[:64].view(torch.int32).tolist()[4] == 15


def test_last_route_starts_unset():
    import threading
    out = []
    t = threading.Thread(target=lambda: out.append(_lib.lib.o1d_last_route()))
    t.start(); t.join()
    assert out == [-1]                                    # per thread, no call made yet
    assert o1d.ops.ROUTE_NAMES[-1] == "none"


def test_cpu_tensors_are_refused():
    m = o1d.DepthwiseOrientedConv1d(8, 8, 7, groups=8, padding=3, angle=0.0)
    with pytest.raises(RuntimeError, match="CUDA"):
        m(torch.zeros(1, 8, 8, 8))


def test_forward_requires_divisible_size_like_reference():
    m = o1d.DepthwiseOrientedConv1d(8, 8, 7, groups=8, stride=2, padding=3, angle=0.0)
    with pytest.raises(RuntimeError, match="divisible"):
        m(torch.zeros(1, 8, 7, 8))


def test_bare_module_names_resolve():
    import sys
    sys.path.insert(0, o1d.compat_path())
    try:
        import dwoconv1d
        import dwoconv1d_specialized
        assert dwoconv1d.DepthwiseOrientedConv1d is o1d.DepthwiseOrientedConv1d
        assert dwoconv1d_specialized.DepthwiseOrientedConv1d is o1d.DepthwiseOrientedConv1d
        assert len(dwoconv1d.oriented_dwconv1d_get_module_from_params("float", 31, 1, 15, Sb=1)) == 5
    finally:
        sys.path.remove(o1d.compat_path())


def test_reference_model_file_runs_on_this_operator():
    """The reference's own models/convnext.py, unmodified, builds its 1D / 1D++ / 2D++ models with
    this package answering `import dwoconv1d` — the drop-in claim, exercised where a checkout of
    the reference exists (skipped elsewhere)."""
    import sys
    import types
    from oracle.build import reference_root
    from oriented1d_b200 import convnext1d
    ref = reference_root()
    if ref is None:
        pytest.skip("no reference checkout")
    saved_path, saved_mods = list(sys.path), dict(sys.modules)
    try:
        layers = types.ModuleType("timm.models.layers")
        layers.trunc_normal_ = torch.nn.init.trunc_normal_
        layers.DropPath = lambda p=0.0: torch.nn.Identity()
        registry = types.ModuleType("timm.models.registry")
        registry.register_model = lambda f: f
        sys.modules.update({"timm": types.ModuleType("timm"), "timm.models": types.ModuleType("timm.models"),
                            "timm.models.layers": layers, "timm.models.registry": registry})
        sys.path.insert(0, o1d.compat_path())
        sys.path.insert(0, ref)
        for k in [k for k in sys.modules if k == "models" or k.startswith("models.")]:
            del sys.modules[k]
        from models import convnext as refmod
        assert refmod.DepthwiseOrientedConv1d is o1d.DepthwiseOrientedConv1d
        for variant in ("1d", "1dpp", "2dpp"):
            m = refmod.ConvNeXt(depths=[1, 1, 1, 1], dims=[16, 32, 48, 64], variant=variant, stem_dim1=8)
            mine = convnext1d.ConvNeXt1D(depths=(1, 1, 1, 1), dims=(16, 32, 48, 64), variant=variant, stem_dim1=8)
            assert {k: tuple(v.shape) for k, v in m.state_dict().items()} == \
                   {k: tuple(v.shape) for k, v in mine.state_dict().items()}
            mine.load_state_dict(m.state_dict())           # a reference checkpoint loads as is
            convs = [x for x in m.modules() if isinstance(x, o1d.DepthwiseOrientedConv1d)]
            assert convs and all(c.kernel_size[1] in (15, 31) for c in convs)
    finally:
        sys.path[:] = saved_path
        for k in list(sys.modules):
            if k not in saved_mods:
                del sys.modules[k]
