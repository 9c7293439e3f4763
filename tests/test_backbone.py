"""Dense-prediction backbone (cropped kernels, `.conv.` keys, per-stage norms) and the
classifier -> backbone checkpoint conversion."""
import json
import os

import numpy as np
import pytest
import torch

from oriented1d_b200 import backbone, convnext1d

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BB_KEYS = json.load(open(os.path.join(ROOT, "tests", "golden", "backbone_keys.json")))


@pytest.mark.parametrize("name,factory,variant", [("tiny_1d", backbone.backbone_tiny, "1d"),
                                                  ("tiny_1dpp", backbone.backbone_tiny, "1dpp"),
                                                  ("tiny_2dpp", backbone.backbone_tiny, "2dpp"),
                                                  ("base_1dpp", backbone.backbone_base, "1dpp")])
def test_backbone_state_dict_matches_reference_file(name, factory, variant):
    """Keys, shapes, parameter count and angles of the reference's own backbone class
    (semantic_segmentation/backbone/convnext.py), from the fixture tests/golden/make_model_keys.py
    wrote by importing that file."""
    m = factory(variant=variant)
    mine = {k: list(v.shape) for k, v in m.state_dict().items()}
    ref = BB_KEYS[name]
    assert set(mine) == set(ref), sorted(set(mine) ^ set(ref))[:10]
    assert all(mine[k] == ref[k] for k in ref)
    assert sum(p.numel() for p in m.parameters()) == BB_KEYS[name + "_params"]
    sd = m.state_dict()
    for k, vals in BB_KEYS[name + "_theta_sample"].items():
        assert np.array_equal(sd[k].flatten()[:16].numpy(), np.array(vals, np.float32)), k


def _small(variant, cls):
    kw = dict(depths=(1, 1, 2, 1), dims=(16, 32, 48, 64), variant=variant, stem_dim1=8)
    return cls(**kw)


@pytest.mark.parametrize("variant", ["1d", "1dpp"])
def test_backbone_layout(variant):
    """Key names and kernel lengths of the reference backbone
    (semantic_segmentation/backbone/convnext.py:74-103, :316-327, :395-399)."""
    m = _small(variant, backbone.ConvNeXt1DBackbone)
    sd = m.state_dict()
    assert not any(k.startswith("head.") or k.startswith("norm.") for k in sd)
    assert all(f"norm{i}.weight" in sd for i in range(4))
    ks = backbone.BACKBONE_BLOCK_KERNELS[variant]
    first = "dwconv" if variant == "1d" else "dwconv1"
    for i in range(4):
        assert sd[f"stages.{i}.0.{first}.conv.weight"].shape[-1] == ks[i][0]
        assert f"stages.{i}.0.{first}.conv.theta" in sd and f"stages.{i}.0.{first}.conv.bias" in sd
        if variant == "1dpp":
            assert sd[f"stages.{i}.0.dwconv2.conv.weight"].shape == (4 * (16, 32, 48, 64)[i], 1, 1, ks[i][1])
    assert sd["downsample_layers.0.dw1.conv.weight"].shape[-1] == backbone.BACKBONE_STEM_KERNEL[variant]


@pytest.mark.parametrize("variant", ["1d", "1dpp"])
def test_convert_classifier_state_dict(variant):
    torch.manual_seed(0)
    clf = _small(variant, convnext1d.ConvNeXt1D)
    for p in clf.parameters():
        torch.nn.init.normal_(p, std=0.1)
    sd = clf.state_dict()
    new = backbone.convert_classifier_state_dict({"model": sd}, variant)
    bb = _small(variant, backbone.ConvNeXt1DBackbone)
    res = bb.load_state_dict(new, strict=False)
    assert not res.unexpected_keys
    assert sorted(res.missing_keys) == sorted(f"norm{i}.{n}" for i in range(4) for n in ("weight", "bias"))
    # cropped kernels are the centre taps; angles and everything else are carried over unchanged
    first = "dwconv" if variant == "1d" else "dwconv1"
    old = sd[f"stages.3.0.{first}.weight"]
    got = bb.state_dict()[f"stages.3.0.{first}.conv.weight"]
    K, Kn = old.shape[-1], got.shape[-1]
    assert Kn == 13 and torch.equal(got, old[..., (K - Kn) // 2:(K - Kn) // 2 + Kn])
    assert torch.equal(bb.state_dict()[f"stages.2.1.{first}.conv.theta"], sd[f"stages.2.1.{first}.theta"])
    assert torch.equal(bb.state_dict()["stages.1.0.pwconv1.weight"], sd["stages.1.0.pwconv1.weight"])
    with pytest.raises(ValueError):
        short = dict(sd)
        short[f"stages.0.0.{first}.weight"] = sd[f"stages.0.0.{first}.weight"][..., :5]
        backbone.convert_classifier_state_dict(short, variant)


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["1d", "1dpp"])
def test_backbone_forward_any_size(variant):
    """Image sizes that are not multiples of 32: four stage maps of the expected extents; the stages
    whose kernels are not cropped reproduce the classifier's maps (after the stage norm)."""
    torch.manual_seed(0)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    clf = _small(variant, convnext1d.ConvNeXt1D)
    for p in clf.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.1)
    bb = _small(variant, backbone.ConvNeXt1DBackbone)
    bb.load_state_dict(backbone.convert_classifier_state_dict(clf.state_dict(), variant), strict=False)
    # the classifier checks divisibility by the stride; switch its convs to the any-size entry
    for mod in clf.modules():
        if isinstance(mod, convnext1d.DepthwiseOrientedConv1d):
            mod.forward = mod.forward_safe
    clf, bb = clf.cuda().eval(), bb.cuda().eval()
    img = torch.randn(2, 3, 104, 136, device="cuda")
    with torch.no_grad():
        outs = bb(img)
        ref = clf.forward_features(img, all_stages=True)
    assert [tuple(o.shape) for o in outs] == [(2, 16, 26, 34), (2, 32, 13, 17), (2, 48, 6, 8), (2, 64, 3, 4)]
    assert all(bool(torch.isfinite(o).all()) for o in outs)
    for i in (0, 1):          # stages 0 and 1 keep their 31-tap (15-tap) kernels
        norm = getattr(bb, f"norm{i}")
        with torch.no_grad():
            want = norm(ref[i].permute(0, 2, 3, 1)).permute(0, 3, 1, 2)
        assert float((outs[i] - want).abs().max()) <= 1e-4 * float(want.abs().max())
