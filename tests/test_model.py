"""The ConvNeXt-1D / 1D++ caller (oriented1d_b200/convnext1d.py): same checkpoint layout as the
reference model (fixture from tests/golden/make_model_keys.py), and — on a GPU — the same
function as a pure-PyTorch restatement of every layer (dense conv2d for the oriented convs)."""
import json
import os

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import oriented1d_b200 as o1d
from oriented1d_b200 import convnext1d

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KEYS = json.load(open(os.path.join(ROOT, "tests", "golden", "convnext_keys.json")))


@pytest.mark.parametrize("name,factory,variant", [("tiny_1d", convnext1d.convnext_tiny, "1d"),
                                                  ("tiny_1dpp", convnext1d.convnext_tiny, "1dpp"),
                                                  ("base_1dpp", convnext1d.convnext_base, "1dpp")])
def test_state_dict_layout_matches_reference(name, factory, variant):
    m = factory(variant=variant)
    mine = {k: list(v.shape) for k, v in m.state_dict().items()}
    ref = KEYS[name]
    assert set(mine) == set(ref), sorted(set(mine) ^ set(ref))[:10]
    assert all(mine[k] == ref[k] for k in ref)
    assert sum(p.numel() for p in m.parameters()) == KEYS[name + "_params"]
    # the same angle per channel and layer as the reference builds (convnext.py:111-114)
    sd = m.state_dict()
    for k, vals in KEYS[name + "_theta_sample"].items():
        assert np.allclose(sd[k].flatten()[:16].numpy(), np.array(vals, np.float32), rtol=0, atol=0), k


def _dense_kernel(conv):
    """(2pad+1)^2 dense kernel of an oriented conv: w[c,k] scatter-added at its rasterised offset."""
    C, K = conv.weight.shape[0], conv.weight.shape[-1]
    pad = K // 2
    dh, dw = o1d.offsets(conv.theta.detach().float().cpu().numpy().reshape(-1), K)
    w = conv.weight.detach().double().cpu().reshape(C, K).clone()
    if conv.add_identity:
        w[:, pad] += 1
    k2d = torch.zeros((C, 1, 2 * pad + 1, 2 * pad + 1), dtype=torch.float64)
    for c in range(C):
        for k in range(K):
            k2d[c, 0, dh[c, k] + pad, dw[c, k] + pad] += w[c, k]
    return k2d, pad


def _ref_conv(conv, x_nhwc):
    k2d, pad = _dense_kernel(conv)
    y = F.conv2d(x_nhwc.permute(0, 3, 1, 2), k2d.to(x_nhwc.device), conv.bias.double(), conv.stride, pad, 1,
                 conv.weight.shape[0])
    return y.permute(0, 2, 3, 1)


def _ref_forward(m, img):
    """Every layer of ConvNeXt1D in float64 PyTorch."""
    d = lambda t: t.double()
    ln = lambda mod, x: F.layer_norm(x, mod.normalized_shape, d(mod.weight), d(mod.bias), mod.eps)
    lin = lambda mod, x: F.linear(x, d(mod.weight), d(mod.bias))
    x = img.double().permute(0, 2, 3, 1)
    for i in range(4):
        ds = m.downsample_layers[i]
        if i == 0:
            x = lin(ds.pw1, x)
            x = F.gelu(ln(ds.norm1, _ref_conv(ds.dw1, x)))
            x = F.gelu(ln(ds.norm2, _ref_conv(ds.dw2, x)))
            x = ln(ds.norm3, lin(ds.pw2, x))
        else:
            x = ln(ds[0], x)
            x = F.conv2d(x.permute(0, 3, 1, 2), d(ds[1].weight), d(ds[1].bias), 2).permute(0, 2, 3, 1)
        for blk in m.stages[i]:
            first = blk.dwconv if hasattr(blk, "dwconv") else blk.dwconv1
            y = F.gelu(lin(blk.pwconv1, ln(blk.norm, _ref_conv(first, x))))
            if hasattr(blk, "dwconv2"):
                y = _ref_conv(blk.dwconv2, y)
            x = x + d(blk.gamma) * lin(blk.pwconv2, y)
    x = x.mean([1, 2])
    return F.linear(F.layer_norm(x, m.norm.normalized_shape, d(m.norm.weight), d(m.norm.bias), m.norm.eps),
                    d(m.head.weight), d(m.head.bias))


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["1d", "1dpp"])
def test_model_forward_matches_pytorch_restatement(variant):
    torch.manual_seed(0)
    torch.backends.cudnn.allow_tf32 = False        # the 2x2 downsampling convs would run in TF32
    torch.backends.cuda.matmul.allow_tf32 = False
    m = convnext1d.ConvNeXt1D(depths=(1, 1, 2, 1), dims=(32, 64, 96, 128), variant=variant, stem_dim1=16,
                              layer_scale_init_value=0.5, num_classes=10).cuda().eval()
    for p in m.parameters():                      # away from the near-zero init so errors show
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.1)
    img = torch.randn(2, 3, 64, 64, device="cuda")
    with torch.no_grad():
        out = m(img)
        ref = _ref_forward(m, img)
    err = float((out.double() - ref).abs().max() / ref.abs().max())
    assert err < 1e-4, err
