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
                                                  ("base_1dpp", convnext1d.convnext_base, "1dpp"),
                                                  ("tiny_2dpp", convnext1d.convnext_tiny, "2dpp"),
                                                  ("tiny_2d", convnext1d.convnext_tiny, "2d")])
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
    """(2pad+1)^2 dense kernel of an oriented conv: w[c,k] scatter-added at its rasterised offset
    (differentiable with respect to conv.weight)."""
    C, K = conv.weight.shape[0], conv.weight.shape[-1]
    pad = K // 2
    dh, dw = o1d.offsets(conv.theta.detach().float().cpu().numpy().reshape(-1), K)
    w = conv.weight.double().reshape(C, K)
    if conv.add_identity:
        eye = torch.zeros((C, K), dtype=torch.float64, device=w.device)
        eye[:, pad] = 1
        w = w + eye
    ci = torch.arange(C).repeat_interleave(K).to(w.device)
    ri = torch.from_numpy(np.ascontiguousarray(dh, dtype=np.int64)).reshape(-1).to(w.device) + pad
    qi = torch.from_numpy(np.ascontiguousarray(dw, dtype=np.int64)).reshape(-1).to(w.device) + pad
    k2d = torch.zeros((C, 1, 2 * pad + 1, 2 * pad + 1), dtype=torch.float64, device=w.device)
    k2d = k2d.index_put((ci, torch.zeros_like(ci), ri, qi), w.reshape(-1), accumulate=True)
    return k2d, pad


def _ref_conv(conv, x_nhwc):
    if not isinstance(conv, o1d.DepthwiseOrientedConv1d):        # the 7x7 depthwise conv of the 2D / 2D++ blocks
        y = F.conv2d(x_nhwc.permute(0, 3, 1, 2), conv.weight.double(), conv.bias.double(), conv.stride,
                     conv.padding, 1, conv.groups)
        return y.permute(0, 2, 3, 1)
    k2d, pad = _dense_kernel(conv)
    y = F.conv2d(x_nhwc.permute(0, 3, 1, 2), k2d, conv.bias.double(), conv.stride, pad, 1,
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
        if i == 0 and not hasattr(ds, "pw1"):                    # 4x4 patchify stem (convnext.py:525-529)
            x = F.conv2d(x.permute(0, 3, 1, 2), d(ds[0].weight), d(ds[0].bias), 4).permute(0, 2, 3, 1)
            x = ln(ds[1], x)
        elif i == 0:
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
@pytest.mark.parametrize("variant", ["1d", "1dpp", "2dpp"])
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


@pytest.mark.gpu
@pytest.mark.parametrize("variant,fuse", [("1dpp", True), ("2dpp", True), ("1dpp", "auto")])
def test_fused_gelu_model_equals_unfused(variant, fuse):
    """fuse_gelu=True moves the GELU in front of each block's second conv into that conv's kernels; the
    model's output and every gradient must not change beyond rounding."""
    torch.manual_seed(3)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    kw = dict(depths=(1, 1, 1, 1), dims=(32, 64, 96, 128), variant=variant, stem_dim1=16, layer_scale_init_value=0.5,
              num_classes=10)
    a = convnext1d.ConvNeXt1D(**kw).cuda().train()
    for p in a.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.1)
    b = convnext1d.ConvNeXt1D(fuse_gelu=fuse, **kw).cuda().train()
    b.load_state_dict(a.state_dict())
    side = 128 if fuse == "auto" else 64       # "auto" fuses on maps of 28x28 and more: stage 1 at 32x32
    img = torch.randn(2, 3, side, side, device="cuda")
    target = torch.randn(2, 10, device="cuda")
    outs = []
    for m in (a, b):
        out = m(img)
        (out * target).sum().backward()
        outs.append(out.detach())
    assert float((outs[0] - outs[1]).abs().max()) <= 1e-4 * float(outs[0].abs().max())
    ga, gb = dict(a.named_parameters()), dict(b.named_parameters())
    for k, p in ga.items():
        if p.grad is None:
            assert gb[k].grad is None
            continue
        err = float((p.grad - gb[k].grad).abs().max() / p.grad.abs().max().clamp_min(1e-30))
        assert err < 5e-4, (k, err)


@pytest.mark.gpu
@pytest.mark.parametrize("variant", ["1d", "1dpp", "2dpp"])
def test_model_training_step_gradients(variant):
    """Forward + backward through the autograd function of every oriented conv in the model
    (stride-2 stems, identity-tap convs of 1D++, every stage size): gradients of all parameters
    and of the input against float64 autograd through the PyTorch restatement."""
    torch.manual_seed(1)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    m = convnext1d.ConvNeXt1D(depths=(1, 1, 1, 1), dims=(32, 64, 96, 128), variant=variant, stem_dim1=16,
                              layer_scale_init_value=0.5, num_classes=10).cuda().train()
    for p in m.parameters():
        if p.dim() > 1:
            torch.nn.init.normal_(p, std=0.1)
    img = torch.randn(2, 3, 64, 64, device="cuda", requires_grad=True)
    target = torch.randn(2, 10, device="cuda")
    (m(img) * target).sum().backward()
    got = {k: p.grad.double().clone() for k, p in m.named_parameters() if p.grad is not None}
    got_img = img.grad.double().clone()
    assert not any(k.endswith("theta") for k in got)              # angles never receive a gradient
    m.zero_grad(set_to_none=True)
    img.grad = None
    (_ref_forward(m, img) * target.double()).sum().backward()
    for k, p in m.named_parameters():
        if k.endswith("theta"):
            continue
        ref = p.grad.double()
        err = float((got[k] - ref).abs().max() / ref.abs().max().clamp_min(1e-30))
        assert err < 5e-4, (k, err)
    err = float((got_img - img.grad.double()).abs().max() / img.grad.abs().max())
    assert err < 5e-4, err
