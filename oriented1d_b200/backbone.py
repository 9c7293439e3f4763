"""Dense-prediction backbone and checkpoint conversion for ConvNeXt-1D / 1D++.

The reference's detection / segmentation backbones (``semantic_segmentation/backbone/
convnext.py:309-443``, the same file under ``object_detection``) differ from the classifier in
four ways, all restated here on top of :mod:`oriented1d_b200.convnext1d`:

* block kernels are cropped per stage — 1D: 31/31/27/13, 1D++: (15,31)/(15,31)/(15,27)/(13,13)
  (``:316-321``) — because a 31-tap line trained at 7x7 or 14x14 resolution has taps that never
  saw data (``README.md:137-142``);
* every oriented conv is built with ``arbitrary_size=True`` and wrapped so that its state-dict
  keys read ``...dwconv.conv.weight`` (``:74-103``);
* there is no classifier head; each requested stage output goes through its own channels-first
  LayerNorm ``norm{i}`` (``:395-399``, ``:433-443``);
* ``forward`` returns the tuple of stage maps (NCHW).

``convert_classifier_state_dict`` is what ``scripts/convert_to_backbone_weights.py:42-55`` is
meant to do (as shipped it calls an undefined ``reshape_kernel`` and stores the cropped tensor
under the old key): rename the oriented convs' keys, centre-crop their kernels to the
backbone's lengths, drop the head.
"""
from __future__ import annotations

import re

import torch
import torch.nn as nn

from .convnext1d import ConvNeXt1D, LayerNorm
from .dwoconv1d import DepthwiseOrientedConv1d

__all__ = ["ConvNeXt1DBackbone", "backbone_tiny", "backbone_base", "convert_classifier_state_dict",
           "BACKBONE_BLOCK_KERNELS", "BACKBONE_STEM_KERNEL"]

BACKBONE_BLOCK_KERNELS = {"2d": [[7], [7], [7], [7]],                           # backbone/convnext.py:315-320
                          "2dpp": [[7, 31], [7, 31], [7, 27], [7, 13]],
                          "1d": [[31], [31], [27], [13]],
                          "1dpp": [[15, 31], [15, 31], [15, 27], [13, 13]]}
BACKBONE_STEM_KERNEL = {"2d": 4, "2dpp": 4, "1d": 31, "1dpp": 15}               # backbone/convnext.py:321-326


class ConvWrapper(nn.Module):
    """backbone/convnext.py:74-80: gives the conv's parameters the ``.conv.`` key prefix."""

    def __init__(self, conv):
        super().__init__()
        self.conv = conv

    def forward(self, x):
        return self.conv(x)


def _wrap_convs(module):
    for name, child in list(module.named_children()):
        if isinstance(child, DepthwiseOrientedConv1d):
            setattr(module, name, ConvWrapper(child))
        else:
            _wrap_convs(child)


class ConvNeXt1DBackbone(ConvNeXt1D):
    """backbone/convnext.py:329-447, every variant: images [N,3,H,W] of any size
    -> tuple of normalised stage maps [N,C_i,ceil(H/4/2^i),ceil(W/4/2^i)] for i in out_indices."""

    def __init__(self, in_chans=3, depths=(3, 3, 9, 3), dims=(96, 192, 384, 768), drop_path_rate=0.0,
                 layer_scale_init_value=1e-6, out_indices=(0, 1, 2, 3), variant="1d", N=8, stem_dim1=64):
        super().__init__(in_chans=in_chans, num_classes=1, depths=depths, dims=dims, drop_path_rate=drop_path_rate,
                         layer_scale_init_value=layer_scale_init_value, variant=variant, N=N, stem_dim1=stem_dim1,
                         arbitrary_size=True, block_kernels=BACKBONE_BLOCK_KERNELS[variant],
                         stem_kernel=BACKBONE_STEM_KERNEL[variant])
        del self.norm, self.head
        _wrap_convs(self)
        self.out_indices = tuple(out_indices)
        for i in range(4):
            self.add_module(f"norm{i}", LayerNorm(dims[i], eps=1e-6, data_format="channels_first"))

    def forward_features(self, x, all_stages=True):
        outs = []
        for i in range(4):
            x = self.downsample_layers[i](x, nchw_input=True) if i == 0 else self.downsample_layers[i](x)
            x = self.stages[i](x)
            if i in self.out_indices:
                outs.append(getattr(self, f"norm{i}")(x).permute(0, 3, 1, 2))
        return tuple(outs)

    def forward(self, x):
        return self.forward_features(x)


def backbone_tiny(variant="1d", **kw):
    return ConvNeXt1DBackbone(depths=(3, 3, 9, 3), dims=(96, 192, 384, 768), variant=variant, **kw)


def backbone_base(variant="1d", **kw):
    return ConvNeXt1DBackbone(depths=(3, 3, 27, 3), dims=(128, 256, 512, 1024), variant=variant, **kw)


_DW_KEY = re.compile(r"^(.*\.(dw1|dw2|dwconv|dwconv1|dwconv2))\.(weight|bias|theta)$")
_STAGE_KEY = re.compile(r"^stages\.(\d+)\.\d+\.(dwconv|dwconv1|dwconv2)\.weight$")


def convert_classifier_state_dict(state_dict, variant="1d"):
    """Classifier checkpoint -> backbone checkpoint (scripts/convert_to_backbone_weights.py:42-55).

    ``state_dict`` may be the checkpoint itself or hold the weights under ``"model"`` (main.py saves
    that way).  Oriented-conv keys gain ``.conv.``; ``[C,1,1,K]`` kernels longer than the backbone's
    are cropped to their centre taps (tap k of the short kernel is tap k + (K-K')/2 of the long one,
    so the line keeps its offsets); ``head.*`` and the classifier's final ``norm.*`` are dropped.
    The backbone's ``norm0..3`` are not in a classifier checkpoint: load with ``strict=False``."""
    sd = state_dict.get("model", state_dict)
    kernels = BACKBONE_BLOCK_KERNELS[variant]
    out = {}
    for key, val in sd.items():
        if key.startswith("head.") or key.startswith("norm."):
            continue
        m = _DW_KEY.match(key)
        if not m:
            out[key] = val
            continue
        new_key = f"{m.group(1)}.conv.{m.group(3)}"
        s = _STAGE_KEY.match(key)
        if val.dim() == 4 and val.shape[2] != 1:          # a 7x7 depthwise conv of the 2D / 2D++ blocks: not wrapped
            out[key] = val
            continue
        if s and val.dim() == 4 and val.shape[2] == 1:
            want = kernels[int(s.group(1))][1 if s.group(2) == "dwconv2" else 0]
            have = val.shape[-1]
            if have < want:
                raise ValueError(f"{key}: kernel of {have} taps cannot fill the backbone's {want}")
            lo = (have - want) // 2
            val = val[..., lo:lo + want].clone()
        out[new_key] = val
    return out
