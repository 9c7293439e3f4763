"""ConvNeXt-1D / 1D++ / 2D++ (and plain 2D) built on the oriented 1D depthwise convolution.

The caller side of the hot path: a timm-free restatement of the reference model
(``models/convnext.py``: angle helpers :60-77, ``get_convolution_1d`` :80-128, ``Stem1D``
:132-191, ``Block2D`` :195-252, ``Block1D`` :255-319, ``Block1DPP`` :322-399, ``Block2DPP``
:402-475, ``ConvNeXt`` :495-610, factories :613-644) with the same module tree and therefore the same state-dict keys and shapes
(``downsample_layers.0.dw1.weight [64,1,1,31]``, ``stages.0.0.dwconv.theta [96]`` ...), so
reference checkpoints load with ``load_state_dict``.

What differs is data movement only.  The reference keeps activations NCHW between blocks and
makes two full ``permute().contiguous()`` copies per block around the channels-last MLP
(``convnext.py:308,316``), and its NCHW kernels add two more transposes whenever a conv is
NHWC.  Here activations stay channels-last (NHWC) from the stem to the pooling: every
depthwise conv runs its native NHWC kernel, LayerNorm / Linear / GELU already want NHWC, and
the 2x2 stride-2 downsampling conv sees the same memory as a channels_last NCHW view.  The
arithmetic of every layer is unchanged.  Inputs and outputs keep the reference convention
(images ``[N,3,H,W]`` in, logits out).
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import ops
from .dwoconv1d import DepthwiseOrientedConv1d

__all__ = ["ConvNeXt1D", "convnext_tiny", "convnext_base", "get_convolution_1d"]

BLOCK_KERNELS = {"2d": [[7]] * 4, "2dpp": [[7, 31]] * 4, "1d": [[31]] * 4, "1dpp": [[15, 31]] * 4}   # convnext.py:483-488
STEM_KERNEL = {"2d": 4, "2dpp": 4, "1d": 31, "1dpp": 15}                                             # convnext.py:490


def channel_cycle_offset(c, C, N):
    """convnext.py:60-65: N groups of ~C/N channels, group n has angle n/N * 180 degrees."""
    return ((N * (c + 1) - 1) // C) / N


def layer_wise_rotation_offset(k, enable_layer_cycle=0):
    """convnext.py:68-72: +90 degrees on layers at odd depth."""
    return (k % 2) / 2 if enable_layer_cycle else 0


def get_convolution_1d(channels, *, kernel_size, padding, stride=1, N=8, layer_offset=0, nhwc=False,
                       resid=False, bias=True, arbitrary_size=False):
    """convnext.py:80-128."""
    theta = [math.pi * ((channel_cycle_offset(k, channels, N) + layer_offset) % 1) for k in range(channels)]
    return DepthwiseOrientedConv1d(channels, channels, kernel_size, groups=channels, stride=stride, nhwc=nhwc,
                                   resid=resid, padding=padding, bias=bias, angle=theta,
                                   arbitrary_size=arbitrary_size)


class LayerNorm(nn.Module):
    """LayerNorm over channels with the reference's parameter names (convnext.py:28-56).  The
    data here is always channels-last, for which the reference's channels_first formula and
    F.layer_norm are the same computation."""

    def __init__(self, normalized_shape, eps=1e-6, data_format="channels_last"):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(normalized_shape))
        self.bias = nn.Parameter(torch.zeros(normalized_shape))
        self.eps, self.data_format, self.normalized_shape = eps, data_format, (normalized_shape,)

    def forward(self, x, gelu=False):
        """gelu=True also applies exact GELU (the stem's LayerNorm -> GELU pairs)."""
        C = x.shape[-1]
        fast = (x.is_cuda and not torch.is_grad_enabled() and x.dtype in (torch.float32, torch.bfloat16)
                and C % (4 if x.dtype == torch.float32 else 8) == 0 and C <= 1024)
        if fast:      # inference: one pass over the tensor (see csrc/o1d_layernorm.cuh)
            return ops.layer_norm_cl(x, self.weight, self.bias, self.eps, gelu)
        if torch.is_grad_enabled() and ops.layer_norm_cl_supported(x, gelu, backward=True):
            return ops.LayerNormCL.apply(x, self.weight, self.bias, self.eps, gelu)   # training: both passes here
        y = F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)
        return F.gelu(y) if gelu else y


class Stem1D(nn.Module):
    """convnext.py:132-191; input and output channels-last."""

    def __init__(self, dim0, dim1, dim2, kernel_size, enable_layer_cycle=0, arbitrary_size=False):
        super().__init__()
        self.pw1 = nn.Linear(dim0, dim1)
        self.pw2 = nn.Linear(dim1, dim2)
        pad = (kernel_size - 2) // 2
        self.dw1 = get_convolution_1d(dim1, kernel_size=kernel_size, stride=2, padding=pad, nhwc=True,
                                      layer_offset=layer_wise_rotation_offset(0, enable_layer_cycle),
                                      arbitrary_size=arbitrary_size)
        self.dw2 = get_convolution_1d(dim1, kernel_size=kernel_size, stride=2, padding=pad, nhwc=True,
                                      layer_offset=layer_wise_rotation_offset(1, enable_layer_cycle),
                                      arbitrary_size=arbitrary_size)
        self.norm1 = LayerNorm(dim1)
        self.norm2 = LayerNorm(dim1)
        self.norm3 = LayerNorm(dim2)

    def forward(self, x, nchw_input=False):     # x: [N, H, W, 3], or the [N, 3, H, W] image itself
        if nchw_input:
            fast = (x.is_cuda and not torch.is_grad_enabled() and x.dtype in (torch.float32, torch.bfloat16)
                    and x.shape[1] <= 4 and self.pw1.out_features % 8 == 0)
            # inference: projection and layout change in one pass (see csrc/o1d_pointwise.cuh)
            x = ops.pointwise_in(x, self.pw1.weight, self.pw1.bias) if fast else self.pw1(x.permute(0, 2, 3, 1))
        else:
            x = self.pw1(x)
        x = self.norm1(self.dw1(x), gelu=True)
        x = self.norm2(self.dw2(x), gelu=True)
        return self.norm3(ops.linear_cl(self.pw2, x))


class Block1D(nn.Module):
    """convnext.py:255-319; channels-last in and out (no permute copies)."""

    def __init__(self, dim, kernel_sizes=(31,), N=8, drop_path=0.0, layer_scale_init_value=1e-6, layer_offset=0,
                 arbitrary_size=False):
        super().__init__()
        self.norm = LayerNorm(dim)
        self.pwconv1 = nn.Linear(dim, 4 * dim)
        self.pwconv2 = nn.Linear(4 * dim, dim)
        self.gamma = (nn.Parameter(layer_scale_init_value * torch.ones(dim)) if layer_scale_init_value > 0 else None)
        self.drop_path = drop_path
        # the reference builds this conv NCHW (nhwc=False, convnext.py:297); the flag is not part
        # of the checkpoint, and the data here is NHWC
        self.dwconv = get_convolution_1d(dim, kernel_size=kernel_sizes[0], padding=kernel_sizes[0] // 2, nhwc=True,
                                         N=N, layer_offset=layer_offset, arbitrary_size=arbitrary_size)

    def _mlp_in(self, x, gelu=True):
        h = ops.linear_cl(self.pwconv1, self.norm(x))
        return F.gelu(h) if gelu else h

    def forward(self, x):
        y = ops.linear_cl(self.pwconv2, self._mlp_in(self.dwconv(x)))
        return self._residual(x, y)

    def _residual(self, x, y):
        """x + drop_path(gamma * y) (convnext.py:314-318); one fused pass when nothing is dropped."""
        if self.drop_path == 0.0 or not self.training:
            return x + y if self.gamma is None else torch.addcmul(x, y, self.gamma)
        if self.gamma is not None:
            y = self.gamma * y
        return x + _drop_path(y, self.drop_path, self.training)


class Block1DPP(Block1D):
    """convnext.py:322-399: a second oriented conv (K=31, identity tap) on the 4*dim hidden tensor."""

    def __init__(self, dim, kernel_sizes=(15, 31), N=8, drop_path=0.0, layer_scale_init_value=1e-6,
                 layer_offset=0, arbitrary_size=False):
        super().__init__(dim, kernel_sizes[:1], N, drop_path, layer_scale_init_value, layer_offset, arbitrary_size)
        self.dwconv1 = self.dwconv                     # reference names: dwconv1, dwconv2
        del self.dwconv
        self.dwconv2 = get_convolution_1d(4 * dim, kernel_size=kernel_sizes[1], padding=kernel_sizes[1] // 2,
                                          nhwc=True, resid=True, N=N, layer_offset=layer_offset,
                                          arbitrary_size=arbitrary_size)

    def forward(self, x):
        fused = getattr(self.dwconv2, "gelu_input", False)      # the GELU then runs inside dwconv2's kernels
        y = ops.linear_cl(self.pwconv2, self.dwconv2(self._mlp_in(self.dwconv1(x), gelu=not fused)))
        return self._residual(x, y)


class Block2D(Block1D):
    """convnext.py:195-252: the plain ConvNeXt block (7x7 depthwise conv); channels-last in and out.
    The library conv runs on the NCHW view of the same memory (channels_last strides, no copy)."""

    def __init__(self, dim, kernel_sizes=(7,), N=0, drop_path=0.0, layer_scale_init_value=1e-6, layer_offset=0,
                 arbitrary_size=False):
        nn.Module.__init__(self)
        self.dwconv = nn.Conv2d(dim, dim, kernel_size=kernel_sizes[0], padding=kernel_sizes[0] // 2, groups=dim)
        self.norm = LayerNorm(dim)
        self.pwconv1 = nn.Linear(dim, 4 * dim)
        self.pwconv2 = nn.Linear(4 * dim, dim)
        self.gamma = (nn.Parameter(layer_scale_init_value * torch.ones(dim)) if layer_scale_init_value > 0 else None)
        self.drop_path = drop_path

    def _dw2d(self, conv, x):
        return conv(x.permute(0, 3, 1, 2)).permute(0, 2, 3, 1)

    def forward(self, x):
        y = ops.linear_cl(self.pwconv2, self._mlp_in(self._dw2d(self.dwconv, x)))
        return self._residual(x, y)


class Block2DPP(Block2D):
    """convnext.py:402-475: 7x7 depthwise conv, then the oriented conv (K=31, identity tap, NHWC) on
    the 4*dim hidden tensor."""

    def __init__(self, dim, kernel_sizes=(7, 31), N=8, drop_path=0.0, layer_scale_init_value=1e-6,
                 layer_offset=0, arbitrary_size=False):
        assert len(kernel_sizes) == 2
        super().__init__(dim, kernel_sizes[:1], N, drop_path, layer_scale_init_value, layer_offset, arbitrary_size)
        self.dwconv1 = self.dwconv                     # reference names: dwconv1, dwconv2
        del self.dwconv
        self.dwconv2 = get_convolution_1d(4 * dim, kernel_size=kernel_sizes[1], padding=kernel_sizes[1] // 2,
                                          nhwc=True, resid=True, N=N, layer_offset=layer_offset,
                                          arbitrary_size=arbitrary_size)

    def forward(self, x):
        fused = getattr(self.dwconv2, "gelu_input", False)
        y = self._mlp_in(self._dw2d(self.dwconv1, x), gelu=not fused).contiguous()
        return self._residual(x, ops.linear_cl(self.pwconv2, self.dwconv2(y)))


class Stem2D(nn.Sequential):
    """convnext.py:525-529: 4x4 stride-4 patchify conv + LayerNorm; image [N,3,H,W] in, channels-last out."""

    def __init__(self, cin, cout):
        super().__init__(nn.Conv2d(cin, cout, kernel_size=4, stride=4), LayerNorm(cout, data_format="channels_first"))

    def forward(self, x, nchw_input=True):
        if not nchw_input:
            x = x.permute(0, 3, 1, 2)
        return self[1](self[0](x).permute(0, 2, 3, 1).contiguous())


BLOCKS = {"2d": Block2D, "2dpp": Block2DPP, "1d": Block1D, "1dpp": Block1DPP}      # convnext.py:477-482


def _drop_path(y, rate, training):
    """Stochastic depth per sample (timm DropPath semantics, as used at convnext.py:292)."""
    if rate == 0.0 or not training:
        return y
    keep = 1.0 - rate
    mask = y.new_empty((y.shape[0],) + (1,) * (y.dim() - 1)).bernoulli_(keep)
    return y * mask / keep


class Downsample(nn.Sequential):
    """LayerNorm + 2x2 stride-2 conv (convnext.py:553-559), on channels-last data: the conv
    runs on the NCHW view of the same memory (channels_last strides, no copy)."""

    def __init__(self, cin, cout):
        super().__init__(LayerNorm(cin, data_format="channels_first"), nn.Conv2d(cin, cout, kernel_size=2, stride=2))

    def forward(self, x):                       # [N, H, W, C] -> [N, H/2, W/2, C']
        x = self[0](x)
        y = self[1](x.permute(0, 3, 1, 2))      # view; memory format channels_last
        return y.permute(0, 2, 3, 1).contiguous()     # contiguous already unless cuDNN chose NCHW


class ConvNeXt1D(nn.Module):
    """convnext.py:495-610, all four variants ("2d", "2dpp", "1d", "1dpp")."""

    def __init__(self, in_chans=3, num_classes=1000, depths=(3, 3, 9, 3), dims=(96, 192, 384, 768),
                 drop_path_rate=0.0, layer_scale_init_value=1e-6, head_init_scale=1.0, variant="1d", N=8,
                 stem_dim1=64, arbitrary_size=False, block_kernels=None, stem_kernel=None, fuse_gelu=False):
        super().__init__()
        assert variant in BLOCKS
        Block = BLOCKS[variant]
        block_kernels = BLOCK_KERNELS[variant] if block_kernels is None else block_kernels
        stem_kernel = STEM_KERNEL[variant] if stem_kernel is None else stem_kernel
        cycle = int(variant != "2d")                   # enable_layer_cycle, convnext.py:523
        stem = (Stem2D(in_chans, dims[0]) if variant in ("2d", "2dpp")
                else Stem1D(in_chans, stem_dim1, dims[0], stem_kernel, cycle, arbitrary_size))
        self.downsample_layers = nn.ModuleList([stem])
        for i in range(3):
            self.downsample_layers.append(Downsample(dims[i], dims[i + 1]))
        rates = torch.linspace(0, drop_path_rate, sum(depths)).tolist()
        self.stages = nn.ModuleList()
        cur = 0
        for i in range(4):
            self.stages.append(nn.Sequential(*[
                Block(dims[i], kernel_sizes=block_kernels[i], N=N, drop_path=rates[cur + j],
                      layer_scale_init_value=layer_scale_init_value,
                      layer_offset=layer_wise_rotation_offset(j, cycle), arbitrary_size=arbitrary_size)
                for j in range(depths[i])]))
            cur += depths[i]
        if fuse_gelu:      # 1D++ / 2D++: dwconv2 takes the pre-activation tensor (True or "auto")
            for m in self.modules():
                # only the operator module itself knows the flag (a wrapper for arbitrary sizes keeps the separate pass)
                if isinstance(m, (Block1DPP, Block2DPP)) and hasattr(m.dwconv2, "_apply_op"):
                    m.dwconv2.gelu_input = fuse_gelu
        self.norm = nn.LayerNorm(dims[-1], eps=1e-6)
        self.head = nn.Linear(dims[-1], num_classes)
        self.apply(self._init_weights)
        self.head.weight.data.mul_(head_init_scale)
        self.head.bias.data.mul_(head_init_scale)

    @staticmethod
    def _init_weights(m):
        if isinstance(m, (nn.Conv2d, nn.Linear)):           # the oriented conv is an nn.Conv2d too
            nn.init.trunc_normal_(m.weight, std=0.02)
            if m.bias is not None:
                nn.init.constant_(m.bias, 0)

    def forward_features(self, x, all_stages=False):
        """x: images [N, 3, H, W].  Returns the last stage's map [N, C, H/32, W/32] (NCHW view),
        or the four stage maps when all_stages is set (the dense-prediction backbones' outputs)."""
        outs = []
        for i in range(4):
            x = self.downsample_layers[i](x, nchw_input=True) if i == 0 else self.downsample_layers[i](x)
            x = self.stages[i](x)
            outs.append(x.permute(0, 3, 1, 2))
        return outs if all_stages else outs[-1]

    def forward(self, x):
        x = self.forward_features(x)
        return self.head(self.norm(x.mean([-2, -1])))


def convnext_tiny(variant="1d", drop_path_rate=0.1, **kw):
    """convnext.py:613-627."""
    return ConvNeXt1D(depths=(3, 3, 9, 3), dims=(96, 192, 384, 768), drop_path_rate=drop_path_rate, variant=variant, **kw)


def convnext_base(variant="1d", drop_path_rate=0.5, **kw):
    """convnext.py:630-644."""
    return ConvNeXt1D(depths=(3, 3, 27, 3), dims=(128, 256, 512, 1024), drop_path_rate=drop_path_rate,
                      variant=variant, **kw)
