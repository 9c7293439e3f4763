"""Drop-in for the reference's operator module.

Mirrors ``models/dwoconv1d/dwoconv1d.py`` (and ``models/dwoconv1d_specialized/
dwoconv1d_specialized.py``, whose public surface is identical): the same
``DepthwiseOrientedConv1d(nn.Conv2d)`` constructor, ``forward`` / ``forward_safe``,
autograd contract and state-dict layout (``weight [C,1,1,K]``, ``bias [C]``,
``theta [C]`` or ``[C,1]``), so ``models/convnext.py`` can import it under the name
``dwoconv1d`` or ``dwoconv1d_specialized`` (see ``oriented1d_b200/compat``).

What differs underneath:

* kernels are prebuilt (``libo1d.so``); nothing is compiled in the constructor
  (reference: dwoconv1d.py:144-152 JIT-compiles one module per template tuple);
* NHWC inputs are convolved in place — no nhwc_to_nchw / nchw_to_nhwc round trips
  (reference: dwoconv1d.py:25-26,36-37,50-51,58-59);
* bias add and the ``w + resid`` identity tap are fused into the kernels
  (reference: dwoconv1d.py:22-23,34-35) and ``db`` comes out of the weight-gradient
  kernel (reference: dwoconv1d.py:66-67);
* any H x W is handled natively, so ``forward_safe`` does not pad to powers of two
  (reference: dwoconv1d.py:154-187); results are identical because the padding is zeros;
* float32 and bfloat16 activations (the reference is float32 only, dwoconv1d.py:144-146).
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops

__all__ = ["DepthwiseOrientedConv1d", "get_dwoconv1d_kernel", "oriented_dwconv1d_get_module_from_params"]


class _DepthwiseOrientedConv1d(torch.autograd.Function):
    """Counterpart of the reference's autograd function (dwoconv1d.py:18-69).

    NCHW inputs whose NHWC form qualifies for the tiled kernels are converted once on the
    way in and out (two 128-bit transposes cost far less than the general NCHW kernels); the
    NHWC copy of x is what is saved for backward.  The reference does the opposite: it
    converts NHWC inputs to NCHW around NCHW-only kernels (dwoconv1d.py:25-26,36-37)."""

    @staticmethod
    def forward(ctx, x, w, theta, bias, plan, stride, nhwc=False, add_identity=False, gelu_input=False):
        x = x.contiguous()
        ctx.set_materialize_grads(False)
        ctx.gelu_input = gelu_input
        via_nhwc = False
        if not nhwc and not gelu_input and x.is_cuda and x.dim() == 4:
            N, C, H, W = x.shape
            via_nhwc = (ops.uses_tiled(plan, N, H, W, stride, True, x.dtype)
                        and not ops.uses_tiled(plan, N, H, W, stride, False, x.dtype))
        ctx.plan, ctx.stride, ctx.nhwc, ctx.add_identity = plan, stride, nhwc, add_identity
        ctx.via_nhwc = via_nhwc
        ctx.has_bias = bias is not None
        if via_nhwc:
            xh = ops.nchw_to_nhwc(x)
            ctx.save_for_backward(xh, w)
            return ops.nhwc_to_nchw(ops.fprop(xh, w, bias, plan, stride, True, add_identity))
        ctx.save_for_backward(x, w)
        return ops.fprop(x, w, bias, plan, stride, nhwc, add_identity, gelu_input)

    @staticmethod
    def backward(ctx, dy):
        if dy is None:
            return None, None, None, None, None, None, None, None, None
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        if dy.dtype != x.dtype:
            dy = dy.to(x.dtype)
        nhwc = ctx.nhwc or ctx.via_nhwc           # layout of the saved x and of the kernels
        if ctx.via_nhwc:
            dy = ops.nchw_to_nhwc(dy)
        dx = dw = db = None
        if nhwc:
            H, W = x.shape[1], x.shape[2]
        else:
            H, W = x.shape[2], x.shape[3]
        if ctx.needs_input_grad[0]:
            dx = ops.dgrad(dy, w, ctx.plan, H, W, ctx.stride, nhwc, ctx.add_identity,
                           pre=x if ctx.gelu_input else None)
            if ctx.via_nhwc:
                dx = ops.nhwc_to_nchw(dx)
        need_db = ctx.has_bias and ctx.needs_input_grad[3]
        if ctx.needs_input_grad[1] or need_db:
            dw, db = ops.wgrad(dy, x, ctx.plan, ctx.stride, nhwc, with_bias=need_db, gelu_input=ctx.gelu_input)
            dw = dw.to(w.dtype) if ctx.needs_input_grad[1] else None
            # bias shares the weight's dtype in an nn.Conv2d
            db = db.to(w.dtype) if need_db else None
        return dx, dw, None, db, None, None, None, None, None


class DepthwiseOrientedConv1d(nn.Conv2d):
    """Oriented 1D depthwise convolution (reference: dwoconv1d.py:92-198).

    ``angle`` is a scalar or a per-channel list in radians.  The kernels use
    ``pad = kernel_size // 2`` regardless of ``padding`` (reference: dwoconv1d.py:133,
    144-146); ``padding`` only lands in ``nn.Conv2d.padding``.
    """

    def __init__(self, in_channels, out_channels, kernel_size=3, *, groups=1, stride=1, padding=1,
                 bias=True, angle=0, nhwc=False, resid=False, arbitrary_size=False):
        super().__init__(in_channels, out_channels, (1, kernel_size), groups=groups, stride=stride,
                         padding=(0, padding), bias=bias)
        assert (isinstance(kernel_size, int) and in_channels == out_channels
                and groups == in_channels and kernel_size % 2 == 1)
        assert self.stride[0] == self.stride[1]

        if isinstance(angle, (float, int)):
            angle = torch.zeros((in_channels, 1)) + angle
        # same construction as the reference (dwoconv1d.py:128-131): python floats -> fp32
        self.theta = torch.nn.Parameter(torch.as_tensor(angle, dtype=torch.float32).clone()
                                        if isinstance(angle, torch.Tensor)
                                        else torch.tensor(angle, dtype=torch.float32))
        self.nhwc = nhwc
        self.add_identity = bool(resid)
        # Set by a caller whose input is a pre-activation tensor: forward then computes
        # conv(GELU(x)) with the GELU applied inside the kernels (the reference runs F.gelu as a
        # separate pass in front of its second block conv, models/convnext.py:389-391).  Not a
        # constructor argument: the reference's signature is kept as it is.  True: always inside
        # the kernels; "auto": inside the kernels where that saves time (large maps, which the
        # tiled kernels serve anyway), as a separate F.gelu pass elsewhere (small maps, where
        # the kernel families without activation-on-load are the faster ones).
        self.gelu_input = False
        # kept for parity with the reference attribute (dwoconv1d.py:136-141); the kernels
        # add the identity tap themselves and never read this tensor
        if resid:
            delta = torch.zeros_like(self.weight)
            delta[:, :, :, kernel_size // 2] = 1
            self.resid = delta
        else:
            self.resid = None
        # fp32 angles as constructed: rasterisation must not see a theta rounded by
        # .bfloat16()/.half() (bf16(pi/2) would move the end taps of a vertical line)
        self._angles_fp32 = self.theta.detach().clone().reshape(-1)
        self._plan = None
        self._plan_key = None
        self._plan_src = None
        if arbitrary_size:
            self.forward = self.forward_safe

    # -- plan cache -------------------------------------------------------------------
    def _get_plan(self) -> ops.Plan:
        th = self.theta
        # the key holds the tensor that backs the parameter: a new tensor swapped in through
        # `theta.data = ...` can then never reuse the old one's address while the plan lives
        key = (th._version, th.data_ptr(), th.dtype)
        if self._plan is None or key != self._plan_key or self._plan_src is not th.data.untyped_storage():
            self._plan_src = th.data.untyped_storage()
            if th.dtype == torch.float32:
                angles = th.detach().reshape(-1)
            else:
                kept = self._angles_fp32.to(th.device)
                same = torch.equal(kept.to(th.dtype), th.detach().reshape(-1))
                angles = kept if same else th.detach().reshape(-1).float()
            self._plan = ops.Plan(angles, self.kernel_size[1])
            self._plan_key = key
        return self._plan

    def _gelu_in_kernel(self, x) -> bool:
        """The "auto" rule: activation on load only on maps of 28x28 and larger that the tiled
        kernels serve anyway.  What it buys is memory (the GELU output is never stored, one 4*dim
        activation less per block kept for backward), not time: the tiled kernels are bound by
        instruction issue, so the erf costs more there than the memory pass it removes (B200,
        ConvNeXt-B-1D++ training step, batch 64: 60.3 ms unfused, 63.5 ms with this rule, 74.1 ms
        with the activation forced into every stage)."""
        if self.gelu_input != "auto":
            return bool(self.gelu_input)
        if not (x.is_cuda and x.dim() == 4 and self.nhwc and self.stride[0] == 1):
            return False
        N, H, W, _ = x.shape
        return H * W >= 28 * 28 and ops.uses_tiled(self._get_plan(), N, H, W, 1, True, x.dtype)

    def _apply_op(self, x):
        gelu = self._gelu_in_kernel(x)
        if self.gelu_input and not gelu:
            x = torch.nn.functional.gelu(x)
        return _DepthwiseOrientedConv1d.apply(x, self.weight, self.theta, self.bias, self._get_plan(),
                                              self.stride[0], self.nhwc, self.add_identity, gelu)

    def forward_safe(self, x):
        """Any H x W; output extents ceil(H/stride) x ceil(W/stride) (dwoconv1d.py:154-187)."""
        return self._apply_op(x)

    def forward(self, x):
        h, w = (x.shape[1], x.shape[2]) if self.nhwc else (x.shape[2], x.shape[3])
        if h % self.stride[0] or w % self.stride[0]:
            # reference: TORCH_CHECK in kernels.cu:19-20
            raise RuntimeError("Invalid input size: H,W not divisible by stride")
        return self._apply_op(x)


# --------------------------------------------------------------------------------------
# The 5-callable "extension module" surface of the reference loader
# (dwoconv1d_kernel.py:30-35,76-90): fprop(x,w,theta), dgrad(dy,w,theta),
# wgrad(dy,x,theta), nhwc_to_nchw(x), nchw_to_nhwc(x) on contiguous NCHW tensors with
# (K, stride, pad) fixed at creation.  Kept so either implementation can be swapped
# under the reference's autograd function.
# --------------------------------------------------------------------------------------
class _KernelModule:
    def __init__(self, kernel_size: int, stride: int, pad: int):
        if pad != kernel_size // 2:
            raise ValueError("pad must equal kernel_size // 2")
        self.K, self.stride = int(kernel_size), int(stride)
        self._plans: dict = {}

    def _plan(self, theta) -> ops.Plan:
        """Plan of these angles.  A cache entry keeps the storage of the tensor it was built from
        alive, so the allocator cannot hand that address to a later tensor with other angles;
        a hit therefore means the same memory at the same version, i.e. the same values."""
        key = (theta.data_ptr(), theta._version, theta.numel())
        hit = self._plans.get(key)
        if hit is not None:
            return hit[1]
        if len(self._plans) > 64:
            self._plans.clear()
        p = ops.Plan(theta, self.K)
        self._plans[key] = (theta.detach().untyped_storage(), p)
        return p

    def fprop(self, x, w, theta):
        if x.shape[2] % self.stride or x.shape[3] % self.stride:
            raise RuntimeError("Invalid input size: H,W not divisible by stride")
        return ops.fprop(x, w, None, self._plan(theta), self.stride, False, False)

    def dgrad(self, dy, w, theta):
        return ops.dgrad(dy, w, self._plan(theta), dy.shape[2] * self.stride, dy.shape[3] * self.stride,
                         self.stride, False, False)

    def wgrad(self, dy, x, theta):
        return ops.wgrad(dy, x, self._plan(theta), self.stride, False, False)[0]

    nhwc_to_nchw = staticmethod(ops.nhwc_to_nchw)
    nchw_to_nhwc = staticmethod(ops.nchw_to_nhwc)


_modules: dict = {}


def get_dwoconv1d_kernel(ftype, kernel_size, stride, pad, Sb=None, verbose=False):
    """Same call as the reference loader (dwoconv1d_kernel.py:76-90); ``Sb`` (tap
    chunking for shared-memory size) has no meaning here and is ignored."""
    if ftype != "float":
        raise ValueError("ftype must be 'float'")
    key = (int(kernel_size), int(stride), int(pad))
    if key not in _modules:
        _modules[key] = _KernelModule(*key)
    return _modules[key]


def oriented_dwconv1d_get_module_from_params(ftype, kernel_size, stride, pad, Sb=None):
    """5-tuple as in dwoconv1d.py:72-80."""
    m = get_dwoconv1d_kernel(ftype, kernel_size, stride, pad, Sb=Sb)
    return (m.fprop, m.dgrad, m.wgrad, m.nhwc_to_nchw, m.nchw_to_nhwc)
