"""torch-facing wrappers of the C ABI: tensors in, tensors out.

torch is used for device memory (its caching allocator owns every buffer) and for the
current stream; all arithmetic happens in libo1d.so.  There is no CPU path: every
function raises on a non-CUDA tensor, as the reference's extension does
(CHECK_CUDA, models/dwoconv1d/kernels/kernels.cu:11).
"""
from __future__ import annotations

import numpy as np
import torch

from . import _lib
from ._lib import lib, check

# kernels launched by one call of each entry point (used by the benchmark's launch count)
KERNELS_PER_CALL = {"fprop": 1, "dgrad": 1, "wgrad": 2, "transpose": 1}

_DTYPES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


def _dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"oriented1d_b200 supports float32 and bfloat16 tensors, got {t.dtype}") from None


def _need_cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("tensor must be a CUDA tensor (oriented1d_b200 has no CPU path)")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def offsets(theta, K: int):
    """Rasterised tap offsets (dh, dw), int8 arrays [C, K], from fp32 angles
    (reference rule: models/dwoconv1d_reference/kernels/kernels.cpp:37,43-44)."""
    th = np.ascontiguousarray(np.asarray(theta, dtype=np.float32).reshape(-1))
    C = th.shape[0]
    dh = np.empty((C, K), np.int8)
    dw = np.empty((C, K), np.int8)
    check(lib.o1d_offsets(th.ctypes.data, C, K, dh.ctypes.data, dw.ctypes.data), "o1d_offsets")
    return dh, dw


class Plan:
    """Per-layer tap table (orientation classes) on the host plus one copy per device."""

    def __init__(self, theta, K: int):
        th = torch.as_tensor(theta).detach().to(device="cpu", dtype=torch.float32).reshape(-1).contiguous()
        self.C, self.K = int(th.numel()), int(K)
        nbytes = lib.o1d_plan_bytes(self.C, self.K)
        if nbytes == 0:
            raise ValueError("o1d_plan_bytes: invalid C or K")
        self.host = torch.zeros(nbytes, dtype=torch.uint8)
        check(lib.o1d_plan_build(th.data_ptr(), self.C, self.K, self.host.data_ptr()), "o1d_plan_build")
        self.num_classes = lib.o1d_plan_num_classes(self.host.data_ptr())
        self._dev: dict[torch.device, torch.Tensor] = {}

    def on(self, device: torch.device) -> torch.Tensor:
        d = self._dev.get(device)
        if d is None:
            d = self.host.to(device)
            self._dev[device] = d
        return d


def _dims(t: torch.Tensor, nhwc: bool):
    if t.dim() != 4:
        raise ValueError("expected a 4-D tensor")
    if nhwc:
        n, h, w, c = t.shape
    else:
        n, c, h, w = t.shape
    return n, c, h, w


def _check_params(plan: Plan, C: int, w=None, bias=None) -> None:
    """The kernels index w as [C, K] and bias as [C]: a shorter buffer would be read past its end."""
    if plan.C != C:
        raise ValueError(f"plan was built for {plan.C} channels, tensor has {C}")
    if w is not None and w.numel() != C * plan.K:
        raise ValueError(f"weight has {w.numel()} elements, expected C*K = {C * plan.K}")
    if bias is not None and bias.numel() != C:
        raise ValueError(f"bias has {bias.numel()} elements, expected C = {C}")


def fprop(x, w, bias, plan: Plan, stride: int = 1, nhwc: bool = False, add_identity: bool = False,
          gelu_input: bool = False):
    """y = oriented conv of x.  x: [N,C,H,W] (or [N,H,W,C] if nhwc), contiguous.  gelu_input: x is a
    pre-activation tensor and exact GELU is applied as it is loaded, y = conv(GELU(x))."""
    N, C, H, W = _dims(x, nhwc)
    K = plan.K
    _check_params(plan, C, w, bias)
    _need_cuda(x, w, bias)
    x = x.contiguous()
    w32 = w.detach().reshape(C, K).to(torch.float32).contiguous()
    b32 = bias.detach().to(torch.float32).contiguous() if bias is not None else None
    P, Q = -(-H // stride), -(-W // stride)
    y = torch.empty((N, P, Q, C) if nhwc else (N, C, P, Q), dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.o1d_fprop(x.data_ptr(), w32.data_ptr(), b32.data_ptr() if b32 is not None else None,
                            plan.host.data_ptr(), plan.on(x.device).data_ptr(), y.data_ptr(),
                            N, H, W, C, K, stride, int(nhwc), _dtype_code(x),
                            int(bool(add_identity)) * _lib.FLAG_IDENTITY + int(bool(gelu_input)) * _lib.FLAG_GELU_INPUT,
                            _stream()), "o1d_fprop")
    return y


def dgrad(dy, w, plan: Plan, H: int, W: int, stride: int = 1, nhwc: bool = False,
          add_identity: bool = False, pre=None):
    """dx [.., H, W ..] from dy [.., ceil(H/s), ceil(W/s) ..].  pre (shape of dx): the forward pass was
    conv(GELU(pre)); the result is then the gradient with respect to pre (times GELU'(pre))."""
    N, C, P, Q = _dims(dy, nhwc)
    if P != -(-H // stride) or Q != -(-W // stride):
        raise ValueError("dy extents do not match ceil(H/stride) x ceil(W/stride)")
    K = plan.K
    _check_params(plan, C, w)
    _need_cuda(dy, w)
    dy = dy.contiguous()
    w32 = w.detach().reshape(C, K).to(torch.float32).contiguous()
    dx = torch.empty((N, H, W, C) if nhwc else (N, C, H, W), dtype=dy.dtype, device=dy.device)
    if pre is not None:
        if tuple(pre.shape) != tuple(dx.shape) or pre.dtype != dy.dtype:
            raise ValueError("pre must have the shape and dtype of dx")
        _need_cuda(pre)
        pre = pre.contiguous()
    with torch.cuda.device(dy.device):
        check(lib.o1d_dgrad_act(dy.data_ptr(), w32.data_ptr(), pre.data_ptr() if pre is not None else None,
                                plan.host.data_ptr(), plan.on(dy.device).data_ptr(), dx.data_ptr(), N, H, W, C, K,
                                stride, int(nhwc), _dtype_code(dy), int(bool(add_identity)), _stream()),
              "o1d_dgrad")
    return dx


def wgrad(dy, x, plan: Plan, stride: int = 1, nhwc: bool = False, with_bias: bool = False,
          gelu_input: bool = False):
    """(dw [C,1,1,K] fp32, db [C] fp32 or None).  Deterministic.  gelu_input: x is the pre-activation
    tensor of a forward pass conv(GELU(x))."""
    if dy.dtype != x.dtype:
        raise TypeError("dy and x must have the same dtype")
    N, C, H, W = _dims(x, nhwc)
    K = plan.K
    _check_params(plan, C)
    P, Q = -(-H // stride), -(-W // stride)
    if tuple(dy.shape) != ((N, P, Q, C) if nhwc else (N, C, P, Q)):
        raise ValueError(f"dy has shape {tuple(dy.shape)}, expected the output shape of x "
                         f"({(N, P, Q, C) if nhwc else (N, C, P, Q)})")
    _need_cuda(dy, x)
    dy, x = dy.contiguous(), x.contiguous()
    code = _dtype_code(x)
    dw = torch.empty((C, 1, 1, K), dtype=torch.float32, device=x.device)
    db = torch.empty((C,), dtype=torch.float32, device=x.device) if with_bias else None
    nbytes = lib.o1d_wgrad_workspace_bytes(N, H, W, C, K, stride, int(nhwc), code)
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.o1d_wgrad_act(dy.data_ptr(), x.data_ptr(), plan.host.data_ptr(),
                                plan.on(x.device).data_ptr(), dw.data_ptr(),
                                db.data_ptr() if db is not None else None, ws.data_ptr(), ws.numel(),
                                N, H, W, C, K, stride, int(nhwc), code,
                                _lib.FLAG_GELU_INPUT if gelu_input else 0, _stream()), "o1d_wgrad")
    return dw, db


def _transpose(t: torch.Tensor, n: int, a: int, b: int, out_shape):
    _need_cuda(t)
    t = t.contiguous()
    out = torch.empty(out_shape, dtype=t.dtype, device=t.device)
    with torch.cuda.device(t.device):
        check(lib.o1d_transpose(t.data_ptr(), out.data_ptr(), n, a, b, _dtype_code(t), _stream()),
              "o1d_transpose")
    return out


def nhwc_to_nchw(x):
    """[N,H,W,C] -> [N,C,H,W], contiguous (reference: kernels.cu:56-61)."""
    N, H, W, C = x.shape
    return _transpose(x, N, H * W, C, (N, C, H, W))


def nchw_to_nhwc(x):
    """[N,C,H,W] -> [N,H,W,C], contiguous (reference: kernels.cu:63-68)."""
    N, C, H, W = x.shape
    return _transpose(x, N, C, H * W, (N, H, W, C))


def layer_norm_cl(x, weight, bias, eps: float = 1e-6, gelu: bool = False):
    """LayerNorm over the last (contiguous) axis, optionally fused with exact GELU.  Forward
    only (no autograd): for inference and for callers that handle gradients themselves."""
    _need_cuda(x, weight, bias)
    x = x.contiguous()
    C = x.shape[-1]
    rows = x.numel() // C
    y = torch.empty_like(x)
    g32 = weight.detach().to(torch.float32).contiguous()
    b32 = bias.detach().to(torch.float32).contiguous()
    with torch.cuda.device(x.device):
        check(lib.o1d_layernorm_cl(x.data_ptr(), g32.data_ptr(), b32.data_ptr(), y.data_ptr(), rows, C, float(eps),
                                   _dtype_code(x), int(gelu), _stream()), "o1d_layernorm_cl")
    return y


def layer_norm_cl_supported(x, gelu: bool = False, backward: bool = False) -> bool:
    """Can layer_norm_cl (and, with backward=True, layer_norm_cl_bwd) take this tensor?"""
    if not (x.is_cuda and x.dtype in (torch.float32, torch.bfloat16)):
        return False
    C, ve = x.shape[-1], (4 if x.dtype == torch.float32 else 8)
    if backward:
        return C % ve == 0 and C // ve <= 128
    return C % ve == 0 and C <= 1024


def layer_norm_cl_bwd(x, dy, weight, eps: float = 1e-6, bias=None, gelu: bool = False):
    """Gradients of layer_norm_cl: dx in x's dtype, dweight and dbias in fp32.  With gelu=True the
    forward call ended in exact GELU and `bias` is needed again.  The statistics are recomputed
    from x; dweight / dbias are summed in a fixed order."""
    _need_cuda(x, dy, weight)
    x, dy = x.contiguous(), dy.contiguous()
    if dy.shape != x.shape or dy.dtype != x.dtype:
        raise ValueError(f"dy {tuple(dy.shape)} {dy.dtype} does not match x {tuple(x.shape)} {x.dtype}")
    C = x.shape[-1]
    if weight.numel() != C:
        raise ValueError(f"weight has {weight.numel()} elements, expected {C}")
    rows = x.numel() // C
    dx = torch.empty_like(x)
    g32 = weight.detach().to(torch.float32).contiguous()
    if gelu and (bias is None or bias.numel() != C):
        raise ValueError("gelu=True needs the forward call's bias")
    b32 = bias.detach().to(torch.float32).contiguous() if gelu else None
    dg = torch.empty((C,), dtype=torch.float32, device=x.device)
    db = torch.empty((C,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        nbytes = lib.o1d_layernorm_cl_bwd_workspace_bytes(rows, C)
        ws = torch.empty((max(nbytes, 4),), dtype=torch.uint8, device=x.device)
        check(lib.o1d_layernorm_cl_bwd(x.data_ptr(), dy.data_ptr(), g32.data_ptr(), b32.data_ptr() if gelu else None,
                                       dx.data_ptr(), dg.data_ptr(), db.data_ptr(), ws.data_ptr(), nbytes, rows, C,
                                       float(eps), _dtype_code(x), int(gelu), _stream()), "o1d_layernorm_cl_bwd")
    return dx, dg, db


class LayerNormCL(torch.autograd.Function):
    """Channels-last LayerNorm with this library's kernels on both passes (F.layer_norm and its
    autograd backward in the reference, models/convnext.py:28-56)."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps, gelu=False):
        x = x.contiguous()
        ctx.save_for_backward(x, weight, bias)
        ctx.eps, ctx.gelu = eps, bool(gelu)
        return layer_norm_cl(x, weight, bias, eps, gelu)

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        dx, dg, db = layer_norm_cl_bwd(x, dy, weight, ctx.eps, bias, ctx.gelu)
        return (dx if ctx.needs_input_grad[0] else None, dg.to(weight.dtype) if ctx.needs_input_grad[1] else None,
                db.to(bias.dtype) if ctx.needs_input_grad[2] else None, None, None)


def colsum(x):
    """Sum over all but the last (contiguous) axis, in fp32 and in a fixed order: [..., C] -> [C]."""
    _need_cuda(x)
    x = x.contiguous()
    C = x.shape[-1]
    rows = x.numel() // C
    out = torch.empty((C,), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        code = _dtype_code(x)
        nbytes = lib.o1d_colsum_workspace_bytes(rows, C, code)
        ws = torch.empty((max(nbytes, 4),), dtype=torch.uint8, device=x.device)
        check(lib.o1d_colsum(x.data_ptr(), out.data_ptr(), ws.data_ptr(), nbytes, rows, C, code, _stream()),
              "o1d_colsum")
    return out


class LinearCL(torch.autograd.Function):
    """F.linear on channels-last activations whose bias gradient is this library's column sum
    (autograd's own is a generic reduction that runs at a fifth of the memory rate on these
    shapes); the two matrix products stay with the GEMM library, as in nn.Linear."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        ctx.bias_dtype = bias.dtype if bias is not None else None
        return torch.nn.functional.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = (dy2 @ weight).reshape(x.shape)
        if ctx.needs_input_grad[1]:
            dw = dy2.t() @ x.reshape(-1, x.shape[-1])
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = colsum(dy2).to(ctx.bias_dtype)
        return dx, dw, db


def linear_cl(module, x):
    """module(x) for an nn.Linear; on CUDA with gradients enabled the bias gradient runs here."""
    C = module.out_features
    if (x.is_cuda and torch.is_grad_enabled() and module.bias is not None and x.dtype == module.weight.dtype
            and x.dtype in (torch.float32, torch.bfloat16) and C % (4 if x.dtype == torch.float32 else 8) == 0):
        return LinearCL.apply(x, module.weight, module.bias)
    return module(x)


def pointwise_in(x, weight, bias):
    """Channels-last ``Linear`` over the few channels of an NCHW image: x [N,Cin,H,W] (Cin <= 4),
    weight [Cout,Cin], bias [Cout] or None -> [N,H,W,Cout] (models/convnext.py:143,170-176 in one
    pass).  Forward only."""
    _need_cuda(x, weight)
    x = x.contiguous()
    N, Cin, H, W = x.shape
    Cout = weight.shape[0]
    y = torch.empty((N, H, W, Cout), dtype=x.dtype, device=x.device)
    w32 = weight.detach().to(torch.float32).contiguous()
    b32 = None if bias is None else bias.detach().to(torch.float32).contiguous()
    with torch.cuda.device(x.device):
        check(lib.o1d_pointwise_in(x.data_ptr(), w32.data_ptr(), 0 if b32 is None else b32.data_ptr(), y.data_ptr(),
                                   N, Cin, H * W, Cout, _dtype_code(x), _stream()), "o1d_pointwise_in")
    return y


def uses_tiled(plan: Plan, N: int, H: int, W: int, stride: int, nhwc: bool, dtype: torch.dtype) -> bool:
    """Would this request run on the tiled kernels (True) or the general ones (False)?"""
    code = _DTYPES.get(dtype)
    if code is None:
        return False
    return bool(lib.o1d_uses_tiled(plan.host.data_ptr(), N, H, W, plan.C, plan.K, stride, int(nhwc), code))


def set_route(route) -> None:
    """Testing aid.  False/0: automatic choice; True/1: general kernels only; 2: prefer the
    tiled kernels; 3: prefer the direct kernels; 4: the whole-line kernels; 5: the walker kernels
    (the last two serve square fp32 NHWC stage maps only and fall through elsewhere)."""
    check(lib.o1d_set_route(int(route)), "o1d_set_route")


ROUTE_NAMES = {-1: "none", 0: "general", 1: "tiled", 2: "direct", 3: "plane7", 4: "lines", 5: "walk"}


def last_route() -> str:
    """Kernel family that served this thread's last fprop / dgrad / wgrad call."""
    return ROUTE_NAMES[lib.o1d_last_route()]


def device_status(device=None, clear: bool = False) -> int:
    """Device-side failure flag (0 = healthy).  Synchronises the device.  ``clear`` resets it."""
    import ctypes
    flag = ctypes.c_int(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        if clear:
            check(lib.o1d_device_status_clear(ctypes.byref(flag)), "o1d_device_status_clear")
        else:
            check(lib.o1d_device_status(ctypes.byref(flag)), "o1d_device_status")
    return flag.value
