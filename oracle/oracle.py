"""numpy front end of the CPU oracle.  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this
module; the package itself never does, and it has no CPU fallback.

``Oracle`` wraps the plain-C restatement (``o1d_oracle.c``); ``Reference`` wraps the
reference's own loops compiled from its checkout (``ref_shim.cpp``).  Both expose the
same calls on NCHW float32 arrays.  The module-level helpers restate what the
reference's Python wrapper does around the loops:

* ``module_forward`` / ``module_backward``: resid, layout and bias handling of
  ``_DepthwiseOrientedConv1d`` (models/dwoconv1d/dwoconv1d.py:20-69).
* ``forward_safe``: zero-pad to a power-of-two multiple, run, crop
  (models/dwoconv1d/dwoconv1d.py:154-187).
* ``model_angles``: the per-channel angle list of ``get_convolution_1d``
  (models/convnext.py:60-77, :111-114).
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_i32p = ctypes.POINTER(ctypes.c_int32)


def _p(a, ty=_f32p):
    return a.ctypes.data_as(ty)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class _Loops:
    """Shared call surface: fprop / dgrad / wgrad on NCHW float32."""

    _prefix = ""
    _lib = None

    def fprop(self, x, w, theta, stride=1):
        x, w, theta = _f32(x), _f32(w).reshape(x.shape[1], -1), _f32(theta).reshape(-1)
        N, C, H, W = x.shape
        K = w.shape[1]
        y = np.empty((N, C, H // stride, W // stride), np.float32)
        getattr(self._lib, self._prefix + "fprop")(_p(x), _p(w), _p(theta), _p(y), N, C, H, W, K, stride)
        return y

    def dgrad(self, dy, w, theta, stride=1):
        dy, w, theta = _f32(dy), _f32(w).reshape(dy.shape[1], -1), _f32(theta).reshape(-1)
        N, C, P, Q = dy.shape
        K = w.shape[1]
        dx = np.empty((N, C, P * stride, Q * stride), np.float32)
        getattr(self._lib, self._prefix + "dgrad")(_p(dy), _p(w), _p(theta), _p(dx), N, C, P, Q, K, stride)
        return dx

    def wgrad(self, dy, x, theta, K, stride=1):
        dy, x, theta = _f32(dy), _f32(x), _f32(theta).reshape(-1)
        N, C, H, W = x.shape
        dw = np.empty((C, 1, 1, K), np.float32)
        getattr(self._lib, self._prefix + "wgrad")(_p(dy), _p(x), _p(theta), _p(dw), N, C, H, W, K, stride)
        return dw


class Oracle(_Loops):
    """The plain-C restatement (oracle/o1d_oracle.c)."""

    _prefix = "o1d_oracle_"

    def __init__(self, path: str | None = None):
        path = path or os.path.join(HERE, "libo1d_oracle.so")
        if not os.path.exists(path):
            from . import build
            build.build_oracle()
        self._lib = ctypes.CDLL(path)
        for f in ("fprop", "dgrad", "wgrad", "fprop_f64", "dgrad_f64", "wgrad_f64", "offsets"):
            getattr(self._lib, "o1d_oracle_" + f).restype = None

    def offsets(self, theta, K):
        theta = _f32(theta).reshape(-1)
        C = theta.shape[0]
        dh = np.empty((C, K), np.int32)
        dw = np.empty((C, K), np.int32)
        self._lib.o1d_oracle_offsets(_p(theta), C, K, _p(dh, _i32p), _p(dw, _i32p))
        return dh, dw

    def fprop_f64(self, x, w, theta, stride=1):
        x, w, theta = _f32(x), _f32(w).reshape(x.shape[1], -1), _f32(theta).reshape(-1)
        N, C, H, W = x.shape
        y = np.empty((N, C, H // stride, W // stride), np.float64)
        self._lib.o1d_oracle_fprop_f64(_p(x), _p(w), _p(theta), _p(y, _f64p), N, C, H, W, w.shape[1], stride)
        return y

    def dgrad_f64(self, dy, w, theta, stride=1):
        dy, w, theta = _f32(dy), _f32(w).reshape(dy.shape[1], -1), _f32(theta).reshape(-1)
        N, C, P, Q = dy.shape
        dx = np.empty((N, C, P * stride, Q * stride), np.float64)
        self._lib.o1d_oracle_dgrad_f64(_p(dy), _p(w), _p(theta), _p(dx, _f64p), N, C, P, Q, w.shape[1], stride)
        return dx

    def wgrad_f64(self, dy, x, theta, K, stride=1):
        dy, x, theta = _f32(dy), _f32(x), _f32(theta).reshape(-1)
        N, C, H, W = x.shape
        dw = np.empty((C, 1, 1, K), np.float64)
        self._lib.o1d_oracle_wgrad_f64(_p(dy), _p(x), _p(theta), _p(dw, _f64p), N, C, H, W, K, stride)
        return dw


class Reference(_Loops):
    """The reference's own kernels.cpp, compiled from its checkout (oracle/_ref/)."""

    _prefix = "o1d_ref_"

    def __init__(self, path: str | None = None):
        import torch  # noqa: F401  (libtorch must be resident before the shim loads)

        path = path or os.path.join(HERE, "_ref", "libo1d_ref.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self._lib = ctypes.CDLL(path)

    @staticmethod
    def available() -> bool:
        return os.path.exists(os.path.join(HERE, "_ref", "libo1d_ref.so"))

    def module(self, x, w, theta, bias, dy, stride=1, nhwc=False, resid=False):
        """Forward + backward through the reference's autograd function
        (kernels.cpp:141-203).  Returns (y, dx, dw, db-or-None)."""
        x, dy, theta = _f32(x), _f32(dy), _f32(theta).reshape(-1)
        if nhwc:
            N, H, W, C = x.shape
        else:
            N, C, H, W = x.shape
        w = _f32(w).reshape(C, -1)
        K = w.shape[1]
        y = np.empty(dy.shape, np.float32)
        dx = np.empty(x.shape, np.float32)
        dw = np.empty((C, 1, 1, K), np.float32)
        db = np.empty((C,), np.float32) if bias is not None else None
        b = _f32(bias) if bias is not None else np.zeros(1, np.float32)
        self._lib.o1d_ref_module(_p(x), _p(w), _p(theta), _p(b), _p(dy), _p(y), _p(dx), _p(dw),
                                 _p(db) if db is not None else None, N, C, H, W, K, stride,
                                 int(nhwc), int(bias is not None), int(resid))
        return y, dx, dw, db


# --------------------------------------------------------------------------------------
# Restatement of the Python wrapper around the loops
# --------------------------------------------------------------------------------------

def _delta(C, K):
    """The resid kernel: 1 at the centre tap (dwoconv1d.py:136-141)."""
    d = np.zeros((C, 1, 1, K), np.float32)
    d[:, :, :, K // 2] = 1
    return d


def module_forward(loops, x, w, theta, bias=None, stride=1, nhwc=False, resid=False):
    """dwoconv1d.py:20-38: w+resid, NHWC->NCHW, fprop, +bias, NCHW->NHWC."""
    w = _f32(w).reshape(-1, 1, 1, np.asarray(w).shape[-1])
    if resid:
        w = w + _delta(w.shape[0], w.shape[-1])
    x = _f32(x)
    if nhwc:
        x = np.ascontiguousarray(x.transpose(0, 3, 1, 2))
    y = loops.fprop(x, w, theta, stride)
    if bias is not None:
        y = y + _f32(bias).reshape(1, -1, 1, 1)
    if nhwc:
        y = np.ascontiguousarray(y.transpose(0, 2, 3, 1))
    return y


def module_backward(loops, x, w, theta, dy, bias=None, stride=1, nhwc=False, resid=False):
    """dwoconv1d.py:41-69: returns (dx, dw, db-or-None) in the module's layout."""
    w = _f32(w).reshape(-1, 1, 1, np.asarray(w).shape[-1])
    K = w.shape[-1]
    if resid:
        w = w + _delta(w.shape[0], K)
    x, dy = _f32(x), _f32(dy)
    if nhwc:
        x = np.ascontiguousarray(x.transpose(0, 3, 1, 2))
        dy = np.ascontiguousarray(dy.transpose(0, 3, 1, 2))
    dx = loops.dgrad(dy, w, theta, stride)
    dw = loops.wgrad(dy, x, theta, K, stride)
    db = dy.sum(axis=(0, 2, 3), dtype=np.float64).astype(np.float32) if bias is not None else None
    if nhwc:
        dx = np.ascontiguousarray(dx.transpose(0, 2, 3, 1))
    return dx, dw, db


def next_power_of_2(x):
    return 1 if x == 0 else 1 << (x - 1).bit_length()


def forward_safe(loops, x, w, theta, bias=None, stride=1, nhwc=False, resid=False, cap=256):
    """dwoconv1d.py:154-187 (cap 256; the specialized module uses 128,
    dwoconv1d_specialized.py:160-161): pad bottom/right to a multiple of
    min(next_pow2(size)//2, cap), run in NCHW, crop pad//stride, restore layout."""
    x = _f32(x)
    if nhwc:
        x = x.transpose(0, 3, 1, 2)
    h, w_ = x.shape[2], x.shape[3]
    hp, wp = min(next_power_of_2(h) // 2, cap), min(next_power_of_2(w_) // 2, cap)
    pad_h, pad_w = (hp - h % hp) % hp, (wp - w_ % wp) % wp
    xp = np.pad(x, ((0, 0), (0, 0), (0, pad_h), (0, pad_w)))
    y = module_forward(loops, xp, w, theta, bias, stride, False, resid)
    y = y[:, :, : y.shape[2] - pad_h // stride, : y.shape[3] - pad_w // stride]
    if nhwc:
        y = y.transpose(0, 2, 3, 1)
    return np.ascontiguousarray(y)


def model_angles(C, N=8, layer_offset=0.0):
    """models/convnext.py:60-77,111-114: blocks of ~C/N channels share an angle;
    float64 arithmetic, rounded to float32 by torch.tensor()."""
    return np.array([np.pi * ((((N * (c + 1) - 1) // C) / N + layer_offset) % 1) for c in range(C)],
                    dtype=np.float64).astype(np.float32)


def round_robin_angles(C, N=8):
    """theta[c] = (c mod N) * pi / N, the assignment the kernel-sweep workload uses."""
    return np.array([(c % N) * np.pi / N for c in range(C)], dtype=np.float64).astype(np.float32)


def backward_safe(loops, x, w, theta, dy, bias=None, stride=1, nhwc=False, resid=False, cap=256):
    """Gradient of ``forward_safe``: autograd through pad -> op -> crop, i.e. dy is
    zero-extended over the cropped outputs and dx is cropped back to H x W."""
    x, dy = _f32(x), _f32(dy)
    if nhwc:
        x, dy = x.transpose(0, 3, 1, 2), dy.transpose(0, 3, 1, 2)
    h, w_ = x.shape[2], x.shape[3]
    hp, wp = min(next_power_of_2(h) // 2, cap), min(next_power_of_2(w_) // 2, cap)
    pad_h, pad_w = (hp - h % hp) % hp, (wp - w_ % wp) % wp
    xp = np.pad(x, ((0, 0), (0, 0), (0, pad_h), (0, pad_w)))
    P, Q = xp.shape[2] // stride, xp.shape[3] // stride
    dyp = np.pad(dy, ((0, 0), (0, 0), (0, P - dy.shape[2]), (0, Q - dy.shape[3])))
    dx, dw, db = module_backward(loops, xp, w, theta, dyp, bias, stride, False, resid)
    dx = dx[:, :, :h, :w_]
    if nhwc:
        dx = dx.transpose(0, 2, 3, 1)
    return np.ascontiguousarray(dx), dw, db


class ReferenceGPU:
    """The reference's own specialised CUDA kernels (models/dwoconv1d_specialized/kernels/
    kernels.h) compiled for sm_100a through refgpu_shim.cu: the GPU baseline to beat.  Built
    for H = W in {56, 28, 14, 7}, K = 31, stride 1, NCHW float32.  Takes and returns torch
    CUDA tensors; launches on the current stream."""

    SHAPES = (56, 28, 14, 7)

    def __init__(self, path: str | None = None):
        path = path or os.path.join(HERE, "_ref", "libo1d_refgpu.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self._lib = ctypes.CDLL(path)

    @staticmethod
    def available() -> bool:
        return os.path.exists(os.path.join(HERE, "_ref", "libo1d_refgpu.so"))

    @staticmethod
    def _stream():
        import torch
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _call(self, name, hw, *tensors, N, C):
        rc = getattr(self._lib, name)(hw, *[ctypes.c_void_p(t.data_ptr()) for t in tensors], N, C, self._stream())
        if rc:
            raise RuntimeError(f"{name}: status {rc}")

    def fprop(self, x, w, theta):
        import torch
        N, C, H, W = x.shape
        y = torch.empty_like(x)
        self._call("o1d_refgpu_fprop", H, y, w, x, theta, N=N, C=C)
        return y

    def dgrad(self, dy, w, theta):
        import torch
        N, C, H, W = dy.shape
        dx = torch.empty_like(dy)
        self._call("o1d_refgpu_dgrad", H, dx, w, dy, theta, N=N, C=C)
        return dx

    def wgrad(self, dy, x, theta, K=31):
        import torch
        N, C, H, W = x.shape
        dw = torch.empty((C, 1, 1, K), dtype=x.dtype, device=x.device)
        self._call("o1d_refgpu_wgrad", H, dw, dy, x, theta, N=N, C=C)
        return dw

    def transpose(self, t, n, a, b, out_shape):
        import torch
        out = torch.empty(out_shape, dtype=t.dtype, device=t.device)
        rc = self._lib.o1d_refgpu_transpose(n, a, b, ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(t.data_ptr()),
                                            self._stream())
        if rc:
            raise RuntimeError(f"o1d_refgpu_transpose: status {rc}")
        return out
