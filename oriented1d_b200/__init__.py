"""oriented1d_b200 — oriented 1D depthwise convolution for NVIDIA B200 (sm_100a).

Hand-written CUDA kernels behind a C ABI (``include/o1d.h``, ``libo1d.so``) and a
Python module with the reference project's operator API (``DepthwiseOrientedConv1d``).
Importing the package loads the shared library and fails if it is unavailable: there is
no CPU or PyTorch fallback.
"""
from . import _lib, ops
from .dwoconv1d import (DepthwiseOrientedConv1d, get_dwoconv1d_kernel,
                        oriented_dwconv1d_get_module_from_params)
from .ops import Plan, dgrad, fprop, nchw_to_nhwc, nhwc_to_nchw, offsets, wgrad

__all__ = ["DepthwiseOrientedConv1d", "get_dwoconv1d_kernel", "oriented_dwconv1d_get_module_from_params",
           "Plan", "fprop", "dgrad", "wgrad", "nhwc_to_nchw", "nchw_to_nhwc", "offsets", "compat_path"]


def compat_path() -> str:
    """Directory to put on ``sys.path`` so that ``import dwoconv1d`` and
    ``import dwoconv1d_specialized`` (the bare names models/convnext.py:18-23 uses)
    resolve to this implementation."""
    import os
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "compat")
