"""ctypes binding of libo1d.so (declared in include/o1d.h).

There is no fallback: if the shared library is missing and cannot be built, importing
this module raises.  ctypes releases the GIL for the duration of each call.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

_c_int = ctypes.c_int
_c_void_p = ctypes.c_void_p
_c_size_t = ctypes.c_size_t
_f32p = ctypes.POINTER(ctypes.c_float)
_i8p = ctypes.POINTER(ctypes.c_int8)

# name -> (restype, argtypes); one entry per declaration in include/o1d.h
SIGNATURES = {
    "o1d_abi_version": (_c_int, []),
    "o1d_strerror": (ctypes.c_char_p, [_c_int]),
    "o1d_last_error": (ctypes.c_char_p, []),
    "o1d_set_route": (_c_int, [_c_int]),
    "o1d_last_route": (_c_int, []),
    "o1d_device_status": (_c_int, [ctypes.POINTER(_c_int)]),
    "o1d_device_status_clear": (_c_int, [ctypes.POINTER(_c_int)]),
    "o1d_selftest_wait_timeout": (_c_int, [_c_void_p, _c_void_p]),
    "o1d_uses_tiled": (_c_int, [_c_void_p] + [_c_int] * 8),
    "o1d_offsets": (_c_int, [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p]),
    "o1d_plan_bytes": (_c_size_t, [_c_int, _c_int]),
    "o1d_plan_build": (_c_int, [_c_void_p, _c_int, _c_int, _c_void_p]),
    "o1d_plan_num_classes": (_c_int, [_c_void_p]),
    "o1d_fprop": (_c_int, [_c_void_p] * 6 + [_c_int] * 9 + [_c_void_p]),
    "o1d_dgrad": (_c_int, [_c_void_p] * 5 + [_c_int] * 9 + [_c_void_p]),
    "o1d_dgrad_act": (_c_int, [_c_void_p] * 6 + [_c_int] * 9 + [_c_void_p]),
    "o1d_wgrad_workspace_bytes": (_c_size_t, [_c_int] * 8),
    "o1d_wgrad": (_c_int, [_c_void_p] * 7 + [_c_size_t] + [_c_int] * 8 + [_c_void_p]),
    "o1d_wgrad_act": (_c_int, [_c_void_p] * 7 + [_c_size_t] + [_c_int] * 9 + [_c_void_p]),
    "o1d_wgrad_static": (_c_int, [_c_void_p] * 6 + [_c_int] * 8 + [_c_void_p]),
    "o1d_layernorm_cl": (_c_int, [_c_void_p] * 4 + [ctypes.c_longlong, _c_int, ctypes.c_float, _c_int, _c_int,
                                                  _c_void_p]),
    "o1d_layernorm_cl_bwd_workspace_bytes": (_c_size_t, [ctypes.c_longlong, _c_int]),
    "o1d_layernorm_cl_bwd": (_c_int, [_c_void_p] * 8 + [_c_size_t, ctypes.c_longlong, _c_int, ctypes.c_float, _c_int,
                                                      _c_int, _c_void_p]),
    "o1d_colsum_workspace_bytes": (_c_size_t, [ctypes.c_longlong, _c_int, _c_int]),
    "o1d_colsum": (_c_int, [_c_void_p] * 3 + [_c_size_t, ctypes.c_longlong, _c_int, _c_int, _c_void_p]),
    "o1d_pointwise_in": (_c_int, [_c_void_p] * 4 + [_c_int, _c_int, ctypes.c_longlong, _c_int, _c_int, _c_void_p]),
    "o1d_transpose": (_c_int, [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p]),
}

ABI_VERSION = 2
NCHW, NHWC = 0, 1
F32, BF16 = 0, 1
FLAG_IDENTITY, FLAG_GELU_INPUT = 1, 2


class O1dError(RuntimeError):
    pass


def _load() -> ctypes.CDLL:
    path = _build.LIB
    if _build.stale():
        try:
            _build.build()
        except Exception as e:  # no CPU path exists, and kernels older than csrc/ must not run
            what = "is missing" if not os.path.exists(path) else "was built from other sources than csrc/"
            raise RuntimeError(
                f"libo1d.so {what} and could not be rebuilt ({e}); "
                "run `python -m oriented1d_b200.build`") from e
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a symbol
        fn.restype, fn.argtypes = res, args
    if lib.o1d_abi_version() != ABI_VERSION:
        raise RuntimeError(f"libo1d.so has ABI {lib.o1d_abi_version()}, binding expects {ABI_VERSION}")
    return lib


lib = _load()


def check(status: int, what: str = "o1d") -> None:
    """Turn a non-zero status into an exception (ValueError for bad arguments,
    O1dError otherwise), like the reference's TORCH_CHECK -> RuntimeError."""
    if status == 0:
        return
    msg = lib.o1d_strerror(status).decode()
    if status == 3:
        msg += ": " + lib.o1d_last_error().decode()
    if status == 1:
        raise ValueError(f"{what}: {msg}")
    raise O1dError(f"{what}: {msg}")
