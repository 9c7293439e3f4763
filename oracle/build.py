"""Build recipe for the test oracle.  TEST INFRASTRUCTURE ONLY.

Two artefacts, both kept out of version control:

* ``oracle/libo1d_oracle.so`` — the plain-C restatement in ``o1d_oracle.c`` (gcc).
* ``oracle/_ref/libo1d_ref.so`` — the reference's own CPU operator
  (models/dwoconv1d_reference/kernels/kernels.cpp), compiled where it lies in the
  reference checkout through ``ref_shim.cpp``.  Only built when a reference checkout
  is present (``O1D_REFERENCE_ROOT``, or a directory named ``reference`` beside this
  repository); elsewhere the prebuilt file is used as is.

Run ``python oracle/build.py`` to (re)build both.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libo1d_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libo1d_ref.so")
REF_SUBDIR = os.path.join("models", "dwoconv1d_reference", "kernels")


def _checkout() -> str:
    """Where a reference checkout would be: O1D_REFERENCE_ROOT, else `reference` beside this repository."""
    beside = os.path.normpath(os.path.join(HERE, os.pardir, os.pardir, "reference"))
    return os.environ.get("O1D_REFERENCE_ROOT", beside)


def reference_root() -> str | None:
    root = _checkout()
    return root if os.path.isfile(os.path.join(root, REF_SUBDIR, "kernels.cpp")) else None


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "o1d_oracle.c")
    if force or _stale(ORACLE_SO, [src]):
        # -ffp-contract=off: the reference loops are separate multiply and add
        # (x86-64 baseline has no FMA), and bit-equality with them is tested.
        cmd = ["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-o", ORACLE_SO, src, "-lm"]
        subprocess.run(cmd, check=True)
    return ORACLE_SO


def build_ref(force: bool = False) -> str | None:
    """Compile the reference's kernels.cpp through ref_shim.cpp; None if no checkout."""
    root = reference_root()
    if root is None:
        return REF_SO if os.path.exists(REF_SO) else None
    shim = os.path.join(HERE, "ref_shim.cpp")
    ref_src = os.path.join(root, REF_SUBDIR, "kernels.cpp")
    if not (force or _stale(REF_SO, [shim, ref_src])):
        return REF_SO
    import torch
    from torch.utils import cpp_extension

    os.makedirs(REF_DIR, exist_ok=True)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-w",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-I" + os.path.join(root, REF_SUBDIR)]
    cmd += ["-I" + p for p in cpp_extension.include_paths()]
    cmd += ["-I" + sysconfig.get_paths()["include"], "-I" + cuda_inc]
    cmd += [shim, "-o", REF_SO, "-L" + torch_lib, "-Wl,-rpath," + torch_lib,
            "-ltorch", "-ltorch_cpu", "-lc10"]
    subprocess.run(cmd, check=True)
    return REF_SO


REFGPU_SO = os.path.join(REF_DIR, "libo1d_refgpu.so")
REFGPU_SUBDIR = os.path.join("models", "dwoconv1d_specialized", "kernels")


def build_refgpu(force: bool = False) -> str | None:
    """Compile the reference's specialised CUDA kernels (kernels.h, nhwc_utils.h) for sm_100a
    through refgpu_shim.cu; None if there is no checkout.  Several minutes: the reference
    fully unrolls its kernels per shape."""
    src_dir = os.path.join(_checkout(), REFGPU_SUBDIR)
    if not os.path.isfile(os.path.join(src_dir, "kernels.h")):
        return REFGPU_SO if os.path.exists(REFGPU_SO) else None
    shim = os.path.join(HERE, "refgpu_shim.cu")
    if not (force or _stale(REFGPU_SO, [shim, os.path.join(src_dir, "kernels.h")])):
        return REFGPU_SO
    os.makedirs(REF_DIR, exist_ok=True)
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w", "-Xcompiler", "-fPIC",
           "-shared", "-I" + src_dir, shim, "-o", REFGPU_SO]
    subprocess.run(cmd, check=True)
    return REFGPU_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_ref(force="--force" in sys.argv))
    if "--gpu-reference" in sys.argv:
        print(build_refgpu(force="--force" in sys.argv))
