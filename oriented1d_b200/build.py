"""In-tree build of libo1d.so (sm_100a only).

``python -m oriented1d_b200.build`` compiles every ``csrc/*.cu`` with nvcc (one object per
file, in parallel) and links them into ``oriented1d_b200/libo1d.so``.  nvcc cross-compiles,
so this works on a machine without a GPU.  The library has no dependency on torch or Python.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libo1d.so")

OBJ_DIR = os.path.join(HERE, "_obj")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def nvcc() -> str:
    exe = shutil.which("nvcc") or os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; libo1d.so cannot be built")
    return exe


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def source_digest() -> str:
    """Hash of everything the library is compiled from (file names and contents)."""
    import hashlib
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    deps = sorted(glob.glob(os.path.join(CSRC, "*"))) + [os.path.join(HERE, "..", "include", "o1d.h")]
    for d in deps:
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def stale() -> bool:
    """True when libo1d.so is missing or was built from other sources (content hash kept
    beside the library; file times are not used because copies do not preserve them)."""
    if not os.path.exists(LIB) or not os.path.exists(LIB + ".digest"):
        return True
    with open(LIB + ".digest") as f:
        return f.read().strip() != source_digest()


def _file_digest(src: str) -> str:
    """Hash of one source file together with every header it could include."""
    import hashlib
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    deps = [src] + sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + sorted(glob.glob(os.path.join(CSRC, "*.h")))
    deps.append(os.path.join(HERE, "..", "include", "o1d.h"))
    for d in deps:
        h.update(os.path.basename(d).encode())
        with open(d, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _compile_one(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
    tag = obj + ".digest"
    digest = _file_digest(src)
    if not force and os.path.exists(obj) and os.path.exists(tag):
        with open(tag) as f:
            if f.read().strip() == digest:
                return obj
    cmd = [nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    with open(tag, "w") as f:
        f.write(digest)
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    if not (force or stale()):
        return LIB
    from concurrent.futures import ThreadPoolExecutor
    os.makedirs(OBJ_DIR, exist_ok=True)
    srcs = sources()
    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(lambda s: _compile_one(s, force, verbose), srcs))
    subprocess.run([nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB, *objs], check=True)
    with open(LIB + ".digest", "w") as f:
        f.write(source_digest())
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
