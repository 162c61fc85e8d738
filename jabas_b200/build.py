"""Compiles ``csrc/*.cu`` into ``jabas_b200/libjabas_b200.so`` for sm_100a with nvcc.

The library is built in-tree so that it travels with the source tree; there is no JIT
cache and no other architecture.  Run ``python -m jabas_b200.build`` (add ``-v`` for
ptxas register/spill output).
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
LIB_PATH = os.path.join(PKG_DIR, "libjabas_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]


def sources() -> list[str]:
    return sorted(glob.glob(os.path.join(PKG_DIR, "csrc", "*.cu")))


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    deps = sources() + glob.glob(os.path.join(ROOT, "include", "*.h")) \
        + glob.glob(os.path.join(PKG_DIR, "csrc", "*.cuh"))
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and not is_stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libjabas_b200.so cannot be built on this machine")
    # one nvcc per translation unit, side by side, then one link
    objdir = os.path.join(PKG_DIR, "csrc", "build")
    os.makedirs(objdir, exist_ok=True)
    jobs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.splitext(os.path.basename(src))[0] + ".o")
        cmd = [nvcc] + NVCC_FLAGS + ["-I", os.path.join(ROOT, "include"), "-c", "-o", obj, src]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        jobs.append((obj, cmd, subprocess.Popen(cmd)))
    for obj, cmd, proc in jobs:
        if proc.wait() != 0:
            raise subprocess.CalledProcessError(proc.returncode, cmd)
    subprocess.check_call([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB_PATH]
                          + [obj for obj, _, _ in jobs])
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force=True, verbose="-v" in sys.argv))
