"""Compile libtllm_b200.so in-tree with nvcc for sm_100a.

    python -m ternary_llm_b200.build [--force] [-v] [--timeline]

--timeline builds a second, diagnostic library, libtllm_b200_timeline.so, with
-DTLLM_TIMELINE: its GEMV kernels record time stamps of their phases (see
csrc/gemv_mma.cu) and it exports tllm_b200_timeline_read.  Point TLLM_B200_LIB at it to
load it instead of the regular library.

The library is a single shared object built from every .cu file under csrc/.
nvcc cross-compiles without a GPU, so this runs on a CPU-only build machine.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
LIB = os.path.join(PKG, "libtllm_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]


def sources():
    return sorted(glob.glob(os.path.join(PKG, "csrc", "*.cu")))


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(PKG, "csrc", "*.cuh")) + \
        glob.glob(os.path.join(ROOT, "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, timeline: bool = False) -> str:
    out = os.path.join(PKG, "libtllm_b200_timeline.so") if timeline else LIB
    if not timeline and not force and not _stale():
        return LIB
    cmd = ["nvcc"] + NVCC_FLAGS + (["-DTLLM_TIMELINE"] if timeline else []) + \
        ["-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(PKG, "csrc"), "-o", out] + sources()
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, timeline="--timeline" in sys.argv))
