"""Builds libflaxattn.so (the C ABI of include/flaxattn.h) in-tree with nvcc for sm_100a,
and checks that every kernel template compiles for sm_100a with a representative mod."""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB = os.path.join(PKG, "libflaxattn.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def host_sources():
    srcs = [os.path.join(HERE, "flaxattn.cu"), os.path.join(PKG, "..", "include", "flaxattn.h")]
    kdir = os.path.join(HERE, "kernels")
    srcs += [os.path.join(kdir, f) for f in sorted(os.listdir(kdir)) if f.endswith(".h")]
    extra = os.path.join(HERE, "flaxattn_static.cu")
    if os.path.exists(extra):
        srcs.append(extra)
    return srcs


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = host_sources()
    if not force and _newer(LIB, srcs):
        return LIB
    cu = [s for s in srcs if s.endswith(".cu")]
    cmd = [NVCC, *ARCH, "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           *cu, "-o", LIB, "-lnvrtc", "-ldl",
           "-Xlinker", f"-rpath={CUDA_HOME}/lib64"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True, cwd=HERE)
    return LIB


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
