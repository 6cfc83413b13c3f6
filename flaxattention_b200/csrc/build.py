"""Builds libflaxattn.so (the C ABI of include/flaxattn.h) in-tree with nvcc for sm_100a,
and checks that every kernel template compiles for sm_100a with a representative mod."""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
LIB = os.path.join(PKG, "libflaxattn.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


STAMP = LIB + ".sources"  # hash of the sources the library was built from


def sources_hash() -> str:
    """Hash of everything the host library is compiled from.  The library computes launch
    parameters (shared-memory sizes, grids, buffer layouts) that have to match the kernel
    templates it sits beside, so a library built from other sources must not be used."""
    h = hashlib.sha256()
    for path in host_sources():
        with open(path, "rb") as f:
            h.update(f.read())
        h.update(b"\0")
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == sources_hash()


def host_sources():
    srcs = [os.path.join(HERE, "flaxattn.cu"), os.path.join(PKG, "..", "include", "flaxattn.h")]
    kdir = os.path.join(HERE, "kernels")
    # the templates count too: the library's launch code mirrors their shared-memory maps
    srcs += [os.path.join(kdir, f) for f in sorted(os.listdir(kdir)) if f.endswith((".h", ".cuh"))]
    extra = os.path.join(HERE, "flaxattn_static.cu")
    if os.path.exists(extra):
        srcs.append(extra)
    return srcs


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = host_sources()
    if not force and is_current():
        return LIB
    cu = [s for s in srcs if s.endswith(".cu")]
    cmd = [NVCC, *ARCH, "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
           *cu, "-o", LIB, "-lnvrtc", "-ldl",
           "-Xlinker", f"-rpath={CUDA_HOME}/lib64"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True, cwd=HERE)
    with open(STAMP, "w") as f:
        f.write(sources_hash() + "\n")
    return LIB


def build_ffi_shim() -> str:
    """Builds libflaxattn_ffi.so (the jax.ffi handlers of ffi_shim.cc).  Needs the XLA FFI headers
    that ship with jaxlib; raises where JAX is not installed."""
    import jax.ffi  # noqa: F401

    out = os.path.join(PKG, "libflaxattn_ffi.so")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", os.path.join(HERE, "ffi_shim.cc"),
           "-I" + os.path.join(PKG, "..", "include"), "-I" + jax.ffi.include_dir(), "-I" + os.path.join(CUDA_HOME, "include"),
           "-L" + PKG, "-l:libflaxattn.so", "-Wl,-rpath," + PKG, "-o", out]
    subprocess.run(cmd, check=True, cwd=HERE)
    return out


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--ffi" in sys.argv:
        print(build_ffi_shim())
