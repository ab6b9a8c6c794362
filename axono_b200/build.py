"""Builds the C-ABI library (axono_b200/lib/libaxono_b200.so) for sm_100a with nvcc, and the native
Python module `libaxono` (host runtime + operator adapters + pybind11 binding) that links against it.

    python -m axono_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU; the library is kept in-tree so it travels with the
source checkout.  Rebuilds only when a source or header is newer than the library.
"""
from __future__ import annotations

import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB = os.path.join(LIB_DIR, "libaxono_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")) + glob.glob(os.path.join(CSRC, "*.cpp")))


def _stale() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(CSRC, "*.h"))
    deps += glob.glob(os.path.join(ROOT, "include", "*.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not _stale():
        return LIB
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "nvcc")
    cmd = [nvcc, *NVCC_FLAGS, "-I", os.path.join(ROOT, "include"), "-I", CSRC]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB, *sources(), "-ldl"]
    subprocess.check_call(cmd)
    return LIB


HOST = os.path.join(CSRC, "host")


def native_module_path() -> str:
    import sysconfig

    return os.path.join(LIB_DIR, "libaxono" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_native(force: bool = False) -> str:
    """The `libaxono` extension module: csrc/host/*.cpp compiled with g++ against pybind11, the CUDA
    runtime and the C-ABI library beside it (rpath $ORIGIN)."""
    import sysconfig

    import pybind11

    lib = build(force=force)
    out = native_module_path()
    srcs = sorted(glob.glob(os.path.join(HOST, "*.cpp")))
    deps = srcs + glob.glob(os.path.join(HOST, "*.h")) + glob.glob(os.path.join(ROOT, "include", "*.h")) + [lib]
    if not force and os.path.exists(out) and all(os.path.getmtime(d) <= os.path.getmtime(out) for d in deps):
        return out
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden",
           "-I", os.path.join(ROOT, "include"), "-I", HOST, "-I", pybind11.get_include(),
           "-I", sysconfig.get_paths()["include"], "-I", os.path.join(cuda_home, "include"),
           "-o", out, *srcs,
           "-L", LIB_DIR, "-laxono_b200", "-L", os.path.join(cuda_home, "lib64"), "-lcudart", "-ldl",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(cuda_home, "lib64")]
    subprocess.check_call(cmd)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_native(force="--force" in sys.argv))
