"""In-tree build of the B200 attention library (sm_100a only).

    python flash-attention-v100_b200/build.py [--force]

Produces, next to this file:
    lib/libfmha_b200.so            the C-ABI library (nvcc; include/fmha_b200.h)
    flash_attn_v100_cuda*.so       the torch extension the Python package imports (g++)

Replaces the reference's setup.py (setup.py:116-149, sm_70 only, external CUTLASS): one
architecture, no third-party headers.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libfmha_b200.so")
EXT_NAME = "flash_attn_v100_cuda"
EXT_PATH = os.path.join(HERE, EXT_NAME + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def _cuda_home() -> str:
    return os.environ.get("CUDA_HOME") or "/usr/local/cuda"


def build_library(force: bool = False, verbose_ptxas: bool = False) -> str:
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh"))]
    sources.append(os.path.join(ROOT, "include", "fmha_b200.h"))
    if not force and _newer(LIB_PATH, sources):
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose_ptxas else [])
    cmd += ["-o", LIB_PATH, os.path.join(CSRC, "fmha_api.cu")]
    _run(cmd)
    return LIB_PATH


def build_extension(force: bool = False) -> str:
    src = os.path.join(CSRC, "torch_ext.cpp")
    deps = [src, os.path.join(ROOT, "include", "fmha_b200.h"), LIB_PATH]
    if not force and _newer(EXT_PATH, deps):
        return EXT_PATH
    import torch
    from torch.utils import cpp_extension

    includes = cpp_extension.include_paths() + [sysconfig.get_paths()["include"],
                                                os.path.join(_cuda_home(), "include")]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w",
           "-DTORCH_EXTENSION_NAME=" + EXT_NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=" + str(int(torch._C._GLIBCXX_USE_CXX11_ABI))]
    for inc in includes:
        cmd += ["-isystem", inc]
    cmd += [src, "-o", EXT_PATH, "-L" + LIB_DIR, "-lfmha_b200", "-L" + torch_lib,
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-L" + os.path.join(_cuda_home(), "lib64"), "-lcudart",
            "-Wl,-rpath,$ORIGIN/lib", "-Wl,-rpath," + torch_lib]
    _run(cmd)
    return EXT_PATH


def build_all(force: bool = False):
    return build_library(force), build_extension(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", LIB_PATH, EXT_PATH)
