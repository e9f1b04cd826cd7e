"""Builds libringattn_b200.so (the C-ABI library with the sm_100a kernels) in-tree with nvcc.

Replaces the reference's CMakeLists.txt:1-32 / makefile:1-7 (one executable per csrc/*.cu,
CUDA_ARCHITECTURES 80, -lnvshmem): one shared library, sm_100a only, NCCL resolved at run time.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libringattn_b200.so")
SOURCES = [os.path.join(CSRC, "ring_attention.cu")]
MAIN = os.path.join(HERE, "ring_attention_main")            # the reference's driver executable, over the library
MAIN_SOURCE = os.path.join(CSRC, "ring_attention_main.cu")
TORCH_EXT = os.path.join(HERE, "_torch_ext.so")             # torch.Tensor front end (optional; needs torch's headers)
TORCH_EXT_SOURCE = os.path.join(CSRC, "torch_ext.cpp")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the library cannot be built")
    return exe


def _stale() -> bool:
    if not os.path.exists(LIB) or not os.path.exists(MAIN):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(os.path.dirname(HERE), "include", "ring_attention_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile if the library is missing or older than its sources; returns its path."""
    if force or _stale():
        cmd = [_nvcc(), *NVCC_FLAGS, "-o", LIB, *SOURCES, "-ldl"]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + res.stdout + res.stderr)
        if verbose:
            print(res.stderr)
        # driver executable mirroring the reference's main(); finds the library next to itself
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-o", MAIN, MAIN_SOURCE,
               "-L" + HERE, "-lringattn_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("nvcc failed on the driver executable:\n" + res.stdout + res.stderr)
    return LIB


def build_torch_ext(force: bool = False) -> str:
    """Compile the torch.Tensor front end (csrc/torch_ext.cpp) against this interpreter's torch; returns its path.

    Host code only: it links to libringattn_b200.so (found next to itself) and to torch's libraries.
    """
    build()
    deps = [TORCH_EXT_SOURCE, LIB, os.path.join(os.path.dirname(HERE), "include", "attention_api.cuh")]
    if not force and os.path.exists(TORCH_EXT) and all(os.path.getmtime(d) <= os.path.getmtime(TORCH_EXT) for d in deps):
        return TORCH_EXT
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    cxx = shutil.which("g++") or "/usr/bin/g++"
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_inc = os.path.join(os.path.dirname(os.path.dirname(_nvcc())), "include")
    cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=_torch_ext",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths() + [sysconfig.get_paths()["include"], cuda_inc]:
        cmd += ["-isystem", inc]
    cmd += ["-o", TORCH_EXT, TORCH_EXT_SOURCE, "-L" + HERE, "-lringattn_b200", "-L" + torch_lib,
            "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("g++ failed on the torch front end:\n" + res.stdout + res.stderr)
    return TORCH_EXT


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--torch" in sys.argv:
        print(build_torch_ext(force="--force" in sys.argv))
