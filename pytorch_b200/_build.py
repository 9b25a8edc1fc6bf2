"""In-tree build of the two shared libraries of the package.

``lib/libb200q.so``      the C ABI declared in ``include/b200q.h``: every CUDA kernel, compiled
                         by nvcc for sm_100a only.  No torch types, no libtorch dependency.
``lib/libb200q_torch.so`` the thin PyTorch extension: ``TORCH_LIBRARY(npu)`` schemas plus CUDA and
                         Meta implementations that validate arguments, allocate outputs and call
                         the C ABI on the current stream.

Both are rebuilt only when a source is newer than the library.  nvcc cross-compiles without
a GPU, so the build runs on any machine with the CUDA toolkit.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
CABI_LIB = os.path.join(LIBDIR, "libb200q.so")
TORCH_LIB = os.path.join(LIBDIR, "libb200q_torch.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]


def _cuda_home() -> str:
    home = os.environ.get("CUDA_HOME") or os.environ.get("CUDA_PATH") or "/usr/local/cuda"
    if not os.path.isdir(home):
        nvcc = shutil.which("nvcc")
        if nvcc:
            home = os.path.dirname(os.path.dirname(nvcc))
    return home


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str], log_name: str) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(os.path.join(LIBDIR, log_name), "w") as f:
        f.write(" ".join(cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout[-8000:])
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ... (log: lib/{log_name})")


def build_cabi(force: bool = False) -> str:
    os.makedirs(LIBDIR, exist_ok=True)
    sources = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith((".cu", ".cuh"))]
    sources.append(os.path.join(ROOT, "include", "b200q.h"))
    if force or _stale(CABI_LIB, sources):
        nvcc = os.path.join(_cuda_home(), "bin", "nvcc")
        _run([nvcc, *NVCC_FLAGS, "-o", CABI_LIB, os.path.join(CSRC, "libb200q.cu")], "build_cabi.log")
    return CABI_LIB


def build_torch_ext(force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    build_cabi(force)
    src = os.path.join(CSRC, "register.cpp")
    if force or _stale(TORCH_LIB, [src, os.path.join(ROOT, "include", "b200q.h"), CABI_LIB]):
        tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
        inc = [f"-I{p}" for p in cpp_extension.include_paths()] + [
            f"-I{os.path.join(_cuda_home(), 'include')}", f"-I{os.path.join(ROOT, 'include')}"]
        abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
        cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
               "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, src, "-o", TORCH_LIB,
               f"-L{LIBDIR}", "-lb200q", f"-L{tlib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10",
               "-lc10_cuda", f"-L{os.path.join(_cuda_home(), 'lib64')}", "-lcudart",
               "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{tlib}"]
        _run(cmd, "build_torch.log")
    return TORCH_LIB


def build_all(force: bool = False) -> None:
    build_torch_ext(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", CABI_LIB, TORCH_LIB)
