"""In-tree build of the native libraries (sm_100a only; nvcc cross-compiles without a GPU).

  lib/libb200tbe.so            CUDA kernels + the C ABI declared in include/b200tbe.h
  lib/libb200tbe_torch_ops.so  C++ torch extension registering torch.ops.fbgemm.* on top of it

Run as `python -m torchlib_xpu_b200._build [--force]`.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIBDIR = os.path.join(PKG, "lib")
OBJDIR = os.path.join(PKG, "lib", "obj")
INCLUDE = os.path.join(ROOT, "include")

CABI_LIB = os.path.join(LIBDIR, "libb200tbe.so")
TORCH_OPS_LIB = os.path.join(LIBDIR, "libb200tbe_torch_ops.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "-I", INCLUDE, "-I", CSRC,
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.sep not in cand or os.path.exists(cand)):
            return cand
    return "nvcc"


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _headers() -> list[str]:
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(INCLUDE, "*.h"))


def build_cabi(force: bool = False) -> str:
    os.makedirs(OBJDIR, exist_ok=True)
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = _headers()
    objs, jobs = [], []
    for src in sources:
        obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append([_nvcc(), *NVCC_FLAGS, "-c", src, "-o", obj])
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(_run, jobs))
    if jobs or not os.path.exists(CABI_LIB):
        _run([_nvcc(), "-shared", "-o", CABI_LIB, *objs, "-cudart", "static"])
    return CABI_LIB


def build_torch_ops(force: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    build_cabi(force)
    os.makedirs(LIBDIR, exist_ok=True)
    src = os.path.join(CSRC, "fbgemm_ops.cpp")
    if force or _stale(TORCH_OPS_LIB, [src, CABI_LIB] + _headers()):
        troot = os.path.dirname(torch.__file__)
        tlib = os.path.join(troot, "lib")
        incs = []
        for inc in cpp_extension.include_paths("cuda"):
            incs += ["-isystem", inc]
        _run(["g++", "-O2", "-fPIC", "-shared", "-std=c++17", "-fvisibility=hidden",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
              "-DTORCH_API_INCLUDE_EXTENSION_H", "-I", INCLUDE, *incs, "-o", TORCH_OPS_LIB, src,
              "-L", LIBDIR, "-lb200tbe", "-Wl,-rpath,$ORIGIN", "-L", tlib, "-Wl,-rpath," + tlib,
              "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda"])
    return TORCH_OPS_LIB


def build_all(force: bool = False) -> dict[str, str]:
    return {"cabi": build_cabi(force), "torch_ops": build_torch_ops(force)}


if __name__ == "__main__":
    for name, path in build_all("--force" in sys.argv).items():
        print(name, path)
