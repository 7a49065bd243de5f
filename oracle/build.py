"""Builds the CPU oracle libraries (test infrastructure; the product never loads them).

  oracle/_build/libtbe_oracle.so       plain-C restatement (tbe_oracle.c), OpenMP
  oracle/_build/libfbgemm_core_ref.so  harness around the FBGEMM-core kernels inside torch's
                                       libtorch_cpu.so (fbgemm_core_ref.cpp)
  oracle/_build/libnv12_oracle.so      NV12 -> RGB24 colour conversion (nv12_oracle.c), built without
                                       floating-point contraction

Run as `python oracle/build.py`; __graft_entry__.build() calls build_all() too.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def build_c_oracle(force: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "tbe_oracle.c")
    lib = os.path.join(OUT, "libtbe_oracle.so")
    if force or _stale(lib, [src]):
        _run(["gcc", "-O2", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden", "-std=c11",
              "-Wall", "-Wextra", "-o", lib, src, "-lm"])
    return lib


def build_nv12_oracle(force: bool = False) -> str:
    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "nv12_oracle.c")
    lib = os.path.join(OUT, "libnv12_oracle.so")
    if force or _stale(lib, [src]):
        _run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-fvisibility=hidden", "-std=c11",
              "-Wall", "-Wextra", "-o", lib, src])
    return lib


def build_fbgemm_core_ref(force: bool = False) -> str:
    import torch

    os.makedirs(OUT, exist_ok=True)
    src = os.path.join(HERE, "fbgemm_core_ref.cpp")
    lib = os.path.join(OUT, "libfbgemm_core_ref.so")
    if force or _stale(lib, [src]):
        troot = os.path.dirname(torch.__file__)
        tlib = os.path.join(troot, "lib")
        _run(["g++", "-O2", "-fopenmp", "-fPIC", "-shared", "-fvisibility=hidden", "-std=c++17",
              "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
              "-I", os.path.join(troot, "include"), "-o", lib, src,
              "-L", tlib, "-Wl,-rpath," + tlib, "-ltorch_cpu", "-lc10"])
    return lib


def build_all(force: bool = False) -> dict[str, str]:
    return {"c_oracle": build_c_oracle(force), "fbgemm_core_ref": build_fbgemm_core_ref(force),
            "nv12_oracle": build_nv12_oracle(force)}


if __name__ == "__main__":
    for name, path in build_all("--force" in sys.argv).items():
        print(name, path)
