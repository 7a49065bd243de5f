"""Builds the CPU oracle libraries (test infrastructure; the product never loads them).

  oracle/_build/libtbe_oracle.so       plain-C restatement (tbe_oracle.c), OpenMP
  oracle/_build/libfbgemm_core_ref.so  harness around the FBGEMM-core kernels inside torch's
                                       libtorch_cpu.so (fbgemm_core_ref.cpp)
  oracle/_build/libnv12_oracle.so      NV12 -> RGB24 colour conversion (nv12_oracle.c), built without
                                       floating-point contraction

  oracle/_ref/libnv12_ref.so           the REFERENCE's own colour-conversion source file
  oracle/_ref/libnv12_ref_fma.so       (packages/torchcodec-xpu/src/torchcodec_xpu/ColorConversionKernel.cpp),
                                       compiled for the host from where it lies in the reference tree
                                       on top of a stand-in for the SYCL names it uses
                                       (nv12_ref_wrap.cpp, sycl_host_shim/); without and with
                                       floating-point contraction. Built only where the reference tree
                                       is present; elsewhere the built files are used as they are.

Run as `python oracle/build.py`; __graft_entry__.build() calls build_all() too.
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build")
REF_OUT = os.path.join(HERE, "_ref")
REFERENCE_SRC_DIR = os.environ.get(
    "B200TBE_REFERENCE_SRC", "/root/reference/packages/torchcodec-xpu/src/torchcodec_xpu")


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


def nv12_reference_libs() -> dict[str, str]:
    return {"nv12_ref": os.path.join(REF_OUT, "libnv12_ref.so"),
            "nv12_ref_fma": os.path.join(REF_OUT, "libnv12_ref_fma.so")}


def build_nv12_reference(force: bool = False) -> dict[str, str]:
    """Compiles the reference's ColorConversionKernel.cpp for the host, when the reference tree is
    there. Returns the libraries that exist afterwards (possibly none)."""
    libs = nv12_reference_libs()
    ref_src = os.path.join(REFERENCE_SRC_DIR, "ColorConversionKernel.cpp")
    if os.path.exists(ref_src):
        os.makedirs(REF_OUT, exist_ok=True)
        wrap = os.path.join(HERE, "nv12_ref_wrap.cpp")
        shim = os.path.join(HERE, "sycl_host_shim")
        deps = [wrap, os.path.join(shim, "sycl", "sycl.hpp"), ref_src]
        for name, extra in (("nv12_ref", ["-ffp-contract=off"]), ("nv12_ref_fma", ["-ffp-contract=fast", "-mfma"])):
            if force or _stale(libs[name], deps):
                _run(["g++", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-std=c++17",
                      "-DWITH_SYCL_KERNELS", *extra, "-I", shim, "-I", REFERENCE_SRC_DIR, "-o", libs[name], wrap])
    return {k: v for k, v in libs.items() if os.path.exists(v)}


def build_all(force: bool = False) -> dict[str, str]:
    out = {"c_oracle": build_c_oracle(force), "fbgemm_core_ref": build_fbgemm_core_ref(force),
           "nv12_oracle": build_nv12_oracle(force)}
    out.update(build_nv12_reference(force))
    return out


if __name__ == "__main__":
    for name, path in build_all("--force" in sys.argv).items():
        print(name, path)
