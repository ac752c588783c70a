"""Builds the two shared objects of this package, in-tree, for sm_100a only.

* ``hf_rocm_kernels/libhfrk_b200.so`` -- the CUDA kernels behind the C ABI of
  ``include/hfrk_b200.h`` (nvcc, no torch).
* ``hf_rocm_kernels/_HFRK_C.so`` -- the torch op registration, a C++ shim linked against the
  first library and libtorch.

Stands where the reference has ``setup.py`` + ``CMakeLists.txt`` (a ROCm/hipify build); here two
compiler invocations are enough. Usage: ``python build.py [--force] [--verbose]``.
"""
import argparse
import os
import shutil
import subprocess
import sys
import sysconfig
from typing import List

ROOT = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(ROOT, "csrc")
PKG = os.path.join(ROOT, "hf_rocm_kernels")
CAPI_LIB = os.path.join(PKG, "libhfrk_b200.so")
TORCH_EXT = os.path.join(PKG, "_HFRK_C.so")

CUDA_SOURCES = ["skinny_gemm_sm100.cu", "skinny_gemm_simt.cu", "swiglu_sm100.cu", "residual_rms_sm100.cu",
                "host_common.cu"]
CUDA_HEADERS = ["ptx_sm100.cuh", "host_common.h", "elementwise_common.cuh", "skinny_gemm_common.cuh",
                "skinny_gemm_kernel.cuh", "skinny_gemm_streamk.cuh", "device_model.cuh",
                os.path.join("..", "..", "include", "hfrk_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found")
    return found


def _stale(target: str, sources: List[str]) -> bool:
    if not os.path.exists(target):
        return True
    built = os.path.getmtime(target)
    return any(os.path.getmtime(s) > built for s in sources if os.path.exists(s))


def _run(cmd: List[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ...")
    if verbose:
        sys.stdout.write(proc.stdout + proc.stderr)


def build_capi(force: bool = False, verbose: bool = False) -> str:
    sources = [os.path.join(CSRC, s) for s in CUDA_SOURCES]
    deps = sources + [os.path.join(CSRC, h) for h in CUDA_HEADERS]
    if force or _stale(CAPI_LIB, deps):
        extra = ["-Xptxas", "-v"] if verbose else []
        _run([_nvcc()] + NVCC_FLAGS + extra + ["-o", CAPI_LIB] + sources, verbose)
    return CAPI_LIB


def build_torch_ext(force: bool = False, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    source = os.path.join(CSRC, "torch_bindings.cpp")
    if not (force or _stale(TORCH_EXT, [source, CAPI_LIB, os.path.join(ROOT, "..", "include", "hfrk_b200.h")])):
        return TORCH_EXT
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    includes = cpp_extension.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in includes]
    cmd += [source, "-o", TORCH_EXT, f"-L{PKG}", "-l:libhfrk_b200.so", f"-L{torch_lib}",
            "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)
    return TORCH_EXT


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_capi(force, verbose)
    build_torch_ext(force, verbose)


if __name__ == "__main__":
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    build_all(args.force, args.verbose)
    print(CAPI_LIB)
    print(TORCH_EXT)
