#!/usr/bin/env python3
"""In-tree build of the sparse-MLA library for sm_100a (one rule, no multi-arch machinery).

Produces, under ``forks-flash-mla-int_b200/lib/``:

* ``libsparse_mla_b200.so`` -- the CUDA kernels behind the C ABI of ``include/sparse_mla_b200.h``
  (no torch, no Python dependency);
* ``flash_mla_cuda.so``     -- the torch-stable-ABI extension (``csrc/flash_api.cpp``) that registers
  ``torch.ops.flash_mla.*`` and calls the C ABI.

    python forks-flash-mla-int_b200/build.py [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "lib")
INCLUDE = os.path.join(ROOT, "include")

CUDA_SOURCES = ["sparse_mla_attn_sm100.cu", "quantize_int8_sm100.cu", "cache_writers_sm100.cu", "c_api.cu", "decode_static_scratch.cu"]
CUDA_HEADERS = ["sm100_ptx.cuh", "smla_internal.h", "row_codec.cuh"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC")
    return cand


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 or verbose:
        sys.stdout.write(r.stdout)
        sys.stderr.write(r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}")


def build_core(force=False, verbose=False) -> str:
    os.makedirs(LIB, exist_ok=True)
    out = os.path.join(LIB, "libsparse_mla_b200.so")
    deps = [os.path.join(CSRC, f) for f in CUDA_SOURCES + CUDA_HEADERS] + [
        os.path.join(INCLUDE, "sparse_mla_b200.h"), os.path.abspath(__file__)]
    if not force and _newer(out, deps):
        return out
    cmd = [_nvcc(), "-O3", "-std=c++17", "-lineinfo", *ARCH, "-shared", "-Xcompiler", "-fPIC",
           "-Xcompiler", "-fvisibility=hidden", "-I", INCLUDE, "-I", CSRC, "--expt-relaxed-constexpr",
           "-cudart", "shared"]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [os.path.join(CSRC, f) for f in CUDA_SOURCES] + ["-o", out]
    _run(cmd, verbose)
    return out


def build_torch_ext(force=False, verbose=False) -> str:
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(LIB, exist_ok=True)
    out = os.path.join(LIB, "flash_mla_cuda.so")
    src = os.path.join(CSRC, "flash_api.cpp")
    deps = [src, os.path.join(INCLUDE, "sparse_mla_b200.h"), os.path.abspath(__file__)]
    if not force and _newer(out, deps):
        return out
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    inc = []
    for p in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(cuda_home, "include"), INCLUDE]:
        inc += ["-I", p]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = [os.environ.get("SMLA_CXX", "g++"), "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden",
           "-DTORCH_STABLE_ONLY", "-DUSE_CUDA", "-DPy_LIMITED_API=0x03090000", *inc, src, "-o", out,
           "-L", LIB, "-lsparse_mla_b200", "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-lc10",
           "-L", os.path.join(cuda_home, "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    _run(cmd, verbose)
    return out


def build_all(force=False, verbose=False):
    return build_core(force, verbose), build_torch_ext(force, verbose)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--core-only", action="store_true")
    args = ap.parse_args()
    if args.core_only:
        print(build_core(args.force, args.verbose))
    else:
        for p in build_all(args.force, args.verbose):
            print(p)
