#!/usr/bin/env python3
"""Recipe (test infrastructure): compile the REFERENCE's two sparse-MLA CUDA files, from where they
lie in the reference checkout, plus ``ref_shim.cu`` into ``oracle/_ref/libref_sparse_mla.so``.

The reference's own build system is not run (its dense-MLA sources need an un-vendored cutlass);
the sparse path is just these two files and ``flash_mla.h``.  Flags follow the reference's
(setup.py:358-377: -O3, --use_fast_math) with SASS for sm_100, which is what its wheels ship for
B200 (.github/workflows/wheels.yaml:33).  Nothing is copied into this repository; the output
directory is git-ignored.

    python oracle/ref_gpu/build_ref.py [/path/to/reference]

Without an argument the checkout is taken from $REFERENCE_ROOT, else from a directory named
``reference`` beside this repository.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT_DIR = os.path.join(ROOT, "oracle", "_ref")
OUT = os.path.join(OUT_DIR, "libref_sparse_mla.so")


def default_reference_root():
    return os.environ.get("REFERENCE_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")


def build(reference_root=None):
    reference_root = reference_root or default_reference_root()
    csrc = os.path.join(reference_root, "csrc")
    srcs = [os.path.join(csrc, "flash_sparse_mla_decode_sm80.cu"),
            os.path.join(csrc, "flash_sparse_mla_prefill_fused_sm80.cu")]
    if not all(os.path.exists(s) for s in srcs):
        return None
    os.makedirs(OUT_DIR, exist_ok=True)
    cmd = ["nvcc", "-O3", "-std=c++17", "--use_fast_math", "-gencode", "arch=compute_100,code=sm_100", "-shared",
           "-Xcompiler", "-fPIC", "-cudart", "shared", "-I", csrc, "-I", os.path.join(ROOT, "include"),
           *srcs, os.path.join(HERE, "ref_shim.cu"), "-o", OUT]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None))
