"""TEST INFRASTRUCTURE ONLY — build the REFERENCE's CUDA kernels for this path.

Compiles the reference's own, unmodified sources where they lie in a checkout of
the reference (REFERENCE_DIR below, or --reference) together with oracle/ref_cuda_binding.cu
into oracle/_ref/libelman_ref_cuda.so (sm_100; the reference's Makefile only
lists sm_80/sm_89).  Nothing is copied out of the reference; only the built
library lands in oracle/_ref/, which is git-ignored.

    python oracle/build_ref.py [--reference /path/to/reference]

The library is the second oracle of the GPU tests (the reference's bf16 rounding
points) and the "reference CUDA build on the same B200" timing of the benchmark.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# where a checkout of the reference lives on the build machine (absent on a GPU-only box)
REFERENCE_DIR = os.environ.get("ELMAN_REFERENCE_DIR", os.path.join(os.sep, "root", "reference"))
OUT = os.path.join(HERE, "_ref")
LIB = os.path.join(OUT, "libelman_ref_cuda.so")
REF_SOURCES = ["mamba_gated_elman_gpu.cu.cc", "stock_elman_gpu.cu.cc",
               "pure_lowrank_elman_fused_gpu.cu.cc"]


def build(reference: str = None, force: bool = False) -> str | None:
    reference = reference or REFERENCE_DIR
    libdir = os.path.join(reference, "elman", "cuda", "lib")
    if not os.path.isdir(libdir):
        return LIB if os.path.exists(LIB) else None
    if os.path.exists(LIB) and not force:
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(OUT, exist_ok=True)
    flags = ["-std=c++17", "-x", "cu", "-Xcompiler", "-fPIC", "-O3", "-I" + libdir,
             "-gencode", "arch=compute_100,code=sm_100", "-w"]
    objs = []
    for src in REF_SOURCES:
        obj = os.path.join(OUT, src.replace(".cu.cc", ".o"))
        subprocess.check_call([nvcc, *flags, "-c", os.path.join(libdir, src), "-o", obj])
        objs.append(obj)
    obj = os.path.join(OUT, "ref_cuda_binding.o")
    subprocess.check_call([nvcc, *flags, "-c", os.path.join(HERE, "ref_cuda_binding.cu"), "-o", obj])
    objs.append(obj)
    subprocess.check_call([nvcc, "-shared", "-cudart", "shared", "-o", LIB, *objs, "-lcublas",
                           "-Xlinker", "-rpath,/usr/local/cuda/lib64"])
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=REFERENCE_DIR)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print(build(a.reference, a.force))
