"""Build the CUDA library in-tree with nvcc (sm_100a only).

    python -m elman_b200.build            # build if sources are newer than the .so
    python -m elman_b200.build --force
    python -m elman_b200.build --microbench   # also the standalone program under csrc/microbench

The result, elman_b200/lib/libelman_b200.so, is a plain C-ABI shared library
(see include/elman_b200.h); it does not link against PyTorch.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libelman_b200.so")
SOURCES = ["api.cu", "gemm_simt.cu", "gemm_tc.cu", "rec_simt.cu", "rec_tc.cu", "lowrank_tc.cu", "extras.cu", "layer_ops.cu", "train_ops.cu", "spectral.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr", "--extended-lambda",
    "-Xcompiler", "-fPIC,-O3,-Wall,-Wno-unused-function",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def needs_build() -> bool:
    if not os.path.exists(LIB):
        return True
    t = os.path.getmtime(LIB)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh", ".h"))]
    deps.append(os.path.join(HERE, "..", "include", "elman_b200.h"))
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and not needs_build():
        return LIB
    nvcc = find_nvcc()
    os.makedirs(LIBDIR, exist_ok=True)
    objdir = os.path.join(LIBDIR, "obj")
    os.makedirs(objdir, exist_ok=True)
    procs = []
    objs = []
    for src in SOURCES:
        obj = os.path.join(objdir, src.replace(".cu", ".o"))
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, pr in procs:
        out, _ = pr.communicate()
        text = out.decode(errors="replace")
        if pr.returncode != 0:
            failed = True
            sys.stderr.write(f"nvcc failed on {src}:\n{text}\n")
        elif verbose or text.strip():
            sys.stderr.write(text)
    if failed:
        raise RuntimeError("nvcc compilation failed")
    # Shared cudart: inside a PyTorch process the runtime PyTorch already loaded is
    # the one that gets bound, so streams and the current device are common state.
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "shared",
           "-o", LIB, *objs, "-Xlinker", "-rpath,/usr/local/cuda/lib64", "-ldl", "-lpthread"]
    subprocess.check_call(cmd)
    return LIB


def build_microbench() -> str:
    """The standalone measurement program under csrc/microbench (MMA issue rate, cluster exchange)."""
    src = os.path.join(CSRC, "microbench", "mma_issue_and_cluster_exchange.cu")
    exe = os.path.join(LIBDIR, "mma_issue_and_cluster_exchange")
    if os.path.exists(exe) and os.path.getmtime(exe) >= max(
            os.path.getmtime(src), os.path.getmtime(os.path.join(CSRC, "sm100_ptx.cuh"))):
        return exe
    os.makedirs(LIBDIR, exist_ok=True)
    subprocess.check_call([find_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O3",
                           "-std=c++17", "-lineinfo", "-o", exe, src])
    return exe


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
    if "--microbench" in sys.argv:
        print(build_microbench())
