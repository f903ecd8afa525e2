"""Builds ``libasrq_b200.so`` in-tree with nvcc for sm_100a.

    python -m asrq_b200.build            # incremental (skips if up to date)
    python -m asrq_b200.build --force

nvcc cross-compiles, so this works on a machine without a GPU.  The library is a
plain C-ABI shared object (see ``include/asrq_b200.h``); it links the CUDA runtime
statically and needs no libcuda at link time (the one driver entry point it uses is
looked up at run time).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libasrq_b200.so")
OBJ_DIR = os.path.join(PKG, "build")

SOURCES = ["api.cu", "gemv_a16.cu", "gemv_a16_splitk.cu", "gemv_a16_staged.cu", "gemm_a16_tc.cu", "gemm_a16_tc2.cu", "gemm_a16_skinny.cu", "act_quant.cu", "glue.cu", "offline.cu", "dense_head.cu", "w4a4_mma.cu", "w4a4_tc.cu"]
HEADERS = ["common.cuh", "tcgen05.cuh", "dequant.cuh", os.path.join("..", "..", "include", "asrq_b200.h")]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return os.path.join(cand, "bin", "nvcc")
    nvcc = shutil.which("nvcc")
    if not nvcc:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return nvcc


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> str:
    """``trace`` compiles with -DASRQ_TRACE: kernels record pipeline clock marks into the workspace when the
    library option "trace" is set (a development build; the shipped library carries no trace code)."""
    nvcc = find_nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.normpath(os.path.join(CSRC, h)) for h in HEADERS]
    objs = []
    procs = []
    for src in SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if not force and _newer(o, [s] + headers):
            continue
        cmd = [nvcc] + NVCC_FLAGS + (["-DASRQ_TRACE"] if trace else []) + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for src, pr in procs:
        out, _ = pr.communicate()
        if pr.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose:
            print(out)
    if force or procs or not _newer(LIB, objs):
        cmd = [nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
        r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv or "--trace" in sys.argv, verbose="-v" in sys.argv, trace="--trace" in sys.argv)
    print(path)
