"""Builds ``libfastnn_cuda.so`` in-tree with nvcc for sm_100a (no GPU needed to compile).

    python -m fastnn_b200.build [--force] [--verbose]

The library has no Python or torch dependency: it is the C-ABI artefact a Rust
``build.rs`` would produce for fastnn's ``src/backend/cuda``.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "csrc", "build")
LIB = os.path.join(HERE, "libfastnn_cuda.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

NVCC = os.environ.get("FNN_NVCC", "/usr/local/cuda/bin/nvcc")
HOST_CXX = os.environ.get("FNN_HOST_CXX", "/usr/bin/g++")

CUDA_SOURCES = ["api.cu", "repack.cu", "qmm_rows.cu", "qmm_mma.cu", "qmm_mma8.cu", "qmm_tc.cu", "plan_ops.cu"]
HOST_SOURCES = ["quantize_host.cpp"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-ccbin", HOST_CXX, "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr",
]
# The host quantizer must keep every f32 rounding of the reference: no FMA contraction.
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fopenmp", "-ffp-contract=off", "-fno-fast-math"]


def _deps_mtime() -> float:
    paths = [os.path.join(CSRC, f) for f in os.listdir(CSRC)
             if f.endswith((".cu", ".cuh", ".cpp", ".h"))]
    paths.append(os.path.join(INCLUDE, "fastnn_cuda.h"))
    paths.append(os.path.abspath(__file__))
    return max(os.path.getmtime(p) for p in paths)


def _run(cmd, verbose):
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stdout + proc.stderr)
    return proc.stdout + proc.stderr


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source for sm_100a and link the shared library in-tree."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _deps_mtime():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    jobs = []
    objs = []
    for src in CUDA_SOURCES:
        obj = os.path.join(OBJ, src + ".o")
        objs.append(obj)
        jobs.append([NVCC, *NVCC_FLAGS, "-I", INCLUDE, "-c", os.path.join(CSRC, src), "-o", obj])
    for src in HOST_SOURCES:
        obj = os.path.join(OBJ, src + ".o")
        objs.append(obj)
        jobs.append([HOST_CXX, *HOST_FLAGS, "-I", INCLUDE, "-c", os.path.join(CSRC, src), "-o", obj])
    with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
        logs = list(pool.map(lambda c: _run(c, verbose), jobs))
    with open(os.path.join(OBJ, "ptxas.log"), "w") as f:
        f.write("\n".join(logs))
    _run([NVCC, "-shared", "-ccbin", HOST_CXX, "-o", LIB, *objs, "-Xcompiler", "-fopenmp",
          "-lgomp"], verbose)
    return LIB


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
