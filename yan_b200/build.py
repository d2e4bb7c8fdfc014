"""Ahead-of-time build of the C-ABI library (yan_b200/lib/libyan_b200.so) for sm_100a.

The reference compiles every kernel at first use (yan/jit/compiler.py:154-254).  The FP8 path is
also shipped prebuilt, because a JIT cache in a home directory does not travel with a source
checkout; the JIT layer in yan_b200/jit remains for user templates and per-shape specialisation.

    python -m yan_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
INCLUDE_DIR = os.path.join(PKG_DIR, "include")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(PKG_DIR, "lib", "obj")
LIB_PATH = os.path.join(LIB_DIR, "libyan_b200.so")

BLOCK_NS = (32, 64, 96, 128, 160, 192, 224, 256)

# No --use_fast_math: the quantizer's divisions and multiplies must be IEEE round-to-nearest.
NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC,-fvisibility=hidden", "-cudart", "static",
    "--diag-suppress=177",
]


def find_nvcc() -> str:
    cand = os.environ.get("YAN_NVCC_COMPILER")
    if cand and os.path.exists(cand):
        return cand
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cand = os.path.join(cuda_home, "bin", "nvcc")
    if os.path.exists(cand):
        return cand
    cand = shutil.which("nvcc")
    if cand:
        return cand
    raise RuntimeError("nvcc not found: set YAN_NVCC_COMPILER or CUDA_HOME")


def _sources() -> List[str]:
    out = []
    for root in (CSRC_DIR, INCLUDE_DIR, os.path.join(os.path.dirname(PKG_DIR), "include")):
        for d, _, files in os.walk(root):
            out += [os.path.join(d, f) for f in files if f.endswith((".cu", ".cuh", ".h"))]
    return out


def is_stale() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    t = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > t for s in _sources())


def _run(cmd: List[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose and r.stdout:
        print(r.stdout, flush=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed ({r.returncode}): {' '.join(cmd)}\n{r.stdout}")


def build_library(force: bool = False, verbose: bool = False) -> str:
    """Compiles the library if it is missing or older than any source.  Returns its path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = find_nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    extra = ["-Xptxas", "-v"] if verbose else []
    jobs = []
    for bn in BLOCK_NS:
        obj = os.path.join(OBJ_DIR, f"gemm_inst_bn{bn}.o")
        jobs.append(([nvcc, *NVCC_FLAGS, *extra, f"-DYAN_BLOCK_N={bn}", f"-I{INCLUDE_DIR}", "-c",
                      os.path.join(CSRC_DIR, "gemm_inst.cu"), "-o", obj], obj))
    for name in ("capi",):
        obj = os.path.join(OBJ_DIR, f"{name}.o")
        jobs.append(([nvcc, *NVCC_FLAGS, *extra, f"-I{INCLUDE_DIR}", "-c", os.path.join(CSRC_DIR, f"{name}.cu"),
                      "-o", obj], obj))
    with ThreadPoolExecutor(max_workers=len(jobs)) as pool:
        list(pool.map(lambda j: _run(j[0], verbose), jobs))
    tmp = LIB_PATH + f".tmp.{os.getpid()}"
    _run([nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp,
          *[j[1] for j in jobs]], verbose)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build_library(force=a.force, verbose=a.verbose))
    sys.exit(0)
