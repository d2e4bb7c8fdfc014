"""TEST / BASELINE INFRASTRUCTURE ONLY -- builds the one piece of the reference that compiles for Blackwell.

comm/gemm.cu of the reference is a stand-alone CUTLASS program (fp16 x fp16 -> fp32 GEMM for sm_100, tile 256x128x64,
cluster 2x2, comm/gemm.cu:93-145) that needs nothing but the CUTLASS headers, which this image ships inside a Python
package.  It is compiled from the source where it lies, into oracle/_ref/ (not tracked), and serves as a same-GPU
yardstick for the FP8 kernel in the one-GPU benchmark: same M, N, K, the reference's own timing loop
(comm/gemm.cu:421-443).  It is never part of the product and never runs on more than one GPU (its cluster loads are
multicast loads).  The reference's FP8 path itself cannot be built (its kernel stops mid-statement).

    python -m oracle.build_ref        # no-op when the reference tree or the headers are missing
"""
from __future__ import annotations

import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "ref_gemm_sm100")
# the reference checkout: YAN_REFERENCE_ROOT, or a directory named `reference` beside this repository
REFERENCE_ROOT = os.environ.get("YAN_REFERENCE_ROOT",
                                os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))


def _cutlass_root():
    for pkg in ("flashinfer",):
        try:
            mod = __import__(pkg)
        except Exception:
            continue
        root = os.path.join(os.path.dirname(mod.__file__), "data", "cutlass")
        if os.path.isdir(os.path.join(root, "include", "cutlass")) and os.path.isdir(os.path.join(root, "tools", "util", "include")):
            return root
    return None


def build(force: bool = False, verbose: bool = False) -> str | None:
    """Returns the binary's path, or None when it cannot be built here."""
    src = os.path.join(REFERENCE_ROOT, "comm", "gemm.cu")
    if not os.path.exists(src):
        return OUT if os.path.exists(OUT) else None
    if os.path.exists(OUT) and not force and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    root = _cutlass_root()
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    if root is None or not os.path.exists(nvcc):
        return None
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    cmd = [nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "--expt-relaxed-constexpr",
           "--expt-extended-lambda", "-w", f"-I{root}/include", f"-I{root}/tools/util/include",
           f"-I{os.path.join(REFERENCE_ROOT, 'comm')}", src, "-o", OUT]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        if verbose:
            print(r.stdout[-2000:], flush=True)
        return None
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
