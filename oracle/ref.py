"""TEST INFRASTRUCTURE ONLY -- torch-CPU oracle for the FP8 fine-grained-scaled GEMM path.

PARITY UNPINNED: the reference has no finished FP8 GEMM, no quantizer, no torch
dequantize-and-matmul path and no golden vectors for it (yan/jit_kernels/gemm.py:1-31
is a template string; yan/include/gemm/fp8_gemm.cuh:187-197 ends mid-statement;
tests/test_jit.py:37 only checks dtype plumbing).  This module restates the arithmetic
fixed by the workload definition (scale = amax/448, 1x128 groups for A, 128x128 blocks
for B, fp32 accumulation, bf16 output) with the layouts recoverable from the
reference fragments (fp8_gemm.cuh:41,55-61; gemm.py:23-27).  It is cross-checked
against the independent C restatement in oracle/fp8_oracle.c and the committed
fixtures in tests/golden/.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module.  The product package never does.

Pinned operation sequence of the quantizers (every step one fp32 round-to-nearest op):
    amax   = max |x| over the group            (exact)
    amax_c = max(amax, 1e-4)                    (guards all-zero groups)
    inv    = 448 / amax_c
    q      = e4m3_rne(x * inv)                  (|x*inv| <= 448(1+2^-23) -> 448, no overflow)
    scale  = amax_c / 448
"""
from __future__ import annotations

from typing import Tuple

import torch

GROUP = 128
FP8_MAX = 448.0
AMAX_FLOOR = 1e-4


def per_token_cast_to_fp8(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16/fp32 [M, K] -> (e4m3 [M, K], fp32 scales [M, K/128]).

    The returned scale tensor is *column-major* (stride (1, M)): M-contiguous per
    k-block, the layout the GEMM consumes (fp8_gemm.cuh:59, gemm.py:25).
    """
    assert x.dim() == 2 and x.size(1) % GROUP == 0
    m, k = x.shape
    xf = x.float().view(m, k // GROUP, GROUP)
    amax = xf.abs().amax(dim=2).clamp_min(AMAX_FLOOR)            # [M, K/128]
    inv = torch.tensor(FP8_MAX, dtype=torch.float32) / amax
    q = (xf * inv.unsqueeze(2)).to(torch.float8_e4m3fn).view(m, k)
    scale = amax / torch.tensor(FP8_MAX, dtype=torch.float32)
    scale_cm = scale.t().contiguous().t()                         # shape [M, K/128], stride (1, M)
    return q, scale_cm


def per_block_cast_to_fp8(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16/fp32 [N, K] -> (e4m3 [N, K], fp32 scales [N/128, K/128])."""
    assert w.dim() == 2 and w.size(0) % GROUP == 0 and w.size(1) % GROUP == 0
    n, k = w.shape
    wf = w.float().view(n // GROUP, GROUP, k // GROUP, GROUP)
    amax = wf.abs().amax(dim=(1, 3)).clamp_min(AMAX_FLOOR)        # [N/128, K/128]
    inv = torch.tensor(FP8_MAX, dtype=torch.float32) / amax
    q = (wf * inv.view(n // GROUP, 1, k // GROUP, 1)).to(torch.float8_e4m3fn).view(n, k)
    scale = amax / torch.tensor(FP8_MAX, dtype=torch.float32)
    return q, scale.contiguous()


def dequant_a(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    m, k = q.shape
    return (q.float().view(m, k // GROUP, GROUP) * scale.view(m, k // GROUP, 1)).view(m, k)


def dequant_b(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    n, k = q.shape
    return (q.float().view(n // GROUP, GROUP, k // GROUP, GROUP)
            * scale.view(n // GROUP, 1, k // GROUP, 1)).view(n, k)


def ref_gemm_f32(lhs: Tuple[torch.Tensor, torch.Tensor], rhs: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
    """dequantize both operands to fp32, matmul in fp32; result left in fp32."""
    return dequant_a(*lhs) @ dequant_b(*rhs).t()


def ref_gemm(lhs, rhs) -> torch.Tensor:
    """The CPU dequantize-and-matmul path: bf16( dequant(A) @ dequant(B)^T )."""
    return ref_gemm_f32(lhs, rhs).to(torch.bfloat16)


def ref_gemm_k_split(lhs, rhs, world: int) -> torch.Tensor:
    """Restates the K-split arithmetic: each of `world` shards (cut on multiples of 128)
    yields a bf16 partial D, and the partials are summed.  The order and intermediate
    rounding of a bf16 allreduce are implementation-defined (ring, tree or in-switch), so
    this oracle sums the bf16 partials in fp32 and rounds to bf16 once; a bf16 ring adds at
    most one extra bf16 rounding per hop on top of this."""
    qa, sa = lhs
    qb, sb = rhs
    k = qa.size(1)
    assert k % (GROUP * world) == 0
    ks = k // world
    acc = None
    for r in range(world):
        sl = slice(r * ks, (r + 1) * ks)
        sl_s = slice(r * ks // GROUP, (r + 1) * ks // GROUP)
        part = ref_gemm((qa[:, sl], sa[:, sl_s]), (qb[:, sl], sb[:, sl_s]))
        acc = part.float() if acc is None else acc + part.float()
    return acc.to(torch.bfloat16)


# ---------------------------------------------------------------------------------------
# error metrics
# ---------------------------------------------------------------------------------------

def rel_frobenius(x: torch.Tensor, y: torch.Tensor) -> float:
    x, y = x.double(), y.double()
    return float((x - y).norm() / y.norm().clamp_min(1e-30))


def max_abs_err(x: torch.Tensor, y: torch.Tensor) -> float:
    return float((x.double() - y.double()).abs().max())


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y>/(|x|^2+|y|^2), the reference's similarity metric (yan/utils.py:109-113)."""
    x, y = x.double(), y.double()
    den = (x * x + y * y).sum()
    return float(1 - 2 * (x * y).sum() / den) if den != 0 else 0.0


def bf16_ulp_at(v: float) -> float:
    """Spacing of bf16 values in the binade of |v| (8 significant bits)."""
    import math
    if v == 0:
        return 0.0
    return 2.0 ** (math.floor(math.log2(abs(v))) - 7)


# ---------------------------------------------------------------------------------------
# synthetic workloads (seeded; these *are* the benchmark inputs -- no public dataset is involved)
# ---------------------------------------------------------------------------------------

def make_inputs(m: int, n: int, k: int, seed: int = 0, outliers: bool = False):
    """A = randn(M,K) -> bf16; B = 0.02 randn(N,K) -> bf16.  With `outliers`, a fixed random
    1 % of A's K channels is multiplied by 20 (the decode workload)."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g, dtype=torch.float32)
    b = torch.randn(n, k, generator=g, dtype=torch.float32) * 0.02
    if outliers:
        go = torch.Generator().manual_seed(seed)
        cols = torch.randperm(k, generator=go)[: k // 100]
        a[:, cols] *= 20.0
    return a.to(torch.bfloat16), b.to(torch.bfloat16)
