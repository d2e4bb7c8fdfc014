"""bf16 -> e4m3 quantizers feeding the FP8 GEMM (CUDA only; kernels in include/quant/fp8_cast.cuh).

The reference names the per-token-group activation quantizer as part of this path but holds no
code for it; the function names follow the project the reference says it derives from
(README.md:24).  Outputs are laid out exactly as the GEMM consumes them
(yan/jit_kernels/gemm.py:23-27, yan/include/gemm/fp8_gemm.cuh:59).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .. import _lib


def _stream_ptr() -> ctypes.c_void_p:
    return _lib.current_stream_ptr()


def per_token_cast_to_fp8(x: torch.Tensor, out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
                          ) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [M, K] -> (e4m3 [M, K], fp32 scales [M, K/128]); scale = max(amax, 1e-4)/448 per 1x128 group.

    The scale tensor is column-major (stride (1, M)): M-contiguous per k-block, so the GEMM takes
    it without a transpose.  Rows of `x` may be strided (x.stride(0) >= K, multiple of 8).
    """
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2
    m, k = x.shape
    assert m > 0 and k > 0 and k % 128 == 0, "K must be a positive multiple of 128"
    assert x.stride(1) == 1 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
    if out is None:
        q = torch.empty((m, k), dtype=torch.float8_e4m3fn, device=x.device)
        s = torch.empty((k // 128, m), dtype=torch.float32, device=x.device).t()
    else:
        q, s = out
        assert q.shape == (m, k) and q.dtype == torch.float8_e4m3fn and q.is_contiguous()
        assert s.shape == (m, k // 128) and s.dtype == torch.float32 and s.stride(0) == 1 and s.stride(1) >= m
    _lib.call("yan_b200_per_token_cast_to_fp8", x.data_ptr(), q.data_ptr(), s.data_ptr(), m, k, x.stride(0),
              s.stride(1) if k > 128 else m, _stream_ptr())
    return q, s


def per_block_cast_to_fp8(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [N, K] -> (e4m3 [N, K], fp32 scales [N/128, K/128]); one scale per 128x128 block."""
    assert w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous()
    n, k = w.shape
    assert n % 128 == 0 and k % 128 == 0 and n > 0 and k > 0
    q = torch.empty((n, k), dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((n // 128, k // 128), dtype=torch.float32, device=w.device)
    _lib.call("yan_b200_per_block_cast_to_fp8", w.data_ptr(), q.data_ptr(), s.data_ptr(), n, k, _stream_ptr())
    return q, s
