"""Operator-level helpers with the reference's names (yan/jit_kernels/utils.py:6-85)."""
from __future__ import annotations

import torch

_num_sms = None


def set_num_sms(num_sms: int) -> None:
    """Caps the persistent grid of every GEMM launch (e.g. to leave SMs to a concurrent collective)."""
    global _num_sms
    assert 0 < num_sms <= torch.cuda.get_device_properties(device="cuda").multi_processor_count
    _num_sms = num_sms


def get_num_sms() -> int:
    """Current cap; the device's SM count when never set."""
    global _num_sms
    if _num_sms is None:
        _num_sms = torch.cuda.get_device_properties(device="cuda").multi_processor_count
    return _num_sms


def ceil_div(x: int, y: int) -> int:
    return (x + y - 1) // y


def get_m_alignment_for_contiguous_layout() -> int:
    """Row alignment of each group in the contiguous grouped layout: one 128-row tile
    (yan/jit_kernels/utils.py:46-55)."""
    return 128


def get_col_major_tensor(x: torch.Tensor) -> torch.Tensor:
    """Column-major version of a 2D (or batched 3D) tensor, shape unchanged: stride (1, rows).
    Returns `x` itself when it already has that layout (yan/jit_kernels/utils.py:58-85)."""
    assert x.dim() in (2, 3)
    if x.dim() == 2 and x.stride(0) == 1 and x.stride(1) == x.shape[0]:
        return x  # the usual case on the hot path: nothing to build
    remove_dim = False
    if x.dim() == 2:
        x, remove_dim = x.unsqueeze(0), True
    b, m, n = x.shape
    if x.stride(1) == 1 and x.stride(2) == m and (b == 1 or x.stride(0) == m * n):
        return x.squeeze(0) if remove_dim else x
    out = x.transpose(1, 2).contiguous().transpose(1, 2)
    return out.squeeze(0) if remove_dim else out
