"""TEST INFRASTRUCTURE ONLY -- ctypes loader for the C restatement (oracle/fp8_oracle.c).

Parity unpinned (see the header of fp8_oracle.c).  `build()` compiles liboracle.so with
gcc next to the source when it is missing or stale.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Tuple

import numpy as np

_DIR = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_DIR, "fp8_oracle.c")
_LIB = os.path.join(_DIR, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    if force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(_SRC):
        subprocess.check_call(["make", "-C", _DIR, "-B", "liboracle.so"], stdout=subprocess.DEVNULL)
    return _LIB


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _lib.yan_oracle_e4m3_decode.restype = ctypes.c_float
        _lib.yan_oracle_e4m3_decode.argtypes = [ctypes.c_uint8]
        _lib.yan_oracle_e4m3_encode.restype = ctypes.c_uint8
        _lib.yan_oracle_e4m3_encode.argtypes = [ctypes.c_float, ctypes.c_int]
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return ctypes.c_void_p(a.ctypes.data)


def e4m3_decode(code: int) -> float:
    return float(lib().yan_oracle_e4m3_decode(code))


def e4m3_encode(v: float, saturate: bool = True) -> int:
    return int(lib().yan_oracle_e4m3_encode(ctypes.c_float(v), int(saturate)))


def per_token_cast_to_fp8(a_bf16_bits: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    """uint16 bf16 bits [M, K] -> (uint8 codes [M, K], fp32 scales [K/128, M] k-block-major)."""
    m, k = a_bf16_bits.shape
    q = np.empty((m, k), np.uint8)
    s = np.empty((k // 128, m), np.float32)
    lib().yan_oracle_per_token_cast_to_fp8(_p(a_bf16_bits), ctypes.c_int64(m), ctypes.c_int64(k), _p(q), _p(s))
    return q, s


def per_block_cast_to_fp8(b_bf16_bits: np.ndarray) -> Tuple[np.ndarray, np.ndarray]:
    n, k = b_bf16_bits.shape
    q = np.empty((n, k), np.uint8)
    s = np.empty((n // 128, k // 128), np.float32)
    lib().yan_oracle_per_block_cast_to_fp8(_p(b_bf16_bits), ctypes.c_int64(n), ctypes.c_int64(k), _p(q), _p(s))
    return q, s


def ref_gemm(qa: np.ndarray, sa_kmajor: np.ndarray, qb: np.ndarray, sb: np.ndarray) -> np.ndarray:
    """-> uint16 bf16 bits [M, N]."""
    m, k = qa.shape
    n = qb.shape[0]
    d = np.empty((m, n), np.uint16)
    lib().yan_oracle_ref_gemm(_p(qa), _p(sa_kmajor), _p(qb), _p(sb), ctypes.c_int64(m), ctypes.c_int64(n),
                              ctypes.c_int64(k), _p(d), ctypes.c_int64(n))
    return d
