"""ctypes binding of the prebuilt C-ABI library (include/yan_b200.h).

There is no fallback: if the library is missing the import of any operator raises, and every
operator raises on a non-zero return code.  Arguments are marshalled the way the reference's
runtime does (yan/jit/runtime.py:54-68, yan/jit/template.py:53-58): tensors as
`c_void_p(tensor.data_ptr())`, streams as `c_void_p(stream.cuda_stream)`, the return code by
reference as the last argument.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
# YAN_B200_LIBRARY points at an alternative build of the same ABI (e.g. one compiled with other flags).
LIB_PATH = os.environ.get("YAN_B200_LIBRARY") or os.path.join(_PKG_DIR, "lib", "libyan_b200.so")

_P = ctypes.c_void_p
_I = ctypes.c_int
_RC = ctypes.POINTER(ctypes.c_int)

# name -> (restype, argtypes); mirrors include/yan_b200.h one to one.
SIGNATURES = {
    "yan_b200_abi_version": (_I, []),
    "yan_b200_return_code_string": (ctypes.c_char_p, [_I]),
    "yan_b200_gemm_fp8_fp8_bf16_nt": (None, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _RC]),
    "yan_b200_gemm_tail_workspace_bytes": (ctypes.c_size_t, [_I]),
    "yan_b200_gemm_fp8_fp8_bf16_nt_tail": (None, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _P, ctypes.c_size_t, _RC]),
    "yan_b200_gemm_fp8_fp8_f32_nt": (None, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _RC]),
    "yan_b200_gemm_fp8_fp8_e4m3_nt": (None, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _RC]),
    "yan_b200_m_grouped_gemm_fp8_fp8_bf16_nt_contiguous": (None, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _RC]),
    "yan_b200_m_grouped_gemm_fp8_fp8_bf16_nt_masked": (None, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _RC]),
    "yan_b200_per_token_cast_to_fp8": (None, [_P, _P, _P, _I, _I, _I, _I, _P, _RC]),
    "yan_b200_per_block_cast_to_fp8": (None, [_P, _P, _P, _I, _I, _P, _RC]),
    "yan_b200_ipc_export": (None, [_P, _P, ctypes.POINTER(ctypes.c_ulonglong), _RC]),
    "yan_b200_ipc_open": (None, [_P, ctypes.POINTER(ctypes.c_void_p), _RC]),
    "yan_b200_ipc_close": (None, [_P, _RC]),
    "yan_b200_allreduce_bf16_two_shot": (None, [ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), _I, _I,
                                                ctypes.c_ulonglong, ctypes.c_ulonglong, ctypes.c_uint, ctypes.c_uint, _I,
                                                _I, _P, _RC]),
    "yan_b200_allreduce_bf16_in_switch": (None, [_P, ctypes.POINTER(ctypes.c_void_p), _I, _I, ctypes.c_ulonglong,
                                                 ctypes.c_ulonglong, ctypes.c_uint, ctypes.c_uint, _I, _I, _P, _RC]),
    "yan_b200_gemm_fp8_fp8_bf16_nt_scatter": (None, [_P, _P, _P, _P, ctypes.POINTER(ctypes.c_void_p), _I, _I, _I, _I, _I, _I, _P,
                                                     _I, _I, _RC]),
    "yan_b200_allreduce_bf16_gather_staged": (None, [_P, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p), _I, _I,
                                                     _I, _I, ctypes.c_uint, ctypes.c_uint, _I, _P, _RC]),
    "yan_b200_fp8_linear_workspace_bytes": (ctypes.c_size_t, [_I, _I]),
    "yan_b200_fp8_linear_bf16": (None, [_P, _P, _P, _P, _P, ctypes.c_size_t, _I, _I, _I, _I, _P, _I, _I, _RC]),
    "yan_b200_fp8_linear_bf16_static": (None, [_P, _P, _P, _P, _I, _I, _I, _I, _P, _I, _I, _RC]),
    "yan_b200_read_device_status": (None, [_RC, _I, _RC]),
    "yan_b200_wait_probe": (None, [ctypes.c_ulonglong, _P, _RC]),
    "yan_b200_set_programmatic_dependent_launch": (None, [_I]),
    "yan_b200_set_wait_timeout_ns": (None, [ctypes.c_ulonglong]),
    "yan_b200_set_clock_probe": (None, [_P]),
    "yan_b200_set_collective_timeout_ns": (None, [ctypes.c_ulonglong]),
}

# YAN_B200_STATIC_SCRATCH_MAX_ELEMENTS of include/yan_b200.h
STATIC_SCRATCH_MAX_ELEMENTS = 8 << 20

_lib: Optional[ctypes.CDLL] = None


class YanB200Error(RuntimeError):
    def __init__(self, fn: str, code: int, text: str) -> None:
        super().__init__(f"{fn} failed with return code {code}: {text}")
        self.code = code


def lib() -> ctypes.CDLL:
    """Loads libyan_b200.so (once).  Raises if it has not been built: `python -m yan_b200.build`."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -m yan_b200.build` "
                              "(there is no CPU or PyTorch fallback for this path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def call(name: str, *args) -> None:
    """Calls a `void f(..., int* return_code)` entry point and raises on a non-zero code."""
    rc = ctypes.c_int(0)
    getattr(lib(), name)(*args, ctypes.byref(rc))
    if rc.value != 0:
        raise YanB200Error(name, rc.value, lib().yan_b200_return_code_string(rc.value).decode())


def call_rc(name: str, *args) -> int:
    """Same call, returning the code instead of raising (what the tuner needs)."""
    rc = ctypes.c_int(0)
    getattr(lib(), name)(*args, ctypes.byref(rc))
    return rc.value


def current_stream_ptr() -> ctypes.c_void_p:
    """The current CUDA stream of the current device as a raw handle.  Uses torch's direct binding where it exists:
    building a torch.cuda.Stream object per call costs several microseconds, which shows on small launches."""
    import torch
    raw = getattr(torch._C, "_cuda_getCurrentRawStream", None)
    if raw is not None:
        return ctypes.c_void_p(raw(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
