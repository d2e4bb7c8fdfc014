"""Loader and caller of one JIT-compiled kernel directory.

Same contract as the reference's yan/jit/runtime.py: a kernel lives in a directory holding
`kernel.cu`, `kernel.args` and `kernel.so` (runtime.py:20-28); `Runtime(path)(*args)` checks the
argument types against `kernel.args`, converts them with `map_ctype`, calls `launch` with the return
code by reference and returns that code (runtime.py:30-68).  `RuntimeCache` memoises by path.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from .template import map_ctype

_REQUIRED = ("kernel.cu", "kernel.args", "kernel.so")


class Runtime:
    def __init__(self, path: str) -> None:
        self.path = path
        self.lib = None
        self.args = None
        assert self.is_path_valid(self.path)

    @staticmethod
    def is_path_valid(path: str) -> bool:
        return os.path.isdir(path) and all(os.path.exists(os.path.join(path, f)) for f in _REQUIRED)

    def _load(self) -> None:
        self.lib = ctypes.CDLL(os.path.join(self.path, "kernel.so"))
        with open(os.path.join(self.path, "kernel.args"), "r") as f:
            # The file is written by `build` from typename_map: a tuple of ('name', type) pairs.
            self.args = eval(f.read(), {"torch": torch, "__builtins__": {"bool": bool, "int": int, "float": float}})

    def __call__(self, *args) -> int:
        if self.lib is None or self.args is None:
            self._load()
        assert len(args) == len(self.args), f"Expected {len(self.args)} arguments, got {len(args)}"
        cargs = []
        for arg, (name, kind) in zip(args, self.args):
            if isinstance(arg, torch.Tensor):
                assert arg.dtype == kind, f"Expected tensor dtype `{kind}` for `{name}`, got `{arg.dtype}`"
            else:
                assert isinstance(arg, kind), f"Expected built-in type `{kind}` for `{name}`, got `{type(arg)}`"
            cargs.append(map_ctype(arg))
        return_code = ctypes.c_int(0)
        self.lib.launch(*cargs, ctypes.byref(return_code))
        return return_code.value

    def read_device_status(self, reset: bool = True) -> int:
        """Status word of this kernel library (0 = no bounded device-side wait ran out), for libraries whose headers
        export one; 0 for the others.  Synchronises the device."""
        if self.lib is None:
            return 0
        try:
            fn = self.lib.yan_jit_read_device_status
        except AttributeError:
            return 0
        status = ctypes.c_int(0)
        rc = fn(ctypes.byref(status), int(reset))
        if rc != 0:
            raise RuntimeError(f"yan_jit_read_device_status failed with code {rc}")
        return status.value

    def set_wait_timeout_ns(self, timeout_ns: int) -> None:
        if self.lib is None:
            self._load()
        try:
            fn = self.lib.yan_jit_set_wait_timeout_ns
        except AttributeError:
            return
        fn.argtypes = [ctypes.c_ulonglong]
        fn(int(timeout_ns))


class RuntimeCache:
    def __init__(self) -> None:
        self.cache: Dict[str, Runtime] = {}

    def __getitem__(self, path: str) -> Optional[Runtime]:
        hit = self.cache.get(path)
        if hit is not None:
            return hit
        if Runtime.is_path_valid(path):
            self.cache[path] = Runtime(path)
            return self.cache[path]
        return None

    def __setitem__(self, path: str, runtime: Runtime) -> None:
        self.cache[path] = runtime
