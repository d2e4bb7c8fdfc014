"""nvcc driver and on-disk kernel cache, retargeted to sm_100a.

Same contract as the reference's yan/jit/compiler.py: `build(name, arg_defs, code) -> Runtime`
compiles `code` into `<cache>/kernel.<name>.<hash12>/kernel.so` unless that directory already
holds a valid build (compiler.py:154-254); the hash covers the name, the package's headers, the
code, the compiler and the flags (compiler.py:204-207); files are published with an atomic rename
(compiler.py:131-151,241-250).  Environment: YAN_NVCC_COMPILER, YAN_CACHE_DIR, YAN_PTXAS_VERBOSE,
YAN_JIT_DEBUG, YANJIT_PRINT_NVCC_COMMAND (compiler.py:58,101,195,233).

Differences, all forced by the target:
  * the architecture table knows compute capability 10.0 -> `-gencode=arch=compute_100a,code=sm_100a`
    (the reference stops at 9.0 and appends a malformed flag otherwise, compiler.py:162-179); without
    a visible GPU the target is YAN_JIT_ARCH (default 100a), so kernels cross-compile on a CPU host;
  * `--use_fast_math` is not passed (compiler.py:159-160 passes it globally): the quantizer is
    specified in IEEE round-to-nearest operations.  `build(..., extra_flags=('--use_fast_math',))`
    restores it for a kernel that wants it;
  * no post-compilation SASS rewriting (the reference hashes yan/jit/interleave_ffma.py but never runs it).
"""
from __future__ import annotations

import functools
import hashlib
import os
import re
import shutil
import subprocess
import uuid
from typing import Iterable, Tuple

import torch

from .runtime import Runtime, RuntimeCache
from .template import typename_map

runtime_cache = RuntimeCache()

_ARCH_FLAGS = {
    "80": "-gencode=arch=compute_80,code=sm_80",
    "86": "-gencode=arch=compute_86,code=sm_86",
    "89": "-gencode=arch=compute_89,code=sm_89",
    "90": "-gencode=arch=compute_90a,code=sm_90a",
    "100": "-gencode=arch=compute_100a,code=sm_100a",
}


def hash_to_hex(s: str) -> str:
    return hashlib.md5(s.encode("utf-8")).hexdigest()[0:12]


@functools.lru_cache(maxsize=None)
def get_jit_include_dir() -> str:
    return os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "include"))


@functools.lru_cache(maxsize=None)
def get_yan_version() -> str:
    """Hash of every header under the package's include directory: editing a kernel invalidates the cache."""
    root = get_jit_include_dir()
    assert os.path.exists(root), f"Cannot find include directory {root}"
    digest = hashlib.md5()
    headers = sorted(os.path.join(d, f) for d, _, files in os.walk(root) for f in files if f.endswith((".cuh", ".h")))
    for path in headers:
        with open(path, "rb") as f:
            digest.update(f.read())
    return digest.hexdigest()[0:12]


@functools.lru_cache(maxsize=None)
def get_nvcc_compiler() -> Tuple[str, str]:
    """(path, version) of the first usable nvcc >= 12.8 (the first release with sm_100a)."""
    from torch.utils.cpp_extension import CUDA_HOME
    candidates = []
    if os.getenv("YAN_NVCC_COMPILER"):
        candidates.append(os.getenv("YAN_NVCC_COMPILER"))
    if CUDA_HOME:
        candidates.append(os.path.join(CUDA_HOME, "bin", "nvcc"))
    candidates.append("/usr/local/cuda/bin/nvcc")
    found = shutil.which("nvcc")
    if found:
        candidates.append(found)
    minimum = (12, 8)
    pattern = re.compile(r"release (\d+)\.(\d+)")
    for path in candidates:
        if not os.path.exists(path):
            continue
        try:
            text = subprocess.check_output([path, "--version"], stderr=subprocess.STDOUT, universal_newlines=True)
        except (subprocess.SubprocessError, OSError) as e:
            print(f"Error checking NVCC version for {path}: {e}")
            continue
        match = pattern.search(text)
        if match and (int(match.group(1)), int(match.group(2))) >= minimum:
            return path, f"{match.group(1)}.{match.group(2)}"
        print(f"NVCC {path} is older than {minimum[0]}.{minimum[1]} or its version cannot be read")
    raise RuntimeError("Cannot find an NVCC compiler >= 12.8; set CUDA_HOME or YAN_NVCC_COMPILER.")


@functools.lru_cache(maxsize=None)
def get_default_user_dir() -> str:
    if "YAN_CACHE_DIR" in os.environ:
        path = os.getenv("YAN_CACHE_DIR")
        os.makedirs(path, exist_ok=True)
        return path
    return os.path.expanduser("~/.cache/yan_b200")


def get_tmp_dir() -> str:
    return os.path.join(get_default_user_dir(), "tmp")


def get_cache_dir() -> str:
    return os.path.join(get_default_user_dir(), "cache")


def make_tmp_dir() -> str:
    os.makedirs(get_tmp_dir(), exist_ok=True)
    return get_tmp_dir()


def put(path: str, data, is_binary: bool = False) -> None:
    """Writes `data` to a unique temporary file and renames it over `path` (atomic on one file system)."""
    tmp = os.path.join(make_tmp_dir(), f"file.tmp.{uuid.uuid4()}.{hash_to_hex(path)}")
    with open(tmp, "wb" if is_binary else "w") as f:
        f.write(data)
    try:
        os.replace(tmp, path)
    except OSError:
        shutil.copy2(tmp, path)
        os.unlink(tmp)


def get_arch_flag() -> str:
    if torch.cuda.is_available():
        major, minor = torch.cuda.get_device_capability()
        code = f"{major}{minor}"
        if code not in _ARCH_FLAGS:
            raise RuntimeError(f"Unsupported GPU architecture sm_{code}: this package targets sm_100a")
        return _ARCH_FLAGS[code]
    arch = os.getenv("YAN_JIT_ARCH", "100a")
    return f"-gencode=arch=compute_{arch},code=sm_{arch}"


def get_flags(extra_flags: Iterable[str] = ()) -> list:
    ptxas = "--ptxas-options=--register-usage-level=10" + (",--verbose" if "YAN_PTXAS_VERBOSE" in os.environ else "")
    cxx = ["-fPIC", "-O3", "-Wno-deprecated-declarations", "-Wno-abi"]
    # YAN_JIT_KERNEL: headers add the per-library status word and its two exports (include/gemm/fp8_gemm.cuh)
    return ["-std=c++20", "-O3", "-DYAN_JIT_KERNEL=1", "--expt-relaxed-constexpr", "--expt-extended-lambda", "-lineinfo", get_arch_flag(),
            "-shared", ptxas, "--diag-suppress=177,174,940", f"--compiler-options={','.join(cxx)}", *extra_flags]


def build(name: str, arg_defs: tuple, code: str, extra_flags: Iterable[str] = ()) -> Runtime:
    flags = get_flags(extra_flags)
    include_dirs = [get_jit_include_dir()]

    signature = f"{name}$${get_yan_version()}$${code}$${get_nvcc_compiler()}$${flags}"
    name = f"kernel.{name}.{hash_to_hex(signature)}"
    path = os.path.join(get_cache_dir(), name)

    global runtime_cache
    cached = runtime_cache[path]
    if cached is not None:
        if os.getenv("YAN_JIT_DEBUG", None):
            print(f"Using cached JIT runtime {name} during build")
        return cached

    os.makedirs(path, exist_ok=True)
    put(os.path.join(path, "kernel.args"), ", ".join(f"('{n}', {typename_map[t]})" for n, t in arg_defs) + ("," if len(arg_defs) == 1 else ""))
    src_path = os.path.join(path, "kernel.cu")
    put(src_path, code)

    lib_path = os.path.join(path, "kernel.so")
    tmp_lib = os.path.join(make_tmp_dir(), f"nvcc.tmp.{uuid.uuid4()}.{hash_to_hex(lib_path)}.so")
    command = [get_nvcc_compiler()[0], src_path, "-o", tmp_lib, *flags, *[f"-I{d}" for d in include_dirs]]
    if os.getenv("YAN_JIT_DEBUG", None) or os.getenv("YANJIT_PRINT_NVCC_COMMAND", False):
        print(f"Compiling JIT runtime {name} with command {command}")
    try:
        subprocess.check_call(command)
    except subprocess.CalledProcessError as e:
        raise RuntimeError(f"Failed to compile {src_path}: {e}")
    try:
        os.replace(tmp_lib, lib_path)
    except OSError:
        shutil.copy2(tmp_lib, lib_path)
        os.unlink(tmp_lib)

    runtime_cache[path] = Runtime(path)
    return runtime_cache[path]
