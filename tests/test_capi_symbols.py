"""CPU check of the drop-in boundary: the built library loads without a GPU or driver and exports every
function include/yan_b200.h declares, and the ctypes table in yan_b200/_lib.py covers the same set."""
import ctypes
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "yan_b200.h")


def _declared():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(yan_b200_\w+)\s*\(", text)))


def test_library_builds_loads_and_exports_every_declared_symbol():
    from yan_b200 import build
    path = build.build_library()
    lib = ctypes.CDLL(path)
    names = _declared()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/yan_b200.h but not exported"
    lib.yan_b200_abi_version.restype = ctypes.c_int
    assert lib.yan_b200_abi_version() == 1
    lib.yan_b200_return_code_string.restype = ctypes.c_char_p
    assert b"bad argument" in lib.yan_b200_return_code_string(1)


def test_ctypes_table_matches_header():
    from yan_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared()
    handle = _lib.lib()
    assert handle.yan_b200_fp8_linear_workspace_bytes(64, 2048) == 64 * 2048 + 256 * ((64 * 16 * 4 + 255) // 256)
    assert handle.yan_b200_fp8_linear_workspace_bytes(64, 100) == 0


def test_no_undefined_driver_dependency():
    """The library must not link libcuda (it has to load on a machine without a driver)."""
    from yan_b200 import build
    out = subprocess.check_output(["ldd", build.LIB_PATH], text=True)
    assert "libcuda.so" not in out and "not found" not in out


def test_entry_points_reject_bad_arguments_without_a_gpu():
    """Argument validation happens before any CUDA call, so it is testable on a CPU-only host."""
    from yan_b200 import _lib
    assert _lib.call_rc("yan_b200_gemm_fp8_fp8_bf16_nt", None, None, None, None, None, 0, 128, 128, 128, None, 1, 0) == 1
    assert _lib.call_rc("yan_b200_per_token_cast_to_fp8", None, None, None, 4, 100, 100, 4, None) == 1
    assert _lib.call_rc("yan_b200_per_block_cast_to_fp8", None, None, None, 100, 128, None) == 1
    assert _lib.call_rc("yan_b200_fp8_linear_bf16_static", None, None, None, None, 4096, 128, 4096, 128, None, 1, 0) == 7


def test_header_is_plain_c_and_a_c_host_can_call_the_library(tmp_path):
    """The boundary is a C ABI: the header compiles as C99 with a C compiler, and a C program that binds the library
    with dlopen gets the documented error codes back (no GPU needed: validation precedes any CUDA call)."""
    src = tmp_path / "host.c"
    src.write_text(r'''
#include <dlfcn.h>
#include <stdio.h>
#include "yan_b200.h"
typedef int (*abi_fn)(void);
typedef void (*gemm_fn)(const void*, const void*, const void*, const void*, void*, int, int, int, int, void*, int, int, int*);
typedef void (*allreduce_fn)(void* const*, void* const*, int, int, unsigned long long, unsigned long long, unsigned int,
                             unsigned int, int, int, void*, int*);
int main(int argc, char** argv) {
    void* h = dlopen(argv[1], RTLD_NOW);
    if (!h) { printf("dlopen failed: %s\n", dlerror()); return 2; }
    abi_fn abi = (abi_fn)dlsym(h, "yan_b200_abi_version");
    gemm_fn gemm = (gemm_fn)dlsym(h, "yan_b200_gemm_fp8_fp8_bf16_nt");
    allreduce_fn allreduce = (allreduce_fn)dlsym(h, "yan_b200_allreduce_bf16_two_shot");
    if (!abi || !gemm || !allreduce) return 3;
    int rc = -1, rc2 = -1;
    gemm(0, 0, 0, 0, 0, 0, 128, 128, 128, 0, 1, 0, &rc);
    allreduce(0, 0, 2, 0, 0, 8, 0, 0, 1, 0, 0, &rc2);
    printf("%d %d %d %d\n", abi(), rc, rc2, (int)YAN_B200_BAD_ARGUMENT);
    return 0;
}
''')
    from yan_b200 import build
    exe = tmp_path / "host"
    inc = f"-I{os.path.join(ROOT, 'include')}"
    only_header = tmp_path / "only_header.c"
    only_header.write_text('#include "yan_b200.h"\nint unused_translation_unit_guard;\n')
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", inc, "-fsyntax-only", str(only_header)])
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", inc, str(src), "-o", str(exe), "-ldl"])
    out = subprocess.check_output([str(exe), build.build_library()], text=True).split()
    assert out == ["1", "1", "1", "1"], out
