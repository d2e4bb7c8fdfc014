"""Code generation for JIT-compiled launch stubs.

Same contract as the reference's yan/jit/template.py: `generate(includes, arg_defs, body)` returns
a translation unit whose only export is

    extern "C" void launch(<one parameter per arg_def>, int& __return_code)

with tensors arriving as `void*` (cast to their element pointer type under the argument's own
name), `torch.cuda.Stream` as `cudaStream_t`, and bool/int/float by value (template.py:12-49,
130-149).  `cpp_format` substitutes `{KEY}` markers without touching other braces (template.py:61-66).
"""
from __future__ import annotations

import ctypes
import os
from typing import Any, Dict, Iterable, Tuple

import torch

# Python type / torch dtype -> (spelling inside kernel.args, ctypes type, C parameter type, C++ type in the body)
_TYPE_TABLE: Dict[Any, Tuple[str, Any, str, str]] = {
    bool: ("bool", ctypes.c_bool, "bool", "bool"),
    int: ("int", ctypes.c_int, "int", "int"),
    float: ("float", ctypes.c_float, "float", "float"),
    torch.int: ("torch.int", ctypes.c_void_p, "void*", "int*"),
    torch.float: ("torch.float", ctypes.c_void_p, "void*", "float*"),
    torch.half: ("torch.half", ctypes.c_void_p, "void*", "__half*"),
    torch.bfloat16: ("torch.bfloat16", ctypes.c_void_p, "void*", "__nv_bfloat16*"),
    torch.float8_e4m3fn: ("torch.float8_e4m3fn", ctypes.c_void_p, "void*", "__nv_fp8_e4m3*"),
    torch.uint8: ("torch.uint8", ctypes.c_void_p, "void*", "uint8_t*"),
    torch.cuda.Stream: ("torch.cuda.Stream", ctypes.c_void_p, "void*", "cudaStream_t"),
}

typename_map: Dict[Any, str] = {k: v[0] for k, v in _TYPE_TABLE.items()}
ctype_map: Dict[Any, Any] = {k: v[1] for k, v in _TYPE_TABLE.items()}
genc_map: Dict[Any, Tuple[str, str]] = {k: (v[2], v[3]) for k, v in _TYPE_TABLE.items()}

_SYSTEM_INCLUDES = ("<cstdint>", "<cuda.h>", "<cuda_bf16.h>", "<cuda_fp16.h>", "<cuda_fp8.h>", "<cuda_runtime.h>",
                    "<iostream>")

_EXPORT_MACRO = """
#ifdef _WIN32
#define EXPORT_API __declspec(dllexport)
#else
#define EXPORT_API __attribute__((visibility("default")))
#endif

"""


def map_ctype(value: Any) -> Any:
    """Python value -> ctypes value: tensors by data pointer, streams by handle."""
    if isinstance(value, torch.Tensor):
        return ctype_map[value.dtype](value.data_ptr())
    if isinstance(value, torch.cuda.Stream):
        return ctype_map[torch.cuda.Stream](value.cuda_stream)
    return ctype_map[type(value)](value)


def cpp_format(template: str, keys: Dict[str, Any]) -> str:
    """Replaces each `{KEY}` by `str(value)`; every other brace of the C++ text is left alone."""
    text = template
    for key, value in keys.items():
        text = text.replace("{" + key + "}", str(value))
    return text


def generate(includes: Iterable[str], arg_defs: Iterable[Tuple], body: str) -> str:
    assert isinstance(includes, (list, tuple))
    sys_inc = sorted(set(_SYSTEM_INCLUDES) | {i for i in includes if i.startswith("<")})
    pkg_inc = sorted({i for i in includes if i.startswith('"')})

    parts = [_EXPORT_MACRO]
    parts.append("".join(f"#include {i}\n" for i in sys_inc) + "\n")
    if pkg_inc:
        parts.append("".join(f"#include {i}\n" for i in pkg_inc) + "\n")

    params, casts = [], []
    for name, kind in arg_defs:
        c_type, cpp_type = genc_map[kind]
        if c_type == cpp_type:
            params.append(f"{c_type} {name}")
        else:
            params.append(f"{c_type} __raw_{name}")
            casts.append(f"    auto {name} = reinterpret_cast<{cpp_type}>(__raw_{name});\n")
    params.append("int& __return_code")

    parts.append('extern "C" EXPORT_API void launch(' + ", ".join(params) + ") {\n")
    parts.append("    // Cast raw types (if needed)\n" + "".join(casts))
    parts.append("\n".join(("    " + line) if line else line for line in body.split("\n")))
    parts.append("}\n\n")
    code = "".join(parts)

    if os.getenv("YAN_JIT_DEBUG", None):
        print(f"Generated code:\n{code}")
    return code
