"""Source generation for JIT kernels.

Mirrors the reference generator's contract (fray/jit/template.py:12-155): an op supplies
its includes, a tuple of ``(name, type)`` argument definitions and a C++ body; the result
is one translation unit exporting ``extern "C" void launch(<args>, int& __return_code)``
where tensors and streams cross the boundary as ``void*`` and are cast to typed pointers
before the body runs.  ``map_ctype`` is the matching Python-side marshalling.
"""
import ctypes
import os
from dataclasses import dataclass
from typing import Any, Dict, Iterable, Tuple

import torch


@dataclass(frozen=True)
class _ArgKind:
    py_name: str    # how the type is written in ``kernel.args`` (evaluated at load time)
    ctype: Any      # ctypes type used when calling ``launch``
    abi_type: str   # type in the exported signature
    body_type: str  # type the body sees (differs from abi_type for pointers)


_KINDS: Dict[Any, _ArgKind] = {
    bool: _ArgKind("bool", ctypes.c_bool, "bool", "bool"),
    int: _ArgKind("int", ctypes.c_int, "int", "int"),
    float: _ArgKind("float", ctypes.c_float, "float", "float"),
    torch.int: _ArgKind("torch.int", ctypes.c_void_p, "void*", "int*"),
    torch.float: _ArgKind("torch.float", ctypes.c_void_p, "void*", "float*"),
    torch.half: _ArgKind("torch.half", ctypes.c_void_p, "void*", "__half*"),
    torch.bfloat16: _ArgKind("torch.bfloat16", ctypes.c_void_p, "void*", "__nv_bfloat16*"),
    torch.float8_e4m3fn: _ArgKind("torch.float8_e4m3fn", ctypes.c_void_p, "void*", "__nv_fp8_e4m3*"),
    torch.cuda.Stream: _ArgKind("torch.cuda.Stream", ctypes.c_void_p, "void*", "cudaStream_t"),
}

# Views of the table under the names the reference exposes.
typename_map: Dict[Any, str] = {t: k.py_name for t, k in _KINDS.items()}
ctype_map: Dict[Any, Any] = {t: k.ctype for t, k in _KINDS.items()}
genc_map: Dict[Any, Tuple[str, str]] = {t: (k.abi_type, k.body_type) for t, k in _KINDS.items()}

_RAW_PREFIX = "__raw_"

_EXPORT_MACRO = """\
#ifdef _WIN32
#define EXPORT_API __declspec(dllexport)
#else
#define EXPORT_API __attribute__((visibility("default")))
#endif
"""

_ALWAYS_INCLUDED = ("<cuda.h>", "<cuda_fp16.h>", "<cuda_bf16.h>", "<cuda_fp8.h>", "<cuda_runtime.h>", "<iostream>")


def map_ctype(value: Any) -> Any:
    """Python value -> ctypes value for one ``launch`` argument (reference: template.py:52-58)."""
    if isinstance(value, torch.Tensor):
        return ctype_map[value.dtype](value.data_ptr())
    if isinstance(value, torch.cuda.Stream):
        return ctype_map[torch.cuda.Stream](value.cuda_stream)
    return ctype_map[type(value)](value)


def cpp_format(template: str, keys: Dict[str, Any]) -> str:
    """Replace ``{KEY}`` markers; all other braces are C++ and stay as they are."""
    text = template
    for key, value in keys.items():
        text = text.replace("{" + str(key) + "}", str(value))
    return text


def generate(includes: Iterable[str], arg_defs: Iterable[Tuple[str, Any]], body: str, epilogue: str = "") -> str:
    """Emit the translation unit for one kernel instance.

    ``epilogue`` (an addition to the reference signature, empty by default) is pasted
    after ``launch`` at file scope; ops use it to export small helpers such as a status
    reader from the same library.
    """
    assert isinstance(includes, (list, tuple))
    arg_defs = tuple(arg_defs)
    system = sorted({*_ALWAYS_INCLUDED, *(i for i in includes if i.startswith("<"))})
    local = sorted({i for i in includes if i.startswith('"')})

    lines = [_EXPORT_MACRO]
    lines += [f"#include {inc}" for inc in system]
    lines.append("")
    lines += [f"#include {inc}" for inc in local]
    lines.append("")

    params = []
    casts = []
    for name, kind in arg_defs:
        abi_type, body_type = genc_map[kind]
        if abi_type == body_type:
            params.append(f"{abi_type} {name}")
        else:
            params.append(f"{abi_type} {_RAW_PREFIX}{name}")
            casts.append(f"    auto {name} = reinterpret_cast<{body_type}>({_RAW_PREFIX}{name});")
    params.append("int& __return_code")

    lines.append(f'extern "C" EXPORT_API void launch({", ".join(params)}) {{')
    lines.append("    // typed views of the raw pointer arguments")
    lines += casts
    lines += [("    " + ln) if ln else ln for ln in body.split("\n")]
    lines.append("}")
    lines.append("")
    if epilogue:
        lines.append(epilogue.rstrip("\n"))
        lines.append("")
    code = "\n".join(lines)

    if os.getenv("FRAY_JIT_DEBUG"):
        print(f"Generated code:\n{code}")
    return code
