"""Host-side JIT boundary: source generation, nvcc build into the hash cache, ctypes marshalling.

Follows the reference's tests/test_jit.py (generate -> build -> launch a host-only body and
compare what it printed with the values passed) but needs no GPU: the body never touches CUDA
and tensors are stood in for by CPU tensors, whose data_ptr() crosses the ABI the same way.
"""
import ctypes
import os

import pytest
import torch

from fray_b200 import jit
from fray_b200.jit import compiler, template
from fray_b200.jit.runtime import Runtime, RuntimeCache


class FakeStream(torch.cuda.Stream if False else object):
    pass


def test_cpp_format_leaves_cpp_braces_alone():
    text = "template<int N> struct A { int x[{N}]; void f() { {BODY} } };"
    out = jit.cpp_format(text, {"N": 4, "BODY": "return;"})
    assert out == "template<int N> struct A { int x[4]; void f() { return; } };"


def test_generate_signature_and_casts():
    args = (("lhs", torch.float8_e4m3fn), ("scale", torch.float), ("out", torch.bfloat16), ("q", torch.half),
            ("n", int), ("alpha", float), ("flag", bool), ("stream", torch.cuda.Stream))
    code = jit.generate(('"flash_attn/host_sm100.cuh"', "<vector>"), args, "\nfoo(lhs, n);\n", epilogue="// tail")
    assert 'extern "C" EXPORT_API void launch(void* __raw_lhs, void* __raw_scale, void* __raw_out, void* __raw_q, ' \
           'int n, float alpha, bool flag, void* __raw_stream, int& __return_code) {' in code
    assert "auto lhs = reinterpret_cast<__nv_fp8_e4m3*>(__raw_lhs);" in code
    assert "auto q = reinterpret_cast<__half*>(__raw_q);" in code
    assert "auto stream = reinterpret_cast<cudaStream_t>(__raw_stream);" in code
    assert "#include <vector>" in code and '#include "flash_attn/host_sm100.cuh"' in code
    assert code.index("#include <cuda.h>") < code.index('#include "flash_attn/host_sm100.cuh"')
    assert code.rstrip().endswith("// tail")
    assert "    foo(lhs, n);" in code


def test_map_ctype():
    t = torch.zeros(4, dtype=torch.half)
    assert template.map_ctype(t).value == t.data_ptr()
    assert isinstance(template.map_ctype(3), ctypes.c_int)
    assert isinstance(template.map_ctype(0.5), ctypes.c_float)
    assert isinstance(template.map_ctype(True), ctypes.c_bool)


def test_nvcc_found_and_new_enough():
    path, version = jit.get_nvcc_compiler()
    assert os.path.exists(path)
    assert tuple(int(p) for p in version.split(".")) >= (12, 8)


def test_build_call_and_cache(tmp_path, monkeypatch, capfd):
    monkeypatch.setenv("FRAY_CACHE_DIR", str(tmp_path))
    args = (("lhs", torch.half), ("rhs", torch.float), ("count", int), ("ratio", float), ("flag", bool))
    body = "\n".join([
        "",
        "std::cout << reinterpret_cast<uint64_t>(lhs) << std::endl;",
        "std::cout << reinterpret_cast<uint64_t>(rhs) << std::endl;",
        "std::cout << count << ' ' << ratio << ' ' << flag << std::endl;",
        "__return_code = count == 7 ? 0 : 42;",
        ""])
    code = jit.generate((), args, body)
    func = jit.build("test_func", args, code)
    assert func.path.startswith(str(tmp_path))
    assert Runtime.is_path_valid(func.path)
    with open(os.path.join(func.path, "kernel.args")) as f:
        assert f.read() == "('lhs', torch.half), ('rhs', torch.float), ('count', int), ('ratio', float), ('flag', bool)"

    a = torch.empty(1, dtype=torch.half)
    b = torch.empty(1, dtype=torch.float)
    capfd.readouterr()
    assert func(a, b, 7, 0.5, True) == 0
    out = capfd.readouterr().out
    assert out == f"{a.data_ptr()}\n{b.data_ptr()}\n7 0.5 1\n"
    assert func(a, b, 8, 0.5, True) == 42  # the return code really comes back

    # wrong dtype / wrong python type / wrong arity are caught before the call
    with pytest.raises(AssertionError):
        func(b, b, 7, 0.5, True)
    with pytest.raises(AssertionError):
        func(a, b, 7.0, 0.5, True)
    with pytest.raises(AssertionError):
        func(a, b, 7, 0.5)

    # same source -> same directory, no rebuild; a fresh RuntimeCache adopts it from disk
    stamp = os.path.getmtime(os.path.join(func.path, "kernel.so"))
    assert jit.build("test_func", args, code) is func
    monkeypatch.setattr(compiler, "runtime_cache", RuntimeCache())
    again = jit.build("test_func", args, code)
    assert again is not func and again.path == func.path
    assert os.path.getmtime(os.path.join(func.path, "kernel.so")) == stamp
    # different source -> different directory
    other = jit.build("test_func", args, code.replace("42", "43"))
    assert other.path != func.path


def test_build_failure_raises(tmp_path, monkeypatch):
    monkeypatch.setenv("FRAY_CACHE_DIR", str(tmp_path))
    args = (("n", int),)
    with pytest.raises(RuntimeError, match="Failed to compile"):
        jit.build("broken", args, jit.generate((), args, "\nthis is not C++;\n"))


def test_put_is_atomic_and_leaves_no_temp(tmp_path, monkeypatch):
    monkeypatch.setenv("FRAY_CACHE_DIR", str(tmp_path))
    target = tmp_path / "x.txt"
    compiler.put(str(target), "one")
    compiler.put(str(target), "two")
    assert target.read_text() == "two"
    assert os.listdir(compiler.get_tmp_dir()) == []


def test_cache_key_ignores_checkout_location():
    flags = " ".join(compiler.get_nvcc_flags())
    assert "-I" not in flags and "compute_100a" in flags and "-lineinfo" in flags
