"""nvcc-backed JIT build with a content-addressed on-disk cache.

Same contract as the reference builder (fray/jit/compiler.py:165-281): the cache key is a
hash over the kernel name, the header tree, the generated source, the compiler and its
flags; a build lands atomically in ``<cache>/kernel.<name>.<hash>/`` as ``kernel.cu``,
``kernel.args`` and ``kernel.so`` and is adopted by later processes.  Differences, all
deliberate: the only target is sm_100a (the reference's table stops at sm_90a and its
fallback flag is malformed, compiler.py:177-190), there is no SASS post-processing step,
and include paths stay out of the key so a cache built in one checkout is valid in a
copy of it elsewhere.
"""
import functools
import hashlib
import os
import re
import shutil
import subprocess
import uuid
from typing import Tuple

from .runtime import Runtime, RuntimeCache
from .template import typename_map

runtime_cache = RuntimeCache()

_MIN_NVCC = (12, 8)  # first toolkit that knows compute_100a
_ARCH_FLAG = "-gencode=arch=compute_100a,code=sm_100a"


def hash_to_hex(s: str) -> str:
    return hashlib.md5(s.encode("utf-8")).hexdigest()[:12]


@functools.lru_cache(maxsize=None)
def get_jit_include_dir() -> str:
    return os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "include"))


@functools.lru_cache(maxsize=None)
def get_fray_version() -> str:
    """Hash of every header under the JIT include tree (reference: compiler.py:43-64)."""
    root = get_jit_include_dir()
    assert os.path.isdir(root), f"Cannot find Fray include directory {root}"
    md5 = hashlib.md5()
    found = []
    for base, _, files in os.walk(root):
        found += [os.path.join(base, f) for f in files if f.endswith((".cuh", ".h"))]
    for path in sorted(found):
        md5.update(os.path.relpath(path, root).encode())
        with open(path, "rb") as f:
            md5.update(f.read())
    return md5.hexdigest()[:12]


def _version_tuple(text: str) -> Tuple[int, ...]:
    return tuple(int(p) for p in text.split("."))


@functools.lru_cache(maxsize=None)
def get_nvcc_compiler() -> Tuple[str, str]:
    """(path, version) of the first usable nvcc: $FRAY_NVCC_COMPILER, $CUDA_HOME, /usr/local/cuda, PATH."""
    candidates = []
    if os.getenv("FRAY_NVCC_COMPILER"):
        candidates.append(os.getenv("FRAY_NVCC_COMPILER"))
    for home in (os.getenv("CUDA_HOME"), os.getenv("CUDA_PATH"), "/usr/local/cuda"):
        if home:
            candidates.append(os.path.join(home, "bin", "nvcc"))
    on_path = shutil.which("nvcc")
    if on_path:
        candidates.append(on_path)

    pattern = re.compile(r"release (\d+\.\d+)")
    for path in candidates:
        if not os.path.exists(path):
            continue
        try:
            out = subprocess.check_output([path, "--version"], stderr=subprocess.STDOUT, universal_newlines=True)
        except (subprocess.SubprocessError, OSError):
            continue
        match = pattern.search(out)
        if match and _version_tuple(match.group(1)) >= _MIN_NVCC:
            return path, match.group(1)
    raise RuntimeError(
        f"Cannot find an nvcc >= {_MIN_NVCC[0]}.{_MIN_NVCC[1]} (needed for sm_100a); "
        "set CUDA_HOME or FRAY_NVCC_COMPILER."
    )


def get_default_user_dir() -> str:
    """$FRAY_CACHE_DIR, else a ``_jit_cache`` directory inside the package so prebuilt kernels ship with it."""
    path = os.getenv("FRAY_CACHE_DIR")
    if not path:
        path = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "_jit_cache"))
        try:
            os.makedirs(path, exist_ok=True)
            if not os.access(path, os.W_OK):
                raise OSError
        except OSError:
            path = os.path.expanduser("~/.cache/fray")
    os.makedirs(path, exist_ok=True)
    return path


def get_tmp_dir() -> str:
    return os.path.join(get_default_user_dir(), "tmp")


def get_cache_dir() -> str:
    return os.path.join(get_default_user_dir(), "cache")


def make_tmp_dir() -> str:
    os.makedirs(get_tmp_dir(), exist_ok=True)
    return get_tmp_dir()


def put(path: str, data, is_binary: bool = False) -> None:
    """Write ``data`` to ``path`` through a private temporary file and an atomic rename."""
    tmp = os.path.join(make_tmp_dir(), f"file.tmp.{uuid.uuid4()}.{hash_to_hex(path)}")
    with open(tmp, "wb" if is_binary else "w") as f:
        f.write(data)
    os.replace(tmp, path)


def get_nvcc_flags() -> Tuple[str, ...]:
    # No --register-usage-level override: the reference's level 10 trades instruction-level
    # parallelism for registers, which the warp-specialised kernel budgets itself (setmaxnreg).
    ptxas = "--ptxas-options=--warn-on-spills" + (",--verbose" if "FRAY_PTXAS_VERBOSE" in os.environ else "")
    extra = tuple(os.getenv("FRAY_NVCC_EXTRA_FLAGS", "").split())  # e.g. -DFRAY_ATTN_TRACE (part of the cache key)
    return (
        "-std=c++17", "-O3", "--expt-relaxed-constexpr", "--expt-extended-lambda", "-lineinfo",
        _ARCH_FLAG, "-shared", ptxas, "--diag-suppress=177,174,940",
        # -fno-gnu-unique: function-local statics of inline functions and templates (per-device bookkeeping in
        # the launchers) must stay private to each built library; as GNU unique symbols they would be shared
        # by every library the process loads, whatever the dlopen flags
        "--compiler-options=-fPIC,-O3,-Wno-deprecated-declarations,-Wno-abi,-fno-gnu-unique", *extra,
    )


def _check_device_arch() -> None:
    """Refuse to build for a visible GPU that is not a compute-capability 10.x part."""
    try:
        import torch
        if torch.cuda.is_available():
            major, minor = torch.cuda.get_device_capability()
            if major != 10:
                raise RuntimeError(f"fray_b200 targets sm_100a only; the current device is sm_{major}{minor}")
    except ImportError:
        pass


def kernel_dir_for(name: str, code: str) -> str:
    flags = get_nvcc_flags()
    signature = f"{name}$${get_fray_version()}$${code}$${get_nvcc_compiler()}$${flags}"
    return os.path.join(get_cache_dir(), f"kernel.{name}.{hash_to_hex(signature)}")


def build(name: str, arg_defs: tuple, code: str) -> Runtime:
    path = kernel_dir_for(name, code)
    cached = runtime_cache[path]
    if cached is not None:
        if os.getenv("FRAY_JIT_DEBUG"):
            print(f"Using cached JIT runtime {os.path.basename(path)} during build")
        return cached

    _check_device_arch()
    os.makedirs(path, exist_ok=True)
    src_path = os.path.join(path, "kernel.cu")
    put(os.path.join(path, "kernel.args"), ", ".join(f"('{n}', {typename_map[t]})" for n, t in arg_defs))
    put(src_path, code)

    lib_path = os.path.join(path, "kernel.so")
    tmp_lib = os.path.join(make_tmp_dir(), f"nvcc.tmp.{uuid.uuid4()}.{hash_to_hex(lib_path)}.so")
    command = [get_nvcc_compiler()[0], src_path, "-o", tmp_lib, *get_nvcc_flags(), f"-I{get_jit_include_dir()}"]
    if os.getenv("FRAY_JIT_DEBUG") or os.getenv("FRAYJIT_PRINT_NVCC_COMMAND"):
        print(f"Compiling JIT runtime {os.path.basename(path)} with command {command}")
    proc = subprocess.run(command, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, universal_newlines=True)
    if proc.returncode != 0:
        raise RuntimeError(f"Failed to compile {src_path}:\n{proc.stdout}")
    if proc.stdout and ("FRAY_PTXAS_VERBOSE" in os.environ or os.getenv("FRAY_JIT_DEBUG")):
        print(proc.stdout)
    os.replace(tmp_lib, lib_path)

    runtime_cache[path] = Runtime(path)
    return runtime_cache[path]
