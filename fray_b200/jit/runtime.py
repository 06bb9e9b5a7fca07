"""Loading and calling built kernels.

A built kernel is a directory holding ``kernel.cu``, ``kernel.args`` and ``kernel.so``
(reference layout: fray/jit/runtime.py:21-28).  ``Runtime`` loads the library on first
use, checks every argument against ``kernel.args`` and calls the exported ``launch``
with a trailing ``int*`` that receives the return code (reference: runtime.py:30-68).
"""
import ctypes
import os
from typing import Dict, Optional

import torch

from .template import ctype_map, map_ctype

_REQUIRED_FILES = ("kernel.cu", "kernel.args", "kernel.so")


class Runtime:
    def __init__(self, path: str) -> None:
        self.path = path
        self.lib = None
        self.args = None
        assert self.is_path_valid(path), f"{path} is not a complete kernel directory"

    @staticmethod
    def is_path_valid(path: str) -> bool:
        return os.path.isdir(path) and all(os.path.exists(os.path.join(path, f)) for f in _REQUIRED_FILES)

    def _load(self) -> None:
        self.lib = ctypes.CDLL(os.path.join(self.path, "kernel.so"))
        self.lib.launch.restype = None
        with open(os.path.join(self.path, "kernel.args"), "r") as f:
            # kernel.args is a Python literal such as "('Q', torch.half), ('n', int)".
            self.args = eval(f.read(), {"__builtins__": {}}, {"torch": torch, "int": int, "float": float, "bool": bool})
        if self.args and not isinstance(self.args[0], tuple):
            self.args = (self.args,)
        # Declared argument types let callers on a fast path pass plain Python numbers.
        self.lib.launch.argtypes = [ctype_map[kind] for _, kind in self.args] + [ctypes.POINTER(ctypes.c_int)]

    def __call__(self, *args) -> int:
        if self.lib is None:
            self._load()
        assert len(args) == len(self.args), f"Expected {len(self.args)} arguments, got {len(args)}"
        cargs = []
        for value, (name, kind) in zip(args, self.args):
            if isinstance(value, torch.Tensor):
                assert value.dtype == kind, f"Expected tensor dtype `{kind}` for `{name}`, got `{value.dtype}`"
            else:
                assert isinstance(value, kind), f"Expected built-in type `{kind}` for `{name}`, got `{type(value)}`"
            cargs.append(map_ctype(value))
        return_code = ctypes.c_int(0)
        self.lib.launch(*cargs, ctypes.byref(return_code))
        return return_code.value

    def raw_launch(self):
        """The bound ``launch`` symbol itself, for callers that have validated and marshalled once already.

        Arguments are plain numbers (pointers and streams as integers) followed by
        ``ctypes.byref(ctypes.c_int)`` for the return code; no per-argument checks are made.
        """
        if self.lib is None:
            self._load()
        return self.lib.launch

    def symbol(self, name: str):
        """An extra exported symbol of the library, or None when it has none by that name."""
        if self.lib is None:
            self._load()
        try:
            return getattr(self.lib, name)
        except AttributeError:
            return None


class RuntimeCache:
    """path -> Runtime, adopting complete kernel directories already on disk (runtime.py:71-86)."""

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
