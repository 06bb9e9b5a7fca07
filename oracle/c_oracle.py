"""ctypes binding of oracle/attn_oracle.c (TEST INFRASTRUCTURE ONLY, see that file's header)."""
import ctypes
import math
import os
import subprocess
from concurrent.futures import ThreadPoolExecutor

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libattn_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside it (no-op when the library is up to date)."""
    src = os.path.join(_HERE, "attn_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libattn_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.fray_oracle_attn_fwd.restype = ctypes.c_int
    return _lib


def attn_fwd_c(q, k, v, causal=False, scale=None, block_n=128, threads=None):
    """fp16 [B,H,S,D] CPU tensors (any strides with contiguous D) -> fp16 output, computed by the C oracle."""
    assert q.dtype == k.dtype == v.dtype == torch.half and q.dim() == 4 and not q.is_cuda
    B, H, S, D = q.shape
    for t in (q, k, v):
        assert t.stride(-1) == 1
    out = torch.empty(B, H, S, D, dtype=torch.half)
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    lib = _load()

    def strides(t):
        return (ctypes.c_int64 * 3)(*t.stride()[:3])

    total = B * H * S
    threads = threads or min(os.cpu_count() or 1, max(1, total // 64))
    chunk = (total + threads - 1) // threads
    sq, sk, sv, so = strides(q), strides(k), strides(v), strides(out)

    def work(i):
        lo, hi = i * chunk, min(total, (i + 1) * chunk)
        if lo >= hi:
            return 0
        return lib.fray_oracle_attn_fwd(
            ctypes.c_void_p(q.data_ptr()), ctypes.c_void_p(k.data_ptr()), ctypes.c_void_p(v.data_ptr()),
            ctypes.c_void_p(out.data_ptr()), B, H, S, D, sq, sk, sv, so, int(bool(causal)),
            ctypes.c_float(scale), int(block_n), ctypes.c_long(lo), ctypes.c_long(hi))

    with ThreadPoolExecutor(max_workers=threads) as pool:
        codes = list(pool.map(work, range(threads)))
    assert all(c == 0 for c in codes), f"C oracle rejected its arguments: {codes}"
    return out
