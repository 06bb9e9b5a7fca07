"""``flash_attn_cute(Q, K, V, Output)`` - fp16 (or bf16) attention forward written in place.

Drop-in for the reference op (fray/jit_kernels/flashattn_cute.py:15-45): four fp16 CUDA
tensors of identical shape ``[B, H, S, D]``, result stored into ``Output``, launch on
the current stream, nothing returned.  The 4-positional call behaves as in the
reference (non-causal, scale ``1/sqrt(D)``); ``causal``, ``scale`` and ``lse`` are keyword-only
extensions, and K / V may carry fewer heads than Q (grouped-query attention).  Unlike the reference, strided views whose last dimension is contiguous are
consumed and produced through their strides (no hidden copies, and a non-contiguous
``Output`` really receives the result).
"""
import ctypes
import math
import os
from typing import Any, Dict, Optional, Tuple

import torch

from .tuner import jit_tuner

includes = ('"flash_attn/flash_attn_sm100.cuh"',)
# bf16 tensors get libraries of their own: this header, sorted ahead of the other one by the generator,
# switches the operand type of the whole translation unit.
includes_bf16 = ('"flash_attn/bf16_operands.cuh"', *includes)

template = """
// Templated args from Python JIT call
fray::flash_attn_sm100<{KIND}, {D}, {BLOCK_N}, {STAGES}, {POLY}>(
    Q, K, V, O, batch_size, num_heads, seq_len,
    q_stride_b, q_stride_h, q_stride_s, k_stride_b, k_stride_h, k_stride_s,
    v_stride_b, v_stride_h, v_stride_s, o_stride_b, o_stride_h, o_stride_s,
    num_kv_heads, seq_len_kv, Lse, causal, scale, stream, __return_code);
"""

# Exported next to `launch`: blocking read (and optional clear) of the device status words.
epilogue = """
extern "C" EXPORT_API int fray_attn_status(int* out4, int clear) {
    return fray::read_attn_status(out4, clear != 0);
}
extern "C" EXPORT_API void fray_attn_kernel_info(int* out4) {
    out4[0] = {KIND}; out4[1] = {D}; out4[2] = {BLOCK_N}; out4[3] = {STAGES} + 16 * {POLY};
}
extern "C" EXPORT_API int fray_attn_operand_is_bf16(void) {
    return fray::kOperandIsBf16;
}
#ifdef FRAY_ATTN_TRACE
extern "C" EXPORT_API int fray_attn_trace_read(unsigned int* out, int max_words) {
    return fray::sm100::read_attn_trace(out, max_words);
}
#endif
"""

_STRIDE_NAMES = tuple(f"{t}_stride_{d}" for t in "qkvo" for d in "bhs")

arg_defs = (
    ("Q", torch.half), ("K", torch.half), ("V", torch.half), ("O", torch.half),
    ("batch_size", int), ("num_heads", int), ("seq_len", int),
    *((n, int) for n in _STRIDE_NAMES),
    ("num_kv_heads", int), ("seq_len_kv", int), ("Lse", torch.float),
    ("causal", bool), ("scale", float), ("stream", torch.cuda.Stream),
)

# the same argument table with bf16 tensors (the generated `launch` prototype is identical: raw pointers)
arg_defs_bf16 = tuple((n, torch.bfloat16 if t is torch.half else t) for n, t in arg_defs)

SUPPORTED_HEAD_DIMS = (64, 128)

# Return codes of `launch` (flash_attn/host_sm100.cuh).
_RC_TEXT = {
    1: "bad shape", 2: "null or misaligned pointer", 3: "unsupported stride",
    5: "cuTensorMapEncodeTiled not resolvable", 6: "tensor map rejected by the driver",
    7: "could not raise the dynamic shared memory limit", 8: "kernel launch failed",
    9: "this kernel kind has no grouped K/V heads or LSE output",
}
_RC_TENSOR_MAP = 6


def tuning_space(d: int) -> Tuple[Dict[str, Any], ...]:
    """Candidate kernels for head dim ``d``.

    KIND: 0 single-role, 1 warp-specialised (whole 128-key steps), 2 persistent, 3 split rows, 4 correction
    group as softmax helper, 5 warp-specialised with 64-key steps; BLOCK_N / STAGES: KV tile and ring depth;
    POLY: exponential mode of kinds 1-4 (flash_attn/flash_attn_sm100.cuh).
    """
    space = [
        {"KIND": 1, "BLOCK_N": 128, "STAGES": 4, "POLY": 0},   # warp-specialised, two tiles per CTA, whole 128-key steps
        {"KIND": 5, "BLOCK_N": 128, "STAGES": 4, "POLY": 0},   # ... 64-key steps in two score buffers per tile
        {"KIND": 6, "BLOCK_N": 128, "STAGES": 2 if d == 128 else 4, "POLY": 0},   # one tile per CTA, three score buffers (STAGES: K ring)
        {"KIND": 0, "BLOCK_N": 128, "STAGES": 1, "POLY": 0},
        {"KIND": 0, "BLOCK_N": 64, "STAGES": 1, "POLY": 0},
    ]
    if d == 128:
        space.insert(3, {"KIND": 7, "BLOCK_N": 128, "STAGES": 4, "POLY": 0})  # three score buffers on a CTA pair (cta_group::2)
    forced = os.getenv("FRAY_ATTN_FORCE")  # e.g. "KIND=0,BLOCK_N=64,STAGES=1"
    if forced:
        point = {"POLY": 0}
        point.update({kv.split("=")[0].strip(): int(kv.split("=")[1]) for kv in forced.split(",")})
        return (point,)
    return tuple(space)


def _seq_class(seq_len: int, units: int) -> str:
    """Coarse workload class the tuner memoises on: sequence bucket and whether the grid fills the GPU."""
    s_bucket = 1 << max(7, (max(seq_len, 1) - 1).bit_length())
    return f"S{min(s_bucket, 16384)}_{'big' if units * seq_len >= 148 * 256 else 'small'}"


def _usable_strides(t: torch.Tensor) -> bool:
    if t.stride(-1) != 1 and t.shape[-1] > 1:
        return False
    if t.data_ptr() % 16 != 0:
        return False
    return all(t.shape[i] == 1 or (t.stride(i) > 0 and t.stride(i) % 8 == 0 and t.stride(i) < 2 ** 31)
               for i in range(3))


def prebuild(head_dims=SUPPORTED_HEAD_DIMS, prune: bool = False):
    """Compile every point of the tuning space ahead of time and return the kernel directories.

    With ``prune`` the cache directory is also cleared of attention kernels that no longer
    belong to the space (left over from older headers).
    """
    import shutil
    from ..jit import build, cpp_format, generate
    from ..jit.compiler import get_cache_dir
    paths = []
    for d in head_dims:
        for point in tuning_space(d):
            keys = {"D": d, **point}
            code = generate(includes, arg_defs, cpp_format(template, keys), cpp_format(epilogue, keys))
            paths.append(build("flash_attn_cute", arg_defs, code).path)
        for point in tuning_space(d):  # bf16 operands: the tuning space only
            keys = {"D": d, **point}
            code = generate(includes_bf16, arg_defs_bf16, cpp_format(template, keys), cpp_format(epilogue, keys))
            paths.append(build("flash_attn_cute", arg_defs_bf16, code).path)
    if prune:
        for entry in os.listdir(get_cache_dir()):
            full = os.path.join(get_cache_dir(), entry)
            if entry.startswith("kernel.flash_attn_cute.") and full not in paths:
                shutil.rmtree(full, ignore_errors=True)
    return paths


_last_runtime = None
# Warm-call fast path: (shapes, strides, dtypes, devices, causal, scale) -> (runtime, launch symbol, int args).
# Everything the slow path validates is a function of that key, so a hit only has to marshal the
# four pointers and the stream.
_fast_path: Dict[Any, Any] = {}


def flash_attn_status(clear: bool = True) -> Tuple[int, int, int, int]:
    """Synchronise and return the device status words of the most recently used kernel library.

    ``(0, 0, 0, 0)`` means healthy.  A non-zero first word is the code of the first wait
    that ran out inside a kernel; the other words are the block indices and an iteration
    number.  The status is sticky: until cleared, later launches of that library return
    immediately without computing.
    """
    if _last_runtime is None:
        return (0, 0, 0, 0)
    fn = _last_runtime.symbol("fray_attn_status")
    assert fn is not None, "kernel library does not export fray_attn_status"
    out = (ctypes.c_int * 4)()
    err = fn(out, ctypes.c_int(1 if clear else 0))
    if err != 0:
        raise RuntimeError(f"reading the attention status failed with CUDA error {err}")
    return tuple(out)


_no_lse: Dict[Any, torch.Tensor] = {}


def flash_attn_cute(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, Output: torch.Tensor, *,
                    causal: bool = False, scale: Optional[float] = None, lse: Optional[torch.Tensor] = None) -> None:
    """See the module docstring.  Extensions beyond the reference's call:

    ``K`` and ``V`` may be ``[B, H_kv, S_k, D]`` with ``H_kv`` a divisor of ``H``: query head ``h`` then attends
    to K/V head ``h // (H // H_kv)`` (grouped-query / multi-query attention), and ``S_k`` may differ from the
    number of queries (cross attention, or new queries against a longer cache); with ``causal`` query ``i``
    sees keys ``0..i``, the top-left alignment of torch's ``is_causal``.
    All four tensors may be bf16 instead of fp16 (P is then rounded to bf16 too; accumulation stays fp32).
    ``lse``: optional contiguous fp32 CUDA tensor ``[B, H, S]`` that receives ``log(sum_j exp(scale * q_i.k_j))``
    over the keys row ``i`` may see, the quantity needed to merge partial attention results.
    """
    global _last_runtime
    fast_key = (Q.shape, Q.stride(), K.shape, K.stride(), V.shape, V.stride(), Output.shape, Output.stride(),
                Q.dtype, K.dtype, V.dtype, Output.dtype, Q.device, K.device, V.device, Output.device,
                bool(causal), scale, os.getenv("FRAY_ATTN_FORCE"),
                None if lse is None else (lse.shape, lse.stride(), lse.dtype, lse.device))
    hit = _fast_path.get(fast_key)
    if hit is not None:
        runtime, launch, ints, sm_scale = hit
        rc = ctypes.c_int(0)
        launch(Q.data_ptr(), K.data_ptr(), V.data_ptr(), Output.data_ptr(), *ints,
               0 if lse is None else lse.data_ptr(), bool(causal), sm_scale,
               torch.cuda.current_stream().cuda_stream, ctypes.byref(rc))
        if rc.value == 0:
            _last_runtime = runtime
            return
        # e.g. a misaligned data pointer this time: let the checked path deal with it
    assert Q.dim() == 4 and K.dim() == 4, "expected [B, H, S, D] tensors"
    batch_size, num_heads, seq_len, d = Q.shape
    num_kv_heads = K.shape[1]
    assert Q.shape == Output.shape and K.shape == V.shape
    seq_len_kv = K.shape[2]
    assert K.shape == (batch_size, num_kv_heads, seq_len_kv, d), "K and V must match Q in batch and head dim"
    assert num_kv_heads > 0 and num_heads % num_kv_heads == 0, "the number of K/V heads must divide the number of Q heads"
    assert Q.dtype == K.dtype == V.dtype == Output.dtype and Q.dtype in (torch.half, torch.bfloat16)
    bf16 = Q.dtype is torch.bfloat16
    assert Q.device.type == "cuda", "flash_attn_cute has no CPU path"
    assert Q.device == K.device == V.device == Output.device
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.device == Q.device and lse.is_contiguous()
        assert lse.shape == (batch_size, num_heads, seq_len), "lse must be [B, H, S]"
    if d not in SUPPORTED_HEAD_DIMS:
        raise ValueError(f"head dim {d} not supported (supported: {SUPPORTED_HEAD_DIMS})")
    if batch_size == 0 or num_heads == 0 or seq_len == 0:
        return
    assert seq_len_kv > 0, "attention over zero keys is undefined"

    q, k, v = (t if _usable_strides(t) else t.contiguous() for t in (Q, K, V))
    out = Output if _usable_strides(Output) else torch.empty_like(Output, memory_format=torch.contiguous_format)

    stream = torch.cuda.current_stream()
    sm_scale = float(scale) if scale is not None else 1.0 / math.sqrt(d)

    lse_arg = lse
    if lse_arg is None:  # a null pointer for the library: an empty tensor's data pointer is 0
        lse_arg = _no_lse.get(Q.device)
        if lse_arg is None:
            lse_arg = _no_lse[Q.device] = torch.empty(0, dtype=torch.float32, device=Q.device)

    def pack(q, k, v, out):
        strides = tuple(int(t.stride(i)) if t.shape[i] > 1 else 8 for t in (q, k, v, out) for i in range(3))
        return (q, k, v, out, int(batch_size), int(num_heads), int(seq_len), *strides, int(num_kv_heads),
                int(seq_len_kv), lse_arg, bool(causal), sm_scale, stream)

    args = pack(q, k, v, out)
    runtime = jit_tuner.compile_and_tune(
        name="flash_attn_cute",
        keys={"D": d, "CAUSAL": int(bool(causal)), "CLASS": _seq_class(max(seq_len, seq_len_kv), batch_size * num_heads),
              "FORCED": os.getenv("FRAY_ATTN_FORCE", ""), **({"BF16": 1} if bf16 else {})},
        space=tuning_space(d),
        includes=includes_bf16 if bf16 else includes,
        arg_defs=arg_defs_bf16 if bf16 else arg_defs,
        template=template,
        args=args,
        epilogue=epilogue,
    )
    _last_runtime = runtime

    rc = runtime(*args)
    if rc == _RC_TENSOR_MAP and not all(t.is_contiguous() for t in (q, k, v, out)):
        # The layout cannot be described to the copy engine: fall back to packed copies.
        q, k, v = (t.contiguous() for t in (q, k, v))
        if not out.is_contiguous():
            out = torch.empty_like(Output, memory_format=torch.contiguous_format)
        rc = runtime(*pack(q, k, v, out))
    if rc != 0:
        raise RuntimeError(f"flash_attn_cute launch failed with code {rc} ({_RC_TEXT.get(rc, 'unknown')})")
    if q is Q and k is K and v is V and out is Output:
        # no copies were needed: remember how to launch this layout directly
        _fast_path[fast_key] = (runtime, runtime.raw_launch(), args[4:4 + 3 + 12 + 2], sm_scale)
    if out is not Output:
        Output.copy_(out)


_host_staging: Dict[Any, Any] = {}


def flash_attn_cute_host(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, Output: torch.Tensor, *,
                         causal: bool = False, scale: Optional[float] = None, chunks: Optional[int] = None,
                         device: Optional[torch.device] = None) -> None:
    """``flash_attn_cute`` for operands in pinned HOST memory: result written to the pinned ``Output``.

    No counterpart in the reference (its op asserts CUDA tensors, fray/jit_kernels/flashattn_cute.py:17-20);
    this is the call a host-side caller of the C ABI makes.  The B*H independent (batch, head) units are cut
    into ``chunks`` slices (default 8) that move through two sets of device staging buffers on three streams:
    while slice c is computed, slice c+1 is copied in and slice c-1 is copied out, so the two directions of
    the host link run at the same time and the kernel hides behind them.  Work is ordered after the current
    stream's earlier work, and the current stream waits for the last copy-out: as with the device op, the
    result is valid for work queued on the current stream afterwards (or after a synchronize), not at return.
    """
    assert all(t.device.type == "cpu" and t.is_pinned() for t in (Q, K, V, Output)), "operands must be pinned host tensors"
    assert Q.dim() == 4 and Q.shape == K.shape == V.shape == Output.shape and Q.dtype == torch.half
    assert all(t.is_contiguous() for t in (Q, K, V, Output)), "host operands must be contiguous"
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    units = Q.shape[0] * Q.shape[1]
    Q, K, V, Output = (t.view(units, t.shape[2], t.shape[3]) for t in (Q, K, V, Output))
    n = max(1, min(units, chunks if chunks else 8))
    bounds = [(units * c) // n for c in range(n + 1)]
    rows = max(b1 - b0 for b0, b1 in zip(bounds, bounds[1:]))
    key = (dev, rows, tuple(Q.shape[1:]))
    st = _host_staging.get(key)
    if st is None:
        st = {
            "bufs": [[torch.empty((rows,) + tuple(Q.shape[1:]), dtype=torch.half, device=dev) for _ in range(4)] for _ in range(2)],
            "s_in": torch.cuda.Stream(device=dev), "s_out": torch.cuda.Stream(device=dev),
        }
        _host_staging.clear()  # one shape at a time: the buffers are as large as the operands' slices
        _host_staging[key] = st
    s_in, s_out = st["s_in"], st["s_out"]
    cur = torch.cuda.current_stream(dev)
    start = torch.cuda.Event()
    start.record(cur)
    s_in.wait_event(start)
    s_out.wait_event(start)
    computed = [None, None]   # per buffer set: kernel of the slice that last used it has finished
    drained = [None, None]    # ... and its result has left the device
    for c, (b0, b1) in enumerate(zip(bounds, bounds[1:])):
        dq, dk, dv, do = (t[: b1 - b0] for t in st["bufs"][c & 1])   # [units in slice, S, D]
        if computed[c & 1] is not None:
            s_in.wait_event(computed[c & 1])      # inputs of slice c-2 are no longer read
        with torch.cuda.stream(s_in):
            dq.copy_(Q[b0:b1], non_blocking=True)
            dk.copy_(K[b0:b1], non_blocking=True)
            dv.copy_(V[b0:b1], non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(s_in)
        cur.wait_event(arrived)
        if drained[c & 1] is not None:
            cur.wait_event(drained[c & 1])        # output buffer of slice c-2 has been copied out
        flash_attn_cute(dq.unsqueeze(0), dk.unsqueeze(0), dv.unsqueeze(0), do.unsqueeze(0), causal=causal, scale=scale)
        computed[c & 1] = torch.cuda.Event()
        computed[c & 1].record(cur)
        s_out.wait_event(computed[c & 1])
        with torch.cuda.stream(s_out):
            Output[b0:b1].copy_(do, non_blocking=True)
            drained[c & 1] = torch.cuda.Event()
            drained[c & 1].record(s_out)
    for ev in drained:
        if ev is not None:
            cur.wait_event(ev)
