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
from collections import OrderedDict
from typing import Any, Dict, Optional, Tuple

import torch

from .tuner import jit_tuner

includes = ('"flash_attn/flash_attn_sm100.cuh"',)
# bf16 tensors get libraries of their own: this header, sorted ahead of the other one by the generator,
# switches the operand type of the whole translation unit.
includes_bf16 = ('"flash_attn/bf16_operands.cuh"', *includes)

template = """
// Templated args from Python JIT call
fray::flash_attn_sm100<{KIND}, {D}, {BLOCK_N}, {STAGES}>(
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
    out4[0] = {KIND}; out4[1] = {D}; out4[2] = {BLOCK_N}; out4[3] = {STAGES};
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
}
_RC_TENSOR_MAP = 6


# Kernel kinds (flash_attn/flash_attn_sm100.cuh).
KIND_SIMPLE, KIND_TWO_TILES, KIND_ALTERNATING, KIND_PAIRED, KIND_ONE_TILE, KIND_PERSISTENT = 0, 1, 2, 3, 4, 5


def tuning_space(d: int) -> Tuple[Dict[str, Any], ...]:
    """Candidate kernels for head dim ``d``: kernel kind (which fixes BLOCK_M: one 128-row tile, two tiles per
    CTA, or 256 rows on a CTA pair driven by ``tcgen05.mma.cta_group::2``) x KV tile length x pipeline depth.

    KIND: 0 single-role, 1 warp-specialised with two query tiles per CTA, 2 warp-specialised with one tile per CTA
    and two softmax groups on alternate KV steps, 3 the same on a pair of CTAs (2-CTA MMA; D = 128 only), 4
    warp-specialised with one tile per CTA and two CTAs per SM (a CTA's start and end run beside its neighbour's
    steady state), 5 kind 1 as a persistent grid of one CTA per SM that walks through the work items (the next
    item's first copies and scores sit behind the current item's last steps); 4 and 5 are the kinds for short
    sequences.
    BLOCK_N: KV tile (64 or 128 for kind 0, 128 otherwise).  STAGES: K/V ring slots of kinds 1, 4 and 5, K ring
    slots of kinds 2 and 3 (their V tiles use three slots).
    """
    space = [
        {"KIND": KIND_TWO_TILES, "BLOCK_N": 128, "STAGES": 4},
        {"KIND": KIND_TWO_TILES, "BLOCK_N": 128, "STAGES": 3},
        {"KIND": KIND_PERSISTENT, "BLOCK_N": 128, "STAGES": 3 if d == 128 else 4},
        {"KIND": KIND_ONE_TILE, "BLOCK_N": 128, "STAGES": 2},
        {"KIND": KIND_ALTERNATING, "BLOCK_N": 128, "STAGES": 2 if d == 128 else 4},
        {"KIND": KIND_SIMPLE, "BLOCK_N": 128, "STAGES": 1},
        {"KIND": KIND_SIMPLE, "BLOCK_N": 64, "STAGES": 1},
    ]
    if d == 128:
        space[4:4] = [{"KIND": KIND_PAIRED, "BLOCK_N": 128, "STAGES": 4}, {"KIND": KIND_PAIRED, "BLOCK_N": 128, "STAGES": 6}]
    else:
        space.insert(1, {"KIND": KIND_TWO_TILES, "BLOCK_N": 128, "STAGES": 6})
    forced = _forced_point()
    if forced is not None:
        if forced["KIND"] == KIND_PAIRED and d != 128:
            raise ValueError("FRAY_ATTN_FORCE: the paired kernel (KIND=3) is built for head dim 128 only")
        return (forced,)
    return tuple(space)


def _forced_point() -> Optional[Dict[str, int]]:
    forced = os.getenv("FRAY_ATTN_FORCE")  # e.g. "KIND=0,BLOCK_N=64,STAGES=1"
    if not forced:
        return None
    point = {"BLOCK_N": 128, "STAGES": 4}
    point.update({kv.split("=")[0].strip(): int(kv.split("=")[1]) for kv in forced.split(",")})
    return point


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


def _space_points(head_dims, forced: bool):
    """(d, point, bf16) for every library of the tuning space (forced: honour FRAY_ATTN_FORCE)."""
    old = None if forced else os.environ.pop("FRAY_ATTN_FORCE", None)
    try:
        return [(d, point, bf16) for d in head_dims for bf16 in (False, True) for point in tuning_space(d)]
    finally:
        if old is not None:
            os.environ["FRAY_ATTN_FORCE"] = old


def prebuild(head_dims=SUPPORTED_HEAD_DIMS, prune: bool = False):
    """Compile every point of the tuning space ahead of time (fp16 and bf16 operands) and return the kernel
    directories.

    With ``prune`` the cache directory is also cleared of attention kernels that belong neither to the
    space nor to a point forced through FRAY_ATTN_FORCE (left over from older headers).
    """
    import shutil
    from ..jit import build, cpp_format, generate
    from ..jit.compiler import get_cache_dir

    def build_point(d, point, bf16):
        keys = {"D": d, **point}
        code = generate(includes_bf16 if bf16 else includes, arg_defs_bf16 if bf16 else arg_defs,
                        cpp_format(template, keys), cpp_format(epilogue, keys))
        return build("flash_attn_cute", arg_defs_bf16 if bf16 else arg_defs, code).path

    paths = [build_point(*p) for p in _space_points(head_dims, forced=False)]
    if os.getenv("FRAY_ATTN_FORCE"):
        paths += [build_point(*p) for p in _space_points(head_dims, forced=True)
                  if not (p[1]["KIND"] == KIND_PAIRED and p[0] != 128)]
    if prune:
        for entry in os.listdir(get_cache_dir()):
            full = os.path.join(get_cache_dir(), entry)
            if entry.startswith("kernel.flash_attn_cute.") and full not in paths:
                shutil.rmtree(full, ignore_errors=True)
    return paths


# Every kernel library this process has launched: the device status words are per library.
_used_runtimes: Dict[str, Any] = {}
# Warm-call fast path: (shapes, strides, dtype, device, causal, scale, lse layout) -> (runtime, launch symbol,
# int args, scale).  Everything the slow path validates is a function of that key, so a hit only has to
# marshal the four pointers and the stream.  Bounded: the oldest entries go first.
_fast_path: "OrderedDict[Any, Any]" = OrderedDict()
_FAST_PATH_ENTRIES = 64


def flash_attn_status(clear: bool = True) -> Tuple[int, int, int, int]:
    """Synchronise and return the device status words: ``(0, 0, 0, 0)`` means healthy.

    Every kernel library keeps its own status; this reads all libraries the process has launched,
    returns the first raised one and (with ``clear``) resets them all.  A non-zero first word is the
    code of the first wait that ran out inside a kernel; the other words are the block indices and an
    iteration number.  The status is sticky: until cleared, later launches of that library return
    immediately WITHOUT computing (``launch`` still reports 0), so a caller that cannot rule out a
    preempted or faulty device should check it before trusting an output.
    """
    first = (0, 0, 0, 0)
    for runtime in list(_used_runtimes.values()):
        fn = runtime.symbol("fray_attn_status")
        assert fn is not None, "kernel library does not export fray_attn_status"
        out = (ctypes.c_int * 4)()
        err = fn(out, ctypes.c_int(1 if clear else 0))
        if err != 0:
            raise RuntimeError(f"reading the attention status failed with CUDA error {err}")
        if out[0] != 0 and first[0] == 0:
            first = tuple(out)
    return first


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

    The launch goes to the current stream of the tensors' device, which must be the current device (as in
    the reference, which takes ``torch.cuda.current_stream()``, fray/jit_kernels/flashattn_cute.py:27).
    A raised device status (see ``flash_attn_status``) turns later launches into no-ops until it is cleared.
    """
    fast_key = (Q.shape, Q.stride(), K.shape, K.stride(), V.shape, V.stride(), Output.shape, Output.stride(),
                Q.dtype, K.dtype, V.dtype, Output.dtype, Q.device, K.device, V.device, Output.device, causal, scale,
                None if lse is None else (lse.shape, lse.stride(), lse.dtype, lse.device))
    hit = _fast_path.get(fast_key)
    if hit is not None:
        runtime, launch, ints, sm_scale, dev_index = hit
        if dev_index == torch.cuda.current_device():
            rc = ctypes.c_int(0)
            launch(Q.data_ptr(), K.data_ptr(), V.data_ptr(), Output.data_ptr(), *ints,
                   0 if lse is None else lse.data_ptr(), bool(causal), sm_scale,
                   torch._C._cuda_getCurrentRawStream(dev_index), ctypes.byref(rc))
            if rc.value == 0:
                return
        # e.g. a misaligned data pointer this time, or another current device: let the checked path deal with it
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
    assert Q.device.index == torch.cuda.current_device(), \
        "the tensors must live on the current CUDA device (wrap the call in torch.cuda.device(...))"
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.device == Q.device and lse.is_contiguous()
        assert lse.shape == (batch_size, num_heads, seq_len), "lse must be [B, H, S]"
    if d not in SUPPORTED_HEAD_DIMS:
        raise ValueError(f"head dim {d} not supported (supported: {SUPPORTED_HEAD_DIMS})")
    if batch_size == 0 or num_heads == 0 or seq_len == 0:
        return
    assert seq_len_kv > 0, "attention over zero keys is undefined"
    assert batch_size * num_heads <= 65535, "batch * heads is a grid dimension: at most 65535"

    q, k, v = (t if _usable_strides(t) else t.contiguous() for t in (Q, K, V))
    out = Output if _usable_strides(Output) else torch.empty_like(Output, memory_format=torch.contiguous_format)

    stream = torch.cuda.current_stream(Q.device)
    sm_scale = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    assert sm_scale > 0 and math.isfinite(sm_scale), "the softmax scale must be positive and finite"

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
    forced = os.getenv("FRAY_ATTN_FORCE", "")
    runtime = jit_tuner.compile_and_tune(
        name="flash_attn_cute",
        keys={"D": d, "CAUSAL": int(bool(causal)), "CLASS": _seq_class(max(seq_len, seq_len_kv), batch_size * num_heads),
              "FORCED": forced, **({"BF16": 1} if bf16 else {})},
        space=tuning_space(d),
        includes=includes_bf16 if bf16 else includes,
        arg_defs=arg_defs_bf16 if bf16 else arg_defs,
        template=template,
        args=args,
        epilogue=epilogue,
    )
    _used_runtimes[runtime.path] = runtime

    rc = runtime(*args)
    if rc == _RC_TENSOR_MAP and not all(t.is_contiguous() for t in (q, k, v, out)):
        # The layout cannot be described to the copy engine: fall back to packed copies.
        q, k, v = (t.contiguous() for t in (q, k, v))
        if not out.is_contiguous():
            out = torch.empty_like(Output, memory_format=torch.contiguous_format)
        rc = runtime(*pack(q, k, v, out))
    if rc != 0:
        raise RuntimeError(f"flash_attn_cute launch failed with code {rc} ({_RC_TEXT.get(rc, 'unknown')})")
    if q is Q and k is K and v is V and out is Output and not forced:
        # no copies were needed: remember how to launch this layout directly
        _fast_path[fast_key] = (runtime, runtime.raw_launch(), args[4:4 + 3 + 12 + 2], sm_scale, Q.device.index)
        while len(_fast_path) > _FAST_PATH_ENTRIES:
            _fast_path.popitem(last=False)
    if out is not Output:
        Output.copy_(out)


_host_staging: Dict[Any, Any] = {}


def flash_attn_cute_host(Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, Output: torch.Tensor, *,
                         causal: bool = False, scale: Optional[float] = None, lse: Optional[torch.Tensor] = None,
                         chunks: Optional[int] = None) -> None:
    """``flash_attn_cute`` for operands in pinned HOST memory: result written to the pinned ``Output``.

    No counterpart in the reference (its op asserts CUDA tensors, fray/jit_kernels/flashattn_cute.py:17-20);
    this is the call a host-side caller of the C ABI makes.  Same operands as the device op: fp16 or bf16,
    ``K``/``V`` with ``H_kv | H`` heads and their own length, optional pinned fp32 ``lse`` ``[B, H, S]``.  The
    B * H_kv independent (batch, K/V head) units (each with its group of query heads) are cut into ``chunks``
    slices (default 8) that move through two sets of device staging buffers on three streams of the current
    device: while slice c is computed, slice c+1 is copied in and slice c-1 is copied out, so the two
    directions of the host link run at the same time and the kernel hides behind them.  Work is ordered
    after the current stream's earlier work, and the current stream waits for the last copy-out: as with the
    device op, the result is valid for work queued on the current stream afterwards (or after a
    synchronize), not at return.
    """
    tensors = (Q, K, V, Output) + ((lse,) if lse is not None else ())
    assert all(t.device.type == "cpu" and t.is_pinned() for t in tensors), "operands must be pinned host tensors"
    assert Q.dim() == 4 and K.dim() == 4 and Q.shape == Output.shape and K.shape == V.shape
    assert Q.dtype == K.dtype == V.dtype == Output.dtype and Q.dtype in (torch.half, torch.bfloat16)
    assert all(t.is_contiguous() for t in tensors), "host operands must be contiguous"
    B, H, Sq, D = Q.shape
    Hkv, Sk = K.shape[1], K.shape[2]
    assert K.shape == (B, Hkv, Sk, D) and Hkv > 0 and H % Hkv == 0
    if lse is not None:
        assert lse.dtype == torch.float32 and lse.shape == (B, H, Sq)
    group = H // Hkv
    dev = torch.device("cuda", torch.cuda.current_device())
    units = B * Hkv                                    # one unit = one K/V head with its `group` query heads
    Qu, Ou = (t.view(units, group, Sq, D) for t in (Q, Output))
    Ku, Vu = (t.view(units, 1, Sk, D) for t in (K, V))
    Lu = lse.view(units, group, Sq) if lse is not None else None
    n = max(1, min(units, chunks if chunks else 8))
    bounds = [(units * c) // n for c in range(n + 1)]
    rows = max(b1 - b0 for b0, b1 in zip(bounds, bounds[1:]))
    key = (dev, rows, group, Sq, Sk, D, Q.dtype, lse is not None)
    st = _host_staging.get(key)
    if st is None:
        def make_set():
            bufs = [torch.empty((rows, group, Sq, D), dtype=Q.dtype, device=dev),
                    torch.empty((rows, 1, Sk, D), dtype=Q.dtype, device=dev),
                    torch.empty((rows, 1, Sk, D), dtype=Q.dtype, device=dev),
                    torch.empty((rows, group, Sq, D), dtype=Q.dtype, device=dev)]
            if lse is not None:
                bufs.append(torch.empty((rows, group, Sq), dtype=torch.float32, device=dev))
            return bufs
        st = {"bufs": [make_set(), make_set()], "s_in": torch.cuda.Stream(device=dev), "s_out": torch.cuda.Stream(device=dev)}
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
        bufs = [t[: b1 - b0] for t in st["bufs"][c & 1]]
        dq, dk, dv, do = bufs[:4]
        if computed[c & 1] is not None:
            s_in.wait_event(computed[c & 1])      # inputs of slice c-2 are no longer read
        with torch.cuda.stream(s_in):
            dq.copy_(Qu[b0:b1], non_blocking=True)
            dk.copy_(Ku[b0:b1], non_blocking=True)
            dv.copy_(Vu[b0:b1], non_blocking=True)
            arrived = torch.cuda.Event()
            arrived.record(s_in)
        cur.wait_event(arrived)
        if drained[c & 1] is not None:
            cur.wait_event(drained[c & 1])        # output buffers of slice c-2 have been copied out
        # a slice is itself an attention problem with batch = units in the slice, H = group, H_kv = 1
        flash_attn_cute(dq, dk, dv, do, causal=causal, scale=scale, lse=bufs[4] if lse is not None else None)
        computed[c & 1] = torch.cuda.Event()
        computed[c & 1].record(cur)
        s_out.wait_event(computed[c & 1])
        with torch.cuda.stream(s_out):
            Ou[b0:b1].copy_(do, non_blocking=True)
            if lse is not None:
                Lu[b0:b1].copy_(bufs[4], non_blocking=True)
            drained[c & 1] = torch.cuda.Event()
            drained[c & 1].record(s_out)
    for ev in drained:
        if ev is not None:
            cur.wait_event(ev)
