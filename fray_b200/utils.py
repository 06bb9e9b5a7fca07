"""Timing and comparison helpers with the reference's protocol (fray/utils.py:5-61)."""
import torch


def bench_kineto(fn, kernel_names, num_tests: int = 100, flush_l2: bool = False, num_warmups: int = 20,
                 verbose: bool = True):
    """Mean device time of ``fn`` in seconds.

    Five 4096^2 fp32 GEMMs and ``num_warmups`` calls warm the device; then ``num_tests``
    calls are timed one by one with CUDA events on the current stream (optionally after a
    256 MB L2 flush), the fastest 10 % are discarded and the rest averaged.  Returns one
    float, or a tuple of that float repeated when ``kernel_names`` is a tuple.
    """
    warm = torch.randn((4096, 4096), device="cuda")
    for _ in range(5):
        warm @ warm
    for _ in range(num_warmups):
        fn()
    torch.cuda.synchronize()

    flusher = torch.empty(int(256e6 // 4), dtype=torch.int, device="cuda") if flush_l2 else None
    times_ms = []
    for _ in range(num_tests):
        if flusher is not None:
            flusher.zero_()
            torch.cuda.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        times_ms.append(start.elapsed_time(end))

    kept = sorted(times_ms)[int(num_tests * 0.1):]
    mean_s = sum(kept) / len(kept) / 1e3
    if verbose:
        print(f"[Bench] {kernel_names}: {mean_s * 1e6:.2f} us (mean of {len(kept)})")
    return tuple([mean_s] * len(kernel_names)) if isinstance(kernel_names, tuple) else mean_s


def calc_diff(x: torch.Tensor, y: torch.Tensor):
    """1 - 2<x,y> / (|x|^2 + |y|^2), accumulated in fp64."""
    x, y = x.double(), y.double()
    return 1 - 2 * (x * y).sum() / (x * x + y * y).sum()


def count_bytes(tensors):
    total = 0
    for t in tensors:
        total += count_bytes(t) if isinstance(t, (tuple, list)) else t.numel() * t.element_size()
    return total
