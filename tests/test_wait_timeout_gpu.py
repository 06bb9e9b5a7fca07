"""The bounded-wait path: a wait that runs out leaves a status word, later launches return at entry,
clearing re-arms.  Uses a test-only kernel (tests/wait_probe.cuh) built through the package's JIT; the
wait that runs out has nothing in flight around it, so the context stays healthy."""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _probe():
    from fray_b200.jit import build, generate
    arg_defs = (("Out", torch.int), ("stream", torch.cuda.Stream))
    body = "fray_test::launch_wait_probe(Out, stream, __return_code);"
    epilogue = ('extern "C" EXPORT_API int fray_attn_status(int* out4, int clear) '
                '{ return fray::read_attn_status(out4, clear != 0); }')
    code = generate((f'"{os.path.join(HERE, "wait_probe.cuh")}"',), arg_defs, body, epilogue)
    return build("wait_probe", arg_defs, code)


def _status(runtime, clear):
    out = (ctypes.c_int * 4)()
    assert runtime.symbol("fray_attn_status")(out, ctypes.c_int(1 if clear else 0)) == 0
    return tuple(out)


def test_a_wait_that_runs_out_raises_the_status_and_clearing_rearms():
    runtime = _probe()
    out = torch.zeros(1, dtype=torch.int, device="cuda")
    stream = torch.cuda.current_stream()
    assert _status(runtime, clear=True)[0] == 0

    assert runtime(out, stream) == 0
    torch.cuda.synchronize()
    assert out.item() == 1                                   # the wait gave up, the kernel returned normally
    status = _status(runtime, clear=False)
    assert status == (0x7E1, 0, 0, 42)                       # site code, block x, block y, extra

    out.zero_()
    assert runtime(out, stream) == 0                         # the launch itself still succeeds ...
    torch.cuda.synchronize()
    assert out.item() == 2                                   # ... but the kernel returned at entry
    assert _status(runtime, clear=True)[0] == 0x7E1          # still raised (sticky); this read clears it
    assert _status(runtime, clear=False)[0] == 0

    out.zero_()
    assert runtime(out, stream) == 0                         # re-armed: the wait runs (and runs out) again
    torch.cuda.synchronize()
    assert out.item() == 1
    assert _status(runtime, clear=True)[0] == 0x7E1
    assert _status(runtime, clear=True)[0] == 0
    # the context is healthy: an ordinary attention call still works
    from fray_b200.jit_kernels import flash_attn_cute, flash_attn_status
    q = torch.randn(1, 2, 256, 64, device="cuda", dtype=torch.half)
    o = torch.zeros_like(q)
    flash_attn_cute(q, q, q, o)
    torch.cuda.synchronize()
    assert flash_attn_status()[0] == 0 and o.abs().sum() > 0
