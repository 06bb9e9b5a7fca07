"""Role timeline of the two-tile attention kernel: where the cycles of a KV step go.

    python -m fray_b200.jit_kernels.timeline [--batch B] [--warm N] [--row R] [--causal]

Builds the two-tile kernel (KIND 1) with ``-DFRAY_ATTN_TRACE``: one thread per role of CTA (0, 0) stamps the
cycle counter into a table (events x tile x KV step, see ``softmax_tile_sm100.cuh``) and the CTA's entry and
exit are stamped with the nanosecond timer as well, which gives the SM clock the kernel really ran at (NVML's
clock reading lags a region of a few milliseconds).  The stamps cost the kernel about 10 %; what they show is
the order and the proportions of a step, not absolute speed.  Needs a B200.
"""

import argparse
import ctypes
import os
import statistics


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--batch", type=int, default=1, help="batch size of the [B, 32, 4096, 128] problem")
    ap.add_argument("--warm", type=int, default=4, help="launches before the one whose table is read")
    ap.add_argument("--row", type=int, default=64, help="row of the tile whose softmax thread stamps (0..127)")
    ap.add_argument("--causal", action="store_true")
    args = ap.parse_args()

    # the build flags are part of the cache key: this never replaces the production library
    os.environ["FRAY_NVCC_EXTRA_FLAGS"] = f"-DFRAY_ATTN_TRACE -DFRAY_TRACE_ROW={args.row}"
    os.environ["FRAY_ATTN_FORCE"] = "KIND=1,BLOCK_N=128,STAGES=4"
    import torch
    from . import flashattn_cute as op

    B, H, S, D = args.batch, 32, 4096, 128
    q, k, v = (torch.randn(B, H, S, D, device="cuda", dtype=torch.half) for _ in range(3))
    out = torch.zeros_like(q)
    for _ in range(args.warm + 1):
        op.flash_attn_cute(q, k, v, out, causal=args.causal)
    torch.cuda.synchronize()
    read = list(op._used_runtimes.values())[-1].symbol("fray_attn_trace_read")
    events, iters = 12, 40
    buf = (ctypes.c_uint * (events * 2 * iters))()
    words = read(buf, events * 2 * iters)
    print("status", op.flash_attn_status(), "words", words)

    t0 = buf[(8 * 2 + 0) * iters + 0]  # first S = Q.K^T issued

    def stamp(event, tile, j):
        x = (buf[(event * 2 + tile) * iters + j] - t0) & 0xFFFFFFFF
        return x - (1 << 32) if x > (1 << 31) else x

    names = {0: "scores ready", 1: "row in registers", 2: "max and offset", 3: "first chunk computed",
             9: "second chunk computed", 10: "first chunk handed over", 11: "second chunk stored", 4: "step done"}
    order = (0, 1, 2, 3, 9, 10, 11, 4)
    steps = range(8, 30)
    for tile in (0, 1):
        parts = "  ".join(f"-> {names[b]} {statistics.mean(stamp(b, tile, j) - stamp(a, tile, j) for j in steps):.0f}"
                          for a, b in zip(order, order[1:]))
        print(f"tile {tile} softmax step (cycles, mean of KV steps 8..29): {parts}")
        print(f"tile {tile}: softmax {statistics.mean(stamp(4, tile, j) - stamp(0, tile, j) for j in steps):.0f}"
              f"  step done -> P.V issued {statistics.mean(stamp(7, tile, j) - stamp(4, tile, j) for j in steps):.0f}"
              f"  -> next S issued {statistics.mean(stamp(8, tile, j + 1) - stamp(7, tile, j) for j in steps):.0f}"
              f"  -> scores ready {statistics.mean(stamp(0, tile, j + 1) - stamp(8, tile, j + 1) for j in steps):.0f}"
              f"  period {statistics.mean(stamp(0, tile, j + 1) - stamp(0, tile, j) for j in steps):.0f}")
    print(f"tile 1 lags tile 0 by {statistics.mean(stamp(0, 1, j) - stamp(0, 0, j) for j in steps):.0f} cycles")
    print("CTA: entry", stamp(6, 0, 0), " set-up done", stamp(6, 0, 1), " first scores", stamp(0, 0, 0),
          " last scores tile 0 / 1", stamp(0, 0, 31), stamp(0, 1, 31), " epilogues start", stamp(6, 1, 0), stamp(6, 1, 1),
          " exit", stamp(6, 0, 2))
    ns = (buf[(6 * 2 + 0) * iters + 11] - buf[(6 * 2 + 0) * iters + 10]) & 0xFFFFFFFF
    cycles = (buf[(6 * 2 + 0) * iters + 2] - buf[(6 * 2 + 0) * iters + 0]) & 0xFFFFFFFF
    print(f"CTA (0,0) of the last launch: {cycles} cycles in {ns} ns -> SM clock {cycles / ns * 1000:.0f} MHz")


if __name__ == "__main__":
    main()
