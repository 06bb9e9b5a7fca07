"""Benchmark of the attention forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one forward pass of `flash_attn_cute` over the whole per-GPU workload.  The
default workload is the shape the headline metric is quoted on: non-causal B=4, H=32,
S=4096, D=128 (1.0995 TFLOP per step per GPU).  With N > 1 (launched by torchrun, one rank
per GPU) every rank runs that workload on its own (b,h) units - the path shards by
independent units, there is no collective on the data path - so scaling is weak and
`value` is total FLOPs of all ranks over the slowest rank's device time.

Prints ONE JSON line (rank 0).  `--impl reference` instead times the CPU oracle (torch CPU
attention, the comparison the reference's own test uses) on a bounded sample of the same
workload, on rank 0 only.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

NOMINAL_FP16_TFLOPS = 2250.0
# DRAM traffic of the warp-specialised kernel from one ncu capture of the `small` workload
# (32 (b,h) units of S=4096, D=128, non-causal): dram__bytes_read.sum + dram__bytes_write.sum.
# Units are independent, so a launch with more units of the same shape moves proportionally more.
NCU_DRAM_BYTES_PER_UNIT_S4096_D128 = (100.783360e6 + 14.093824e6) / 32
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}

WORKLOADS = {
    # name: (B, H, S, D, causal)
    "headline": (4, 32, 4096, 128, False),
    "c2": (2, 16, 2048, 128, False),
    "c3": (4, 32, 4096, 128, True),
    "c4": (1, 32, 16384, 128, True),
    "c5": (16, 16, 1024, 64, False),
    # one batch of the headline shape: 134 MB of operands (> L2), small enough for profiler captures
    "small": (1, 32, 4096, 128, False),
    "small_causal": (1, 32, 4096, 128, True),
}


def flops_of(B, H, S, D, causal):
    f = 4.0 * B * H * S * S * D
    return f / 2 if causal else f


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            peaks = json.load(f)
        return peaks, "measured"
    except (OSError, ValueError):
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML from a thread while the timed region runs."""

    def __init__(self, gpu_index: int, period_s: float = 0.002):
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples = []       # (sm_mhz, reasons bitmask)
        self.sm_max = None
        self._stop = threading.Event()
        self.thread = None
        self.error = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            index = self.gpu_index
            if visible:
                entry = visible.split(",")[self.gpu_index].strip()
                index = int(entry) if entry.isdigit() else self.gpu_index
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
        except Exception as exc:  # NVML missing: report it, do not fail the benchmark
            self.error = repr(exc)
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nvml
        while not self._stop.is_set():
            try:
                clk = nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)
                why = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                self.samples.append((float(clk), int(why)))
            except Exception as exc:
                self.error = repr(exc)
                return
            time.sleep(self.period_s)

    def stop(self):
        self._stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [f"no samples: {self.error}"], "samples": 0}
        nv = self.nvml
        names = {
            "hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
            "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
            "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
            "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap,
        }
        seen = 0
        for _, why in self.samples:
            seen |= why
        reasons = sorted(n for n, bit in names.items() if seen & bit)
        return {"sm_mhz": statistics.median(c for c, _ in self.samples), "sm_max_mhz": self.sm_max,
                "reasons": reasons, "samples": len(self.samples)}


def cpu_attention_sample(B, H, S, D, causal, budget_s=12.0):
    """Times torch CPU attention (fp32 math on the fp16 inputs) on successive (b,h) units until the
    budget is used; returns (TFLOP/s, units done, seconds, threads)."""
    import torch.nn.functional as F
    from oracle import attention_ref as ref
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, RuntimeError):
        pass
    threads = torch.get_num_threads()
    q, k, v = ref.make_slice(5, 0, S, D)
    q, k, v = (t.float().reshape(1, 1, S, D) for t in (q, k, v))
    F.scaled_dot_product_attention(q, k, v, is_causal=causal)  # warm-up
    done, t0 = 0, time.perf_counter()
    while (time.perf_counter() - t0) < budget_s:
        F.scaled_dot_product_attention(q, k, v, is_causal=causal)
        done += 1
    dt = time.perf_counter() - t0
    return flops_of(1, done, S, D, causal) / dt / 1e12, done, dt, threads


def run_reference(args, B, H, S, D, causal, rank):
    """CPU arm: torch CPU attention on a bounded sample of the workload, rank 0 only."""
    if rank != 0:
        return
    import torch.nn.functional as F
    from oracle import attention_ref as ref
    # torchrun pins OMP_NUM_THREADS=1; the CPU arm is meant to use every core this process may run on
    try:
        torch.set_num_threads(len(os.sched_getaffinity(0)))
    except (AttributeError, RuntimeError):
        pass
    threads = torch.get_num_threads()
    units_per_step = 2
    q, k, v = ref.make_inputs(5, range(units_per_step)) if (B, H, S, D) == (4, 32, 4096, 128) else tuple(
        torch.randn(units_per_step, S, D).half() for _ in range(3))
    q, k, v = (t.float().unsqueeze(0) for t in (q, k, v))
    for _ in range(max(args.warmup, 1)):
        F.scaled_dot_product_attention(q, k, v, is_causal=causal)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        F.scaled_dot_product_attention(q, k, v, is_causal=causal)
    dt = time.perf_counter() - t0
    value = flops_of(1, units_per_step, S, D, causal) * args.steps / dt / 1e12
    sample = f"{units_per_step} of {B * H} (b,h) units per step, torch CPU scaled_dot_product_attention in fp32"
    line = {
        "impl": "reference", "metric": "flash_attn_fwd_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "B": B, "H": H, "S": S, "D": D, "causal": causal,
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="headline", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--kernel-only", action="store_true", help="skip the end-to-end and CPU legs (profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    B, H, S, D, causal = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference(args, B, H, S, D, causal, rank)
        return

    assert torch.cuda.is_available(), "bench.py needs a GPU: the attention path has no CPU fallback"
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from fray_b200.jit_kernels import flash_attn_cute, flash_attn_cute_host, flash_attn_status
    from fray_b200.jit_kernels.tuner import jit_tuner

    # Synthetic inputs with the workload's shape and N(0,1) values, seeded per rank.
    gen = torch.Generator(device="cuda").manual_seed(42 * 1000 + rank)
    q, k, v = (torch.randn(B, H, S, D, generator=gen, device="cuda", dtype=torch.half) for _ in range(3))
    out = torch.zeros_like(q)
    flops = flops_of(B, H, S, D, causal)

    def step():
        flash_attn_cute(q, k, v, out, causal=causal)

    def barrier():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    step()  # JIT lookup + tuning happen here, outside every timed region
    for _ in range(args.warmup):
        step()
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    stream = torch.cuda.current_stream()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        step()
    ev1.record(stream)
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None
    status = flash_attn_status()
    assert status[0] == 0, f"device status {status}"

    # ---- end to end: pinned host inputs -> device, op, result -> pinned host, every step
    if args.kernel_only:
        if rank == 0:
            value = flops * world / (ms_total / args.steps * 1e-3) / 1e12
            print(json.dumps({"metric": "flash_attn_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
                              "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_total / args.steps,
                              "config": {"workload": args.workload}, "kernel_only": True, "clocks": clocks}), flush=True)
        return
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    hout = torch.empty_like(hq).pin_memory()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        # the package's host-buffer call: batch slices staged through the device on three streams,
        # every step copies all inputs in and the whole result out
        flash_attn_cute_host(hq, hk, hv, hout, causal=causal)

    for _ in range(2):
        e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    e1.record(stream)
    barrier()
    e2e_ms_total = e0.elapsed_time(e1)

    times = torch.tensor([ms_total / args.steps, e2e_ms_total / e2e_steps], device="cuda", dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms_step, e2e_ms_step = times.tolist()

    if rank == 0:
        peaks, peak_src = load_peaks()
        value = flops * world / (ms_step * 1e-3) / 1e12
        per_gpu = value / world
        e2e_value = flops * world / (e2e_ms_step * 1e-3) / 1e12
        # burst GEMM figure when the timed region ran unthrottled, sustained one when the power cap was seen
        capped = bool(clocks and "sw_power_cap" in (clocks.get("reasons") or []))
        peak_key = "bf16_tflops_sustained" if capped else "bf16_tflops"
        peak = float(peaks.get(peak_key, FALLBACK_PEAKS[peak_key]))
        traffic = None
        if (S, D, causal) == (4096, 128, False):
            traffic = NCU_DRAM_BYTES_PER_UNIT_S4096_D128 * B * H
        tuned = {str(sig[1]): keys for sig, keys in jit_tuner.tuned_keys.items()}
        line = {
            "metric": "flash_attn_fwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": args.workload, "B_per_gpu": B, "H": H, "S": S, "D": D, "causal": causal,
                       "flops_per_step_per_gpu": flops, "l2": "inputs (537 MB per step) larger than the 126 MB L2"
                       if B * H * S * D * 8 > 126e6 else "inputs smaller than L2, no flush",
                       "kernel": tuned},
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peak, "unit": "TFLOP/s",
                         "frac": per_gpu / peak, "traffic": traffic,
                         "traffic_note": "bytes per launch per GPU, ncu capture of the one-batch case scaled by units",
                         "algorithmic_bytes": 4 * B * H * S * D * 2,
                         "peak_source": f"{peak_src} {'sustained' if capped else 'burst'} bf16 GEMM "
                                        f"({'power cap seen' if capped else 'no throttle reason'} during the timed region)",
                         "frac_of_nominal_2250": per_gpu / NOMINAL_FP16_TFLOPS,
                         "frac_of_sustained_gemm": per_gpu / float(peaks.get("bf16_tflops_sustained",
                                                                         FALLBACK_PEAKS["bf16_tflops_sustained"]))},
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms_step,
                    "h2d_bytes_per_step": 3 * q.numel() * 2 * world, "d2h_bytes_per_step": out.numel() * 2 * world},
            "gpu_launches": args.steps * world,
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            cpu_v, cpu_units, cpu_s, cpu_threads = cpu_attention_sample(B, H, S, D, causal)
            line["cpu_baseline"] = {
                "value": cpu_v, "unit": "TFLOP/s", "cores": cpu_threads, "kind": "port",
                "sample": f"{cpu_units} single-(b,h)-unit passes (the workload has {B * H} units) in {cpu_s:.1f} s, torch CPU "
                          f"scaled_dot_product_attention in fp32, host has {os.cpu_count()} logical cores"}
        print(json.dumps(line), flush=True)

    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
