"""Two CPU ranks (gloo) shard the (b,h) units, compute their slices and all-gather the result.

The compute on each rank is the CPU oracle standing in for the kernel; what is tested is
the sharding, the per-unit seeding (identical data for any world size) and the gather.
"""
import os
import socket

import torch
import torch.multiprocessing as mp

from fray_b200.multi_gpu import gather_units, shard_units
from oracle import attention_ref as ref

CFG = 0  # config 1: 4 units of [256, 64]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_units, result_path):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    lo, hi = shard_units(n_units, rank, world)
    q, k, v = ref.make_inputs(CFG, range(lo, hi))
    local = ref.flash_fp16p(q, k, v, causal=True)
    full = gather_units(local, n_units)
    if rank == 0:
        torch.save(full, result_path)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reassemble_the_single_rank_answer(tmp_path):
    n_units = ref.CONFIGS[CFG]["B"] * ref.CONFIGS[CFG]["H"] - 1  # 3 units: uneven split 2 + 1
    result = str(tmp_path / "full.pt")
    mp.spawn(_worker, args=(2, _free_port(), n_units, result), nprocs=2, join=True)
    full = torch.load(result)
    q, k, v = ref.make_inputs(CFG, range(n_units))
    want = ref.flash_fp16p(q, k, v, causal=True)
    assert full.shape == want.shape
    assert torch.equal(full, want)
