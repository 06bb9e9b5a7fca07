"""Sharding of the (batch x head) grid over the GPUs of one box.

Each (b, h) slice is an independent attention problem (the reference kernel indexes it
by blockIdx.y alone, fray/include/flash_attn/flashattn_cute.cuh:29), so ranks never
exchange data on the compute path.  The only collective is an optional all-gather that
assembles ``out`` for verification.
"""
from typing import Tuple

import torch


def shard_units(n_units: int, rank: int, world_size: int) -> Tuple[int, int]:
    """Contiguous block [lo, hi) of flat (b*H + h) units owned by ``rank``; sizes differ by at most one."""
    assert 0 <= rank < world_size and n_units >= 0
    base, extra = divmod(n_units, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def gather_units(local_out: torch.Tensor, n_units: int, group=None) -> torch.Tensor:
    """All-gather per-rank ``[n_local, S, D]`` outputs into the full ``[n_units, S, D]`` tensor (verification only)."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = [shard_units(n_units, r, world)[1] - shard_units(n_units, r, world)[0] for r in range(world)]
    assert local_out.shape[0] == sizes[rank]
    biggest = max(sizes)
    padded = local_out.new_zeros((biggest, *local_out.shape[1:]))
    padded[: sizes[rank]] = local_out
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)
