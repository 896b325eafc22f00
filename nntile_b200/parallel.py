"""Sharding of the path over one process per GPU.

Every (batch, kv head) slice of the SDPA tensors is an independent attention
problem (src/tensor/flash_sdpa_fwd_cudnn.cc:221-233: the outer loop runs over
output tiles, only the inner K/V-sequence loop carries a dependency), which is
how the reference spreads tile tasks over StarPU CUDA workers.  Here the units
are dealt out in contiguous blocks, one block per rank, and no collective sits
on the data path; ``regather`` is the optional all-gather for a caller that
wants the whole output on every rank.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_units: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous block [lo, hi) of `n_units` for `rank`; sizes differ by at most 1."""
    if world <= 0 or not (0 <= rank < world) or n_units < 0:
        raise ValueError("bad shard arguments")
    base, extra = divmod(n_units, world)
    lo = rank*base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_units(tensor: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Slice a (kv_heads, group, batch, ...) buffer by (kv head, batch) units.

    Units are numbered kv_head*batch + b; a rank's block must not split a kv
    head unevenly across the batch axis unless it covers whole batches, so the
    split is done on the kv-head axis when it divides and on the batch axis
    otherwise."""
    H, G, B = tensor.shape[:3]
    if H % world == 0:
        lo, hi = shard_range(H, rank, world)
        return tensor[lo:hi]
    if B % world == 0:
        lo, hi = shard_range(B, rank, world)
        return tensor[:, :, lo:hi]
    raise ValueError(f"neither kv_heads={H} nor batch={B} divides over {world} ranks")


def regather(local: torch.Tensor, axis: int = 0, group=None) -> torch.Tensor:
    """All-gather equally sized shards along `axis` (NCCL on GPUs, gloo on CPU)."""
    world = dist.get_world_size(group)
    if world == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(world)]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=axis)


def max_over_ranks(value: float, device, group=None) -> float:
    t = torch.tensor([value], dtype=torch.float64, device=device)
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
