"""Sharding of the (batch, kv_head) units over the GPUs of one node.

Every unit is independent end to end (quantize, flush, attention), so rank r
of `world` permanently owns a contiguous run of units and no KV ever crosses
NVLink.  The one exchange per layer-step is an all-gather of the attention
outputs [units, n_rep, D] (the reference is single-device: nothing to cite).
Works on any torch.distributed backend: NCCL on GPUs, gloo in the CPU tests.
"""
from typing import Tuple

import torch

__all__ = ["unit_partition", "all_gather_units"]


def unit_partition(n_units: int, rank: int, world: int) -> Tuple[int, int]:
    """[u0, u1) of rank `rank`: contiguous, sizes differ by at most one, the
    first n_units % world ranks hold the extra unit."""
    assert 0 <= rank < world and n_units >= 0
    base, extra = divmod(n_units, world)
    u0 = rank * base + min(rank, extra)
    return u0, u0 + base + (1 if rank < extra else 0)


def all_gather_units(local: torch.Tensor, n_units: int, rank: int, world: int, group=None) -> torch.Tensor:
    """local [u1-u0, ...] of every rank -> [n_units, ...] on every rank, in unit
    order.  Equal shards use one all_gather_into_tensor; ragged shards pad to
    the largest shard first."""
    import torch.distributed as dist
    if world == 1:
        return local
    sizes = [unit_partition(n_units, r, world) for r in range(world)]
    biggest = max(b - a for a, b in sizes)
    tail = local.shape[1:]
    if all(b - a == biggest for a, b in sizes):
        out = torch.empty((n_units,) + tuple(tail), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest,) + tuple(tail), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    buf = torch.empty((world * biggest,) + tuple(tail), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    return torch.cat([buf[r * biggest: r * biggest + (b - a)] for r, (a, b) in enumerate(sizes)], dim=0)
