"""Data-parallel sharding of the matmul path over the GPUs of one box: one process
per GPU, rows of the left operand (or whole batches) split across ranks, the
right operand replicated; no collective on the compute path.  The reference has no
multi-GPU code at all (`Device::CUDA(n)` only names a device).  An all-gather of
the row-sharded output over NCCL is offered separately."""
from __future__ import annotations

from typing import Tuple

import torch


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [lo, hi) of `total` units owned by `rank`: the first `total % world`
    ranks get one extra unit, so ragged totals and world > total both work."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_rows(x: torch.Tensor, rank: int, world: int, dim: int = 0) -> torch.Tensor:
    lo, hi = shard_range(x.shape[dim], rank, world)
    return x.narrow(dim, lo, hi - lo)


def all_gather_rows(local: torch.Tensor, total_rows: int, group=None) -> torch.Tensor:
    """Gathers row shards made by `shard_rows(dim=0)` into the full matrix on every rank."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = [shard_range(total_rows, r, world) for r in range(world)]
    rows = [hi - lo for lo, hi in sizes]
    if len(set(rows)) == 1:
        full = local.new_empty((total_rows, *local.shape[1:]))
        dist.all_gather_into_tensor(full, local.contiguous(), group=group)
        return full
    # ragged shards: pad every shard to the largest, gather, drop the padding
    most = max(rows)
    padded = local.new_zeros((most, *local.shape[1:]))
    padded[: local.shape[0]] = local
    gathered = local.new_empty((world * most, *local.shape[1:]))
    dist.all_gather_into_tensor(gathered, padded, group=group)
    return torch.cat([gathered[r * most: r * most + rows[r]] for r in range(world)], dim=0)
