"""Data-parallel plumbing for the routing path.

The path shards by batch with no forward exchange; the only cross-rank quantity is the
gradient of the connection weights (``read_weight`` / ``write_weight``: 2*C*S floats per
connection event, 2 MB for the largest model here).  Under ``DistributedDataParallel`` those
gradients ride in the ordinary buckets (reference: sihc/training/train.py:515-523).  For
callers that drive the operators directly, :func:`allreduce_weight_grads` packs any number of
small gradient tensors into one flat fp32 buffer and issues a single all-reduce, so the exchange
costs one collective launch regardless of the number of events.
"""

from __future__ import annotations

from typing import Sequence

import torch
import torch.distributed as dist
from torch import Tensor


def shard_batch(batch: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous ``[start, stop)`` range of images owned by ``rank`` (remainder to the low ranks)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def allreduce_weight_grads(grads: Sequence[Tensor], group=None, average: bool = True) -> None:
    """Sum (or average) the given gradient tensors over the process group, in place, with ONE collective."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    if not grads:
        return
    world = dist.get_world_size(group)
    if len(grads) == 1 and grads[0].is_contiguous() and grads[0].dtype == torch.float32:
        # already one flat fp32 buffer (the kernels can write both gradients into it): reduce it where it lies
        flat = grads[0].detach()
        dist.all_reduce(flat, group=group)
        if average:
            flat /= world
        return
    flat = torch.cat([g.detach().reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=group)
    if average:
        flat /= dist.get_world_size(group)
    offset = 0
    for g in grads:
        n = g.numel()
        g.detach().copy_(flat[offset:offset + n].view_as(g))
        offset += n
