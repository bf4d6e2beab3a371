"""Batch sharding of the matmul / conv2d path across the GPUs of one node.

dfdx itself is single-device (its only multi-device affordance is the ordinal of
`Cuda::try_build`, dfdx-core/src/tensor/cuda/device.rs:72-74).  The path shards along the batch
dimension with no data-path exchange in the forward pass; in the backward pass only the gradient of
the operand shared by all shards (the broadcast rhs of `MatMatBrKernel`, the conv2d filters) needs a
sum over ranks.  One process per GPU; `torch.distributed` carries the collective (NCCL on GPUs,
gloo in CPU tests).
"""
from __future__ import annotations

from typing import Iterable, Tuple

import torch
import torch.distributed as dist


def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, end) of rank's contiguous share of n batch items; the first n % world ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(t: torch.Tensor, world: int, rank: int, dim: int = 0) -> torch.Tensor:
    """Zero-copy view of this rank's batch items."""
    s, e = shard_range(t.shape[dim], world, rank)
    return t.narrow(dim, s, e - s)


def allreduce_shared_grads(grads: Iterable[torch.Tensor], group=None) -> None:
    """Sums, over ranks, the gradients of operands that every shard shares (in place).  Gradients of
    batch-sharded operands stay local.  A no-op without an initialised process group."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return
    for g in grads:
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)


def gather_batch(local: torch.Tensor, group=None) -> torch.Tensor:
    """Optional final gather of a batch-sharded output (equal shard sizes)."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local
    parts = [torch.empty_like(local) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=0)
