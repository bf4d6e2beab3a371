"""Partitioning of the matmul / conv2d path across the GPUs of one node, and its one exchange step.

dfdx itself is single-device (its only multi-device affordance is the ordinal of
`Cuda::try_build`, dfdx-core/src/tensor/cuda/device.rs:72-74), so the partition is this library's own:

* batched problems (`MatMatBrKernel`, `MatMatBatch3/4Kernel`, conv2d) are cut along the batch
  (`shard_batch`), a single large matmul (`MatMatKernel`) along the rows of its left operand
  (`shard_rows`).  Forward passes and the gradient of the partitioned operand need no exchange;
* the gradient of the operand every shard shares (the broadcast rhs of `MatMatBrKernel`, the rhs of a
  row-partitioned `MatMatKernel`, the conv2d filters) is a sum over ranks: one all-reduce per step.
  `OverlappedReducer` runs it on a side stream under the GEMM that follows, `allreduce_shared_grads`
  runs it in line, and `FlatBucket` lets many small gradients travel as one collective.

One process per GPU; `torch.distributed` carries the collective (NCCL over NVLink on GPUs, gloo in CPU
tests).  Weak scaling keeps the per-GPU problem fixed; `strong_shard` cuts one fixed problem.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def _active(group=None) -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1


def shard_range(n: int, world: int, rank: int) -> Tuple[int, int]:
    """[start, end) of rank's contiguous share of n items; the first n % world ranks get one more."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_batch(t: torch.Tensor, world: int, rank: int, dim: int = 0) -> torch.Tensor:
    """Zero-copy view of this rank's batch items."""
    s, e = shard_range(t.shape[dim], world, rank)
    return t.narrow(dim, s, e - s)


def shard_rows(t: torch.Tensor, world: int, rank: int, align: int = 128) -> torch.Tensor:
    """Zero-copy view of this rank's rows (dim -2) of a matrix, for the M-partition of one large matmul.
    Cuts fall on multiples of `align` rows (the MMA tile height) wherever the extent allows, so that no
    rank computes a ragged tile that another rank's cut created."""
    m = t.shape[-2]
    blocks = (m + align - 1) // align
    s, e = shard_range(blocks, world, rank)
    lo, hi = min(s * align, m), min(e * align, m)
    return t.narrow(-2, lo, hi - lo)


def strong_shard(tensors: Sequence[torch.Tensor], world: int, rank: int, dim: int = 0) -> List[torch.Tensor]:
    """This rank's share of every tensor of one fixed problem (strong scaling), cut along `dim`."""
    return [shard_batch(t, world, rank, dim) for t in tensors]


def allreduce_shared_grads(grads: Iterable[torch.Tensor], group=None) -> None:
    """Sums, over ranks, the gradients of operands that every shard shares (in place).  Gradients of
    partitioned operands stay local.  A no-op without an initialised process group."""
    if not _active(group):
        return
    for g in grads:
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)


class FlatBucket:
    """Many small gradients as one collective: views into one flat buffer (a collective's cost at these sizes
    is its launch latency, not its bytes).  `views` alias the bucket, so kernels write gradients in place."""

    def __init__(self, shapes: Sequence[Sequence[int]], dtype: torch.dtype, device) -> None:
        sizes = [int(torch.Size(s).numel()) for s in shapes]
        self.flat = torch.zeros(sum(sizes), dtype=dtype, device=device)
        self.views, off = [], 0
        for s, n in zip(shapes, sizes):
            self.views.append(self.flat[off:off + n].view(*s))
            off += n

    def allreduce(self, group=None) -> None:
        allreduce_shared_grads([self.flat], group)


class OverlappedReducer:
    """The all-reduce of a shared operand's gradient, hidden under the GEMM that follows it.

    `start(grads)` is called right after the GEMM that produced `grads` was enqueued on the current stream: the
    collective is enqueued on a side stream behind an event, so it runs while the current stream goes on with the
    next GEMM; `finish()` makes the current stream wait for it.  The GEMM kernels of this library are persistent and
    fill every SM, so the caller leaves a few SMs to the collective for the overlapped stretch
    (`b200_set_max_ctas`) and bounds the collective's own CTAs (`nccl_group`).  On CPU tensors (gloo) `start` reduces
    in line and `finish` does nothing."""

    def __init__(self, device: Optional[torch.device] = None, group=None) -> None:
        self.group = group
        self.stream = torch.cuda.Stream(device) if device is not None and device.type == "cuda" else None
        self.device = device

    def start(self, grads: Iterable[torch.Tensor]) -> None:
        grads = list(grads)
        if not _active(self.group):
            return
        if self.stream is None:
            allreduce_shared_grads(grads, self.group)
            return
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream):
            for g in grads:
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group)

    def finish(self) -> None:
        if self.stream is not None and _active(self.group):
            torch.cuda.current_stream(self.device).wait_stream(self.stream)


def nccl_group(max_ctas: int):
    """A second NCCL communicator over all ranks whose kernels use at most `max_ctas` CTAs, for collectives that run
    beside a GEMM.  Returns None (use the default group) when the backend does not offer the option."""
    if not _active():
        return None
    try:
        opts = dist.ProcessGroupNCCL.Options()
        opts.config.max_ctas = int(max_ctas)
        opts.config.min_ctas = 1
        return dist.new_group(ranks=list(range(dist.get_world_size())), backend="nccl", pg_options=opts)
    except Exception:  # noqa: BLE001 - an older backend: the default communicator serves
        return None


def gather_batch(local: torch.Tensor, group=None) -> torch.Tensor:
    """Optional final gather of a batch-partitioned output (equal shard sizes)."""
    if not _active(group):
        return local
    parts = [torch.empty_like(local) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat(parts, dim=0)
