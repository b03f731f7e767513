"""Data parallelism around the Metis layer: the token batch is sharded across ranks, weights are
replicated, and nothing crosses GPUs inside the layer (per-tensor units and column means are per
rank, as they are in the reference under DDP).  The one exchange of a training step is the
all-reduce of the weight gradients, done here in one flat bucket per dtype over NCCL (gloo on CPU).
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch
import torch.distributed as dist
from torch._utils import _flatten_dense_tensors, _unflatten_dense_tensors


def shard_tokens(batch: torch.Tensor, rank: int, world: int, dim: int = 0) -> torch.Tensor:
    """The contiguous slice of `batch` along `dim` that belongs to `rank` (sizes differ by at most one)."""
    n = batch.shape[dim]
    lo, hi = (n * rank) // world, (n * (rank + 1)) // world
    return batch.narrow(dim, lo, hi - lo)


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group: Optional[dist.ProcessGroup] = None,
                        average: bool = False) -> int:
    """Sum (or average) the .grad of every parameter over the group, one collective per dtype.
    Returns the number of bytes reduced.  A no-op without an initialised process group."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    world = dist.get_world_size(group)
    by_dtype = {}
    for p in params:
        if p.grad is not None:
            by_dtype.setdefault(p.grad.dtype, []).append(p.grad)
    total = 0
    for grads in by_dtype.values():
        flat = _flatten_dense_tensors(grads)
        dist.all_reduce(flat, group=group)
        if average:
            flat.div_(world)
        for g, synced in zip(grads, _unflatten_dense_tensors(flat, grads)):
            g.copy_(synced)
        total += flat.numel() * flat.element_size()
    return total
