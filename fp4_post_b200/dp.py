"""Data parallelism around the Metis layer: the token batch is sharded across ranks, weights are
replicated, and nothing crosses GPUs inside the layer (per-tensor units and column means are per
rank, as they are in the reference under DDP).  The one exchange of a training step is the
all-reduce of the weight gradients over NCCL (gloo on CPU): large gradients in place, the small
ones in one flat bucket per dtype; either after backward (`allreduce_gradients`) or started inside
the fused backward, beside the input-gradient GEMM (`GradientReducer`).
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


class GradientReducer:
    """All-reduce of weight gradients started from INSIDE the backward pass, as soon as each gradient
    is final, so that the collective of the large residual gradient runs beside the input-gradient
    GEMM instead of after it (what DDP's bucket hooks do across layers, here inside one layer).

        reducer = GradientReducer(); reducer.attach()      # once, after init_process_group
        loss.backward()                                    # gradients arrive summed over the group

    `ready(t)` starts an asynchronous in-place all-reduce of a large tensor and just remembers a small
    one (with `overlap_sms` > 0 the fused backward caps its input-gradient GEMM at that many SMs fewer
    than the device has, so that the collective really runs beside it); `flush()` reduces the small ones in one flat bucket and makes the current stream wait for
    everything.  The fused Metis backward calls both; `flush()` runs before backward returns, so
    autograd never sees a gradient that is still being reduced."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, average: bool = False, small_bytes: int = 8 << 20,
                 overlap_sms: int = 0, across_layers: bool = False):
        self.group, self.average, self.small_bytes = group, average, small_bytes
        self.overlap_sms = overlap_sms        # SMs the GEMMs leave to a collective that runs beside them
        # across_layers: the fused backward stores the weight gradients in .grad itself (autograd gets None for
        # them, so nothing copies a tensor whose all-reduce is still in flight) and the wait moves to the end
        # of the whole backward pass: the collective of layer k then runs beside the backward of layer k-1
        self.across_layers = across_layers
        self._work, self._small, self._buckets, self.bytes_reduced = [], [], [], 0
        self._deferred = False

    def pending(self) -> bool:
        """A collective started by this reducer may still be running."""
        return bool(self._work or self._buckets)

    def adopt(self, param: torch.nn.Parameter, grad: Optional[torch.Tensor]) -> None:
        """across_layers mode: `grad` becomes (or is added to) param.grad and its all-reduce starts (large) or is
        remembered for the bucket (small).  The caller returns None to autograd for this parameter."""
        if grad is None:
            return
        grad = grad.to(param.dtype) if grad.dtype != param.dtype else grad
        if param.grad is None:
            param.grad = grad
            self.ready(grad)
        else:                                  # gradient accumulation: reduce the new part, then add
            self.ready(grad)
            self._accumulate = getattr(self, "_accumulate", [])
            self._accumulate.append((param, grad))

    def finish_at_end_of_backward(self) -> None:
        """Ask the autograd engine to call flush() when the backward pass that is running has finished."""
        if self._deferred or not self.active():
            return
        self._deferred = True

        def done():
            self._deferred = False
            self.flush()
            for param, grad in getattr(self, "_accumulate", []):
                param.grad.add_(grad)
            self._accumulate = []
        torch.autograd.Variable._execution_engine.queue_callback(done)

    def gemm_sm_limit(self, device) -> int:
        """SM budget of a GEMM that overlaps an all-reduce (0: no cap).  The persistent GEMM
        kernels otherwise hold every SM and the collective's kernel would wait for them to finish."""
        if self.overlap_sms <= 0 or not self.active():
            return 0
        total = torch.cuda.get_device_properties(device).multi_processor_count
        return max(2, (total - self.overlap_sms) & ~1)

    def active(self) -> bool:
        return dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1

    def ready(self, t: torch.Tensor) -> None:
        if t is None or not self.active():
            return
        if t.numel() * t.element_size() < self.small_bytes or not t.is_contiguous():
            self._small.append(t)
            return
        self._work.append((dist.all_reduce(t, group=self.group, async_op=True), t))

    def start_small(self) -> None:
        """Start the all-reduce of the small gradients remembered so far (one flat bucket per dtype)
        without waiting for it: called before a long kernel, the collective runs beside it."""
        if not self.active() or not self._small:
            return
        by_dtype = {}
        for t in self._small:
            by_dtype.setdefault(t.dtype, []).append(t)
        for tensors in by_dtype.values():
            flat = _flatten_dense_tensors(tensors)
            self._buckets.append((dist.all_reduce(flat, group=self.group, async_op=True), flat, tensors))
        self._small = []

    def flush(self) -> None:
        if not self.active():
            return
        world = dist.get_world_size(self.group)
        self.start_small()
        for work, flat, tensors in self._buckets:
            work.wait()                       # the current stream waits for the collective
            if self.average:
                flat.div_(world)
            for t, synced in zip(tensors, _unflatten_dense_tensors(flat, tensors)):
                t.copy_(synced)
            self.bytes_reduced += flat.numel() * flat.element_size()
        for work, t in self._work:
            work.wait()
            if self.average:
                t.div_(world)
            self.bytes_reduced += t.numel() * t.element_size()
        self._work, self._small, self._buckets = [], [], []

    def attach(self) -> "GradientReducer":
        from fp4_post_b200.Metis.Metis import bitlinear
        bitlinear.GRADIENT_REDUCER = self
        return self

    @staticmethod
    def detach() -> None:
        from fp4_post_b200.Metis.Metis import bitlinear
        bitlinear.GRADIENT_REDUCER = None


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group: Optional[dist.ProcessGroup] = None,
                        average: bool = False, small_bytes: int = 8 << 20) -> int:
    """Sum (or average) the .grad of every parameter over the group: gradients of at least
    `small_bytes` (8 MiB: every collective costs tens of microseconds of latency at 8 ranks) are reduced in place, one collective each, the small ones share one flat bucket per
    dtype.  Returns the number of bytes reduced.  A no-op without an initialised process group."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    red = GradientReducer(group, average, small_bytes)
    if not red.active():
        # a group of one still counts the bytes, as the collective would
        return sum(p.grad.numel() * p.grad.element_size() for p in params if p.grad is not None)
    for p in params:
        red.ready(p.grad)
    red.flush()
    return red.bytes_reduced
