"""CUDA-graph capture of a whole training (or rollout) step of Metis layers.

One forward + backward of a Metis layer is some 35 kernel launches and as many small torch ops; issued
one by one from Python they cost more host time than the GPU needs to run them.  Everything on the
path is capturable: the kernels take their workspaces from torch's allocator, the Philox offset of
the stochastic quantizer lives on the device (`METIS_Q_OFFSET_ON_DEVICE`), nothing reads a result back
to the host, and the NCCL all-reduce of `fp4_post_b200.dp.GradientReducer` is captured like any kernel.

    step = GraphedStep(lambda: train_step(x_static, g_static))   # runs it a few times, then captures
    x_static.copy_(batch); g_static.copy_(grad)                  # refill the static inputs
    out = step()                                                 # one graph launch

Before capturing, drop (or detach) every tensor that still carries the autograd graph of an earlier
eager step: its gradient accumulators belong to the stream of that step, and the capture is
invalidated when backward has to synchronise with them.

What a captured step freezes: shapes, the Python control flow taken during capture, and every
host-side cache decision.  In particular a layer built with `cache_quantized_weight=True` that hit
its cache during capture will keep using those packed weights: capture with the cache off (the weight
quantization is then part of the graph) whenever the weights change between replays.
"""
from __future__ import annotations

from typing import Any, Callable, Optional

import torch


_CAPTURE_STREAMS = {}


def _capture_stream() -> "torch.cuda.Stream":
    """The stream every capture on the current device runs on (one per device: autograd ties a parameter's gradient
    accumulation to the stream of its first backward, so a second capture on another stream would depend on
    uncaptured work).  High priority in a single-process step: the capturing stream carries the step's critical
    path, and the streams the library keeps for deferred scale passes have the lowest, so where both have CTAs
    waiting the path goes first."""
    dev = torch.cuda.current_device()
    st = _CAPTURE_STREAMS.get(dev)
    if st is None:                # the priority is settled by the first capture of the process
        from fp4_post_b200.Metis.Metis.bitlinear import critical_path_priority
        st = _CAPTURE_STREAMS[dev] = torch.cuda.Stream(priority=critical_path_priority())
    return st


class GraphedStep:
    """`fn` (no arguments; it reads static input tensors and returns tensors or None) captured into one
    CUDA graph.  Calling the object replays the graph and returns what `fn` returned during capture
    (the same tensor objects, refreshed in place)."""

    def __init__(self, fn: Callable[[], Any], warmup: int = 3, pool: Optional[Any] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("GraphedStep needs a CUDA device")
        self.fn = fn
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        # parameters that already took part in a backward on another stream make autograd warn about
        # the stream of their gradient accumulators; here the change of stream is intended
        quiet = getattr(torch.autograd.graph, "set_warn_on_accumulate_grad_stream_mismatch", None)
        if quiet is not None:
            quiet(False)
        try:
            with torch.cuda.stream(side):             # warm-up off the default stream, as capture requires
                for _ in range(max(1, warmup)):
                    fn()
            cur.wait_stream(side)
            torch.cuda.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, pool=pool, stream=_capture_stream()):
                self.outputs = fn()
        finally:
            if quiet is not None:
                quiet(True)

    def __call__(self):
        self.graph.replay()
        return self.outputs

    def pool(self):
        return self.graph.pool()

    def release(self):
        """Destroy the captured graph.  A process that captured NCCL collectives must do this before
        `destroy_process_group()`, which otherwise waits forever for kernels the graphs still own."""
        self.outputs = None
        self.graph.reset()
