"""One layer call of fixed shapes captured as a CUDA graph.

A layer call is 8 to 14 short launches (quantise, sort, two GEMM stages, finalize; with expert parallelism also
the exchange kernels and two or three NCCL collectives). From Python each launch costs tens of microseconds of
host time, which shows as gaps between the kernels once the per-rank work shrinks (8 ranks: ~1 ms of kernels per
call). The captured graph replays the same launches, with the same arguments and work buffers, from one driver
call. The reference surrounds its layers with a capture context for the same purpose
(aiter/dist/parallel_state.py:623 ``GroupCoordinator.graph_capture``, :1673 ``graph_capture``); this module is that
capture for a caller that has no engine around the layer.

Everything the layer allocates while being captured lives in the graph's private pool and keeps its address
for every replay, the input tensors included: ``CapturedLayer.__call__`` copies new inputs into the captured
ones (device copies on the current stream) unless the caller wrote them there already (``inputs``).
"""

from __future__ import annotations

import torch


class CapturedLayer:
    """``CapturedLayer(fn, *example_inputs)``: ``fn(*tensors) -> tensor`` is run ``warmup`` times eagerly (so every
    lazily built buffer, tensor map and peer mapping exists), then once under stream capture.

    With ``torch.distributed`` collectives inside ``fn`` the construction is a collective call: every rank of
    the group must build its CapturedLayer at the same point, and replays must be issued in the same order on
    all ranks, exactly as the eager calls would be.

    ``inputs`` are the captured input tensors (write into them in place, or pass new tensors to ``__call__``);
    ``output`` is the tensor every replay overwrites."""

    def __init__(self, fn, *example_inputs, warmup: int = 2):
        if not example_inputs or not all(isinstance(t, torch.Tensor) and t.is_cuda for t in example_inputs):
            raise ValueError("CapturedLayer: example_inputs must be CUDA tensors")
        dev = example_inputs[0].device
        self.inputs = tuple(t.clone() for t in example_inputs)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                fn(*self.inputs)
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=side):
            self.output = fn(*self.inputs)
        if not isinstance(self.output, torch.Tensor):
            raise TypeError("CapturedLayer: fn must return one tensor")

    def release(self):
        """Destroys the captured graph and drops its tensors. A graph that holds captured collectives must be
        released before the process group is destroyed (the communicator's teardown otherwise waits for ever on
        the work the graph still references); a collective point like the construction."""
        if self.graph is not None:
            self.graph.reset()
        self.graph, self.output, self.inputs = None, None, ()

    def replay(self):
        """Runs the captured launches on the current stream with whatever ``inputs`` hold now."""
        if self.graph is None:
            raise RuntimeError("CapturedLayer: replay after release()")
        self.graph.replay()
        return self.output

    def __call__(self, *tensors):
        if len(tensors) != len(self.inputs):
            raise ValueError(f"CapturedLayer: expected {len(self.inputs)} tensors, got {len(tensors)}")
        for dst, src in zip(self.inputs, tensors):
            if dst.shape != src.shape or dst.dtype != src.dtype:
                raise ValueError(f"CapturedLayer: captured {tuple(dst.shape)} {dst.dtype}, "
                                 f"got {tuple(src.shape)} {src.dtype}")
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        return self.replay()
