"""CUDA-graph replay of a forward pass with fixed shapes.

One encoder forward is a few hundred kernel launches of 40-140 us each; launching them from
Python one by one leaves the GPU idle between kernels for about a tenth of the step.  Capturing
the forward once and replaying the graph removes those gaps.  Everything the forward touches
(activations, the mixers' cached filter tables, TMA descriptors, which are kernel parameters)
lives at fixed addresses inside the graph's private memory pool, so a replay runs exactly the
kernels of the captured call on whatever the static input buffers hold at that moment.
"""
from __future__ import annotations

import torch

from . import ops


class GraphedForward:
    """graphed = GraphedForward(model, example_inputs...); out = graphed(inputs...).

    `model(*inputs)` is run under torch.no_grad() (and torch.autocast(bfloat16) unless
    autocast=False) a few times eagerly -- this fills the modules' filter caches -- and then
    captured.  Calling the object copies the new inputs into the static buffers, replays the
    graph on the current stream and returns the static outputs: they are overwritten by the
    next call, so copy what must survive it.  Inputs must keep the example's shapes and dtypes.
    """

    def __init__(self, model, *example_inputs, autocast=True, warmup=3):
        if not all(isinstance(t, torch.Tensor) and t.is_cuda for t in example_inputs):
            raise RuntimeError("GraphedForward needs CUDA tensors as example inputs")
        self.model = model
        self.autocast = bool(autocast)
        self.static_in = [t.clone() for t in example_inputs]
        cur = torch.cuda.current_stream()
        side = torch.cuda.Stream()
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(max(int(warmup), 1)):
                self._run()
        cur.wait_stream(side)
        torch.cuda.synchronize()
        before = ops.LAUNCHES
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_out = self._run()
        self.launches_per_replay = ops.LAUNCHES - before     # kernels of this library inside the graph

    def _run(self):
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16, enabled=self.autocast):
            return self.model(*self.static_in)

    def __call__(self, *inputs):
        if len(inputs) != len(self.static_in):
            raise RuntimeError(f"expected {len(self.static_in)} inputs, got {len(inputs)}")
        for dst, src in zip(self.static_in, inputs):
            if src.shape != dst.shape or src.dtype != dst.dtype:
                raise RuntimeError(f"input of shape {tuple(src.shape)} / {src.dtype} does not match the captured "
                                   f"{tuple(dst.shape)} / {dst.dtype}")
            if src.data_ptr() != dst.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        ops.LAUNCHES += self.launches_per_replay
        return self.static_out
