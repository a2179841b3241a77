"""Serving-loop helper: one sampling step as a CUDA graph.

The reference's sampler calls the model once per step from Python and creates a
few small tensors around every call (``diffusion/rectified_flow.py:85,
107-109``).  At serving batch sizes of a few images a step of the DiT-MoE model
is dozens of short kernels per layer and the GPU waits for the host between
them.  On ONE GPU every kernel of the MoE block is launched without a host
synchronisation and with shapes that do not depend on the routing (the tile
lists are built on the device), so a whole step can be captured once and
replayed:

    step = GraphedStep(lambda z, t: model_step(z, t), example_z, example_t)
    for i in range(n_steps):
        z = step(z, t_i)            # copies the inputs into the captured buffers, replays

What cannot be captured: the expert-parallel exchange (every call carries a
sequence number that grows from step to step, which a graph would freeze) —
``GraphedStep`` refuses blocks in expert-parallel mode — and anything that
synchronises with the host inside the step.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedStep:
    """Capture ``fn(*inputs)`` (tensors in, a tensor or a tuple of tensors out)
    into a CUDA graph after ``warmup`` eager calls, then replay it on every
    call with the caller's inputs copied into the captured buffers.  The
    returned tensors are the graph's output buffers: they are overwritten by
    the next call."""

    def __init__(self, fn: Callable, *example_inputs: torch.Tensor, warmup: int = 3, modules: Sequence = ()):
        for m in modules:
            for sub in m.modules():
                mode = getattr(sub, "para_mode", None)
                if mode is not None and getattr(mode, "ep", False):
                    raise RuntimeError("an expert-parallel block cannot be captured: its exchange kernels take a "
                                       "sequence number per call")
        if not all(t.is_cuda for t in example_inputs):
            raise RuntimeError("GraphedStep captures CUDA work only")
        self._fn = fn
        self._static_in = [t.clone() for t in example_inputs]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(max(1, warmup)):  # first-call set-up (function attributes, packed weights) stays outside
                fn(*self._static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self._graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self._graph):
            self._static_out = fn(*self._static_in)

    def __call__(self, *inputs: torch.Tensor):
        for dst, src in zip(self._static_in, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self._graph.replay()
        return self._static_out
