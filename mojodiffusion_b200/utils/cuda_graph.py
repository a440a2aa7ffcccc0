"""CUDA-graph capture of a steady-state step.

``GraphedCallable`` warms a function up, captures one call into a ``torch.cuda.CUDAGraph`` and afterwards replays
it: inputs are copied into the captured (static) input tensors, outputs are the captured output tensors. All kernels
of this package are capture-safe: launch arguments (tensor maps included) are by value, scratch comes from the
caching allocator's capture pool, and peer-memory flags take their epochs from device-side counters.

Mirrors the reference's warm-up / capture / replay lifecycle (serenitymojo/autograd_v2/capture.mojo:34-180) whose
precondition is an identical allocation sequence per step (serenitymojo/autograd_v2/step_slab.mojo:40-90); here the
allocator's private pool gives the same guarantee.
"""
from __future__ import annotations

from typing import Callable, Sequence, Tuple

import torch


class GraphedCallable:
    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 2):
        self.fn = fn
        self.static_in = [t.clone() for t in example_inputs]
        self.graph = None
        self.static_out = None
        self.warmup = warmup

    def capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s), torch.no_grad():
            for _ in range(self.warmup):
                self.fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(self.graph):
            self.static_out = self.fn(*self.static_in)
        return self

    def __call__(self, *inputs):
        if self.graph is None:
            self.capture()
        for dst, src in zip(self.static_in, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_out


def graphs_equal_eager(fn: Callable, inputs: Sequence[torch.Tensor]) -> Tuple[bool, float]:
    """Gate of the capture path: captured replay must reproduce the eager result bit for bit."""
    with torch.no_grad():
        eager = fn(*[t.clone() for t in inputs])
    g = GraphedCallable(fn, inputs).capture()
    out = g(*inputs)
    torch.cuda.synchronize()
    flat_e = eager if isinstance(eager, (tuple, list)) else [eager]
    flat_o = out if isinstance(out, (tuple, list)) else [out]
    err = max(float((a.float() - b.float()).abs().max()) for a, b in zip(flat_e, flat_o))
    return all(torch.equal(a, b) for a, b in zip(flat_e, flat_o)), err
