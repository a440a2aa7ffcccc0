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


class GraphedTrainStep:
    """Forward + backward of a training step as one CUDA graph.

    ``loss_fn(*inputs) -> scalar loss`` is warmed up eagerly, then captured together with ``loss.backward()`` while every
    trainable parameter's ``.grad`` is None, so the gradient buffers are created inside the capture and stay at fixed
    addresses: each replay overwrites them. The optimizer (and any gradient collective) runs after the replay on those
    static gradients. Inputs are copied into the captured input tensors before a replay; everything ``loss_fn`` reads
    besides its inputs and the parameters must itself be static. The capture covers the recompute of checkpointed blocks
    (their forward runs again inside the captured backward), which is why the block checkpoints of this package do not
    stash RNG state (serenitymojo/autograd_v2/capture.mojo:34-180: 5,774 forward + 21,036 backward graph nodes per step)."""

    def __init__(self, loss_fn: Callable, params: Sequence[torch.nn.Parameter], example_inputs: Sequence[torch.Tensor],
                 warmup: int = 3, zero_grad: Callable = None):
        """``zero_grad``: for optimizers whose gradients are views of one flat buffer (the fused data-parallel AdamW): it is
        called INSIDE the capture before the forward, so every replay clears the buffer and the backward accumulates into
        the same views. Without it the gradients are created by the captured backward itself."""
        self.zero_grad = zero_grad
        self.loss_fn = loss_fn
        self.params = [p for p in params]
        self.static_in = [t.clone() for t in example_inputs]
        self.warmup = warmup
        self.graph = None
        self.static_loss = None

    def _clear(self):
        for p in self.params:
            p.grad = None

    def capture(self):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(self.warmup):
                self.zero_grad() if self.zero_grad is not None else self._clear()
                self.loss_fn(*self.static_in).backward()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        if self.zero_grad is None:
            self._clear()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            if self.zero_grad is not None:
                self.zero_grad()
            self.static_loss = self.loss_fn(*self.static_in)
            self.static_loss.backward()
        return self

    def __call__(self, *inputs) -> torch.Tensor:
        if self.graph is None:
            self.capture()
        for dst, src in zip(self.static_in, inputs):
            if dst.data_ptr() != src.data_ptr():
                dst.copy_(src, non_blocking=True)
        self.graph.replay()
        return self.static_loss
