"""Running a stack of blocks whose weights stream through the block-swap loader.

``StreamedStack`` rebinds the parameters of block i to views of the slot that holds block i, runs it, and hands the
slot back. For training with frozen streamed weights (LoRA on a base too large to keep resident) each block is a
recompute boundary: the forward keeps only the block's inputs, the backward walks the blocks in reverse, streams the
weights again (prefetching i-1 while i computes), re-runs the block under autograd and backpropagates, so neither
weights nor inner activations are held between the two passes
(serenitymojo/models/flux/flux_stack_lora.mojo:1619-2019 offload variants; training/checkpoint_block.mojo:245-485)."""
from __future__ import annotations

from typing import Callable, Dict, Sequence

import torch
from torch import nn

from .loader import BlockSwapLoader


def _bind(block: nn.Module, prefix: str, views: Dict[str, torch.Tensor]) -> None:
    for name, p in list(block.named_parameters()) + list(block.named_buffers()):
        key = prefix + name
        if key in views:
            p.data = views[key]


class StreamedStack:
    """``blocks[i]`` corresponds to plan block i. Parameters named ``<plan prefix><param name>`` are streamed; any
    other parameter of the block (adapters) stays where it is and trains normally."""

    def __init__(self, blocks: Sequence[nn.Module], loader: BlockSwapLoader):
        assert len(blocks) == len(loader.plan)
        self.blocks, self.loader = list(blocks), loader
        self.prefixes = [b.prefix for b in loader.plan.blocks]

    def detach_weights(self) -> None:
        """Drops the blocks' own copies of streamed weights (they live in the pinned store now)."""
        names = [set(m.name for m in mem) for mem in self.loader.store.members]
        for i, blk in enumerate(self.blocks):
            for n, p in blk.named_parameters():
                if self.prefixes[i] + n in names[i]:
                    p.requires_grad_(False)
                    p.data = torch.empty(0, dtype=p.dtype, device=self.loader.device)

    def run_block(self, i: int, fn: Callable, *args, reverse: bool = False):
        views = self.loader.await_block(i)
        self.loader.prefetch_next(i, reverse)
        _bind(self.blocks[i], self.prefixes[i], views)
        try:
            return fn(self.blocks[i], *args)
        finally:
            self.loader.mark_done(i)

    def forward(self, call: Callable, *state):
        """Inference: ``state = call(block, *state)`` for every block in order."""
        for i in range(len(self.blocks)):
            out = self.run_block(i, call, *state)
            state = out if isinstance(out, tuple) else (out,)
        return state if len(state) > 1 else state[0]

    def step(self, i: int, call: Callable, *inputs):
        """One block, ``call(block, *inputs)``: plain streamed run without autograd, recompute boundary with it.
        Tensors that need gradients must be passed in ``inputs`` (not captured by ``call``)."""
        if not torch.is_grad_enabled():
            return self.run_block(i, call, *inputs)
        extra = [p for p in self.blocks[i].parameters() if p.requires_grad]
        return _StreamedBlockFn.apply(self, i, call, len(inputs), *inputs, *extra)

    def forward_train(self, call: Callable, *state):
        """Training: every block is a recompute boundary (see module docstring)."""
        for i in range(len(self.blocks)):
            out = self.step(i, call, *state)
            state = out if isinstance(out, tuple) else (out,)
        return state if len(state) > 1 else state[0]


class _StreamedBlockFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, stack: StreamedStack, i: int, call, n_state: int, *args):
        state = args[:n_state]
        ctx.stack, ctx.i, ctx.call, ctx.n_state = stack, i, call, n_state
        ctx.save_for_backward(*[s.detach() for s in state])
        ctx.needs = [s.requires_grad for s in state]
        with torch.no_grad():
            out = stack.run_block(i, call, *state)
        return out

    @staticmethod
    def backward(ctx, *grads):
        stack, i = ctx.stack, ctx.i
        state = [s.detach().requires_grad_(need) for s, need in zip(ctx.saved_tensors, ctx.needs)]
        extra = [p for p in stack.blocks[i].parameters() if p.requires_grad]
        with torch.enable_grad():
            out = stack.run_block(i, ctx.call, *state, reverse=True)
            outs = out if isinstance(out, tuple) else (out,)
            pairs = [(o, g) for o, g in zip(outs, grads) if g is not None and o.requires_grad]
            inputs = [s for s in state if s.requires_grad] + extra
            got = torch.autograd.grad([o for o, _ in pairs], inputs, [g for _, g in pairs], allow_unused=True)
        it = iter(got)
        g_state = [next(it) if s.requires_grad else None for s in state]
        g_extra = [next(it) for _ in extra]
        return (None, None, None, None, *g_state, *g_extra)
