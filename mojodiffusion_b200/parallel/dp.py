"""Data-parallel gradient synchronisation for adapter (LoRA) training.

All trainable gradients live in ONE flat buffer (``p.grad`` of every parameter is a view into it), so the
collective is a single large message. Modes:

* ``"allreduce"``: ``torch.distributed.all_reduce`` on the flat buffer (NCCL on GPUs, gloo on CPU ranks), then the
  fused multi-tensor AdamW with ``grad_scale = 1/world``. This is the baseline path.
* ``"fused"``: the gradient all-reduce, the 1/world scale, the clip coefficient and the AdamW update run in one
  kernel over NVLink peer memory (see ``parallel/fused_dp.py``); GPU only.

The reference has no data parallelism; its design note (serenitymojo/docs/AUDIT_SIMPLETUNER_PARITY_2026-06-11.md:86-100)
names the gate used in the tests here: DP-N must reproduce the single-rank batch-N trajectory.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist


class FlatGradBuffer:
    """One contiguous gradient buffer with a view per parameter (same dtype as the parameters)."""

    def __init__(self, params: Sequence[torch.nn.Parameter], buffer: Optional[torch.Tensor] = None):
        self.params = list(params)
        p0 = self.params[0]
        # 16-byte aligned segments so vector loads and multimem accesses stay aligned
        align = 16 // p0.element_size()
        self.offsets: List[int] = []
        n = 0
        for p in self.params:
            self.offsets.append(n)
            n += (p.numel() + align - 1) // align * align
        self.numel = n
        self.flat = buffer if buffer is not None else torch.zeros(n, dtype=p0.dtype, device=p0.device)
        assert self.flat.numel() >= n
        self.attach()

    def attach(self):
        for p, off in zip(self.params, self.offsets):
            p.grad = self.flat[off:off + p.numel()].view_as(p)

    def zero(self):
        self.flat.zero_()


class DataParallelGrads:
    def __init__(self, params: Sequence[torch.nn.Parameter], group=None, mode: str = "allreduce"):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.mode = mode
        self.buf = FlatGradBuffer(params)

    def zero_grad(self):
        self.buf.zero()
        self.buf.attach()

    def sync(self) -> float:
        """Sum gradients over ranks in place; returns the scale (1/world) the optimizer must apply."""
        if self.world > 1:
            dist.all_reduce(self.buf.flat, op=dist.ReduceOp.SUM, group=self.group)
        return 1.0 / self.world


def broadcast_parameters(params: Sequence[torch.Tensor], src: int = 0, group=None) -> None:
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    for p in params:
        dist.broadcast(p.data, src=src, group=group)
