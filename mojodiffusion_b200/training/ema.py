"""Exponential moving average of the trainable tensors with the power-decay schedule
decay(step) = clamp(1 - (1 + (step - start) / inv_gamma)^(-power), min, max), 0 (skip) while step <= start.
The update itself is the multi-tensor CUDA kernel on a GPU (one launch for all tensors)
(serenitymojo/training/ema_schedule.mojo:30-52, serenitymojo/training/lora_ema.mojo, schedule.mojo ema_update)."""
from __future__ import annotations

from typing import Dict, Iterable, List

import torch

from ..ops import native


def ema_decay_at_step(step: int, update_after_step: int = 0, inv_gamma: float = 1.0, power: float = 2.0 / 3.0,
                      min_decay: float = 0.0, max_decay: float = 0.9999) -> float:
    if step <= update_after_step:
        return 0.0
    eff = float(step - update_after_step)
    v = 1.0 - (1.0 + eff / max(inv_gamma, 1e-8)) ** (-power)
    return min(max(v, min_decay), max_decay)


class EMA:
    """fp32 shadows of ``params``. ``update(step)`` applies shadow = d * shadow + (1 - d) * live."""

    def __init__(self, params: Iterable[torch.nn.Parameter], decay: float = 0.9999, use_schedule: bool = False,
                 update_after_step: int = 0, inv_gamma: float = 1.0, power: float = 2.0 / 3.0, min_decay: float = 0.0):
        self.params = list(params)
        self.shadow = [p.detach().float().clone() for p in self.params]
        self.decay, self.use_schedule = decay, use_schedule
        self.sched = dict(update_after_step=update_after_step, inv_gamma=inv_gamma, power=power, min_decay=min_decay,
                          max_decay=decay)
        self._table = None

    def decay_at(self, step: int) -> float:
        return ema_decay_at_step(step, **self.sched) if self.use_schedule else self.decay

    @torch.no_grad()
    def update(self, step: int) -> float:
        d = self.decay_at(step)
        if self.use_schedule and d == 0.0:
            return d
        if self.params and self.params[0].is_cuda and native.use_native(self.params[0]):
            from .optim import build_tensor_table
            if self._table is None:
                self._table = build_tensor_table(self.shadow, self.params)
            from .optim import CHUNK
            native.ops().ema_multi(self._table[0], self._table[1], CHUNK, self.params[0].dtype == torch.bfloat16, d)
        else:
            for s, p in zip(self.shadow, self.params):
                s.mul_(d).add_(p.detach().float(), alpha=1.0 - d)
        return d

    def state_dict(self, names: List[str]) -> Dict[str, torch.Tensor]:
        return {n: s.clone() for n, s in zip(names, self.shadow)}

    def load_state_dict(self, sd: Dict[str, torch.Tensor], names: List[str]) -> None:
        for n, s in zip(names, self.shadow):
            s.copy_(sd[n].to(s.device, torch.float32))

    @torch.no_grad()
    def swap_in(self):
        """Context manager: parameters temporarily take the shadow values (sampling with EMA weights)."""
        ema = self

        class _Swap:
            def __enter__(self_):
                self_.saved = [p.detach().clone() for p in ema.params]
                for p, s in zip(ema.params, ema.shadow):
                    p.data.copy_(s.to(p.dtype))

            def __exit__(self_, *a):
                for p, s in zip(ema.params, self_.saved):
                    p.data.copy_(s)

        return _Swap()
