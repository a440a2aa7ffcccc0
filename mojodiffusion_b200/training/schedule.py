"""Training-time schedules: timestep / sigma sampling, LR schedules, EMA decay.

Timestep rules follow serenitymojo/training/schedule.mojo:253-385: logit-normal ``sigma = sigmoid(N(0,1))`` followed
by the shift ``s*t/(1+(s-1)t)`` clamped to [1e-3, 1]; the discrete OneTrainer variant (idx in [0, 999],
sigma = (idx+1)/1000, model timestep idx/1000; :287-350); uniform; sigmoid with scale. LR schedules follow
serenitymojo/training/lr_schedule.mojo:27-169 (constant / linear / cosine / cosine-restarts / polynomial / REX + warmup).
"""
from __future__ import annotations

import math
from typing import Optional

import torch


def sample_sigmas(batch: int, generator: Optional[torch.Generator] = None, kind: str = "logit_normal",
                  shift: float = 1.0, mean: float = 0.0, std: float = 1.0, device="cpu") -> torch.Tensor:
    """Per-sample noise level in (0, 1]."""
    if kind == "logit_normal":
        u = torch.randn(batch, generator=generator) * std + mean
        t = torch.sigmoid(u)
    elif kind == "uniform":
        t = torch.rand(batch, generator=generator)
    elif kind == "sigmoid":
        t = torch.sigmoid(torch.randn(batch, generator=generator) * std)
    else:
        raise ValueError(kind)
    t = shift * t / (1.0 + (shift - 1.0) * t)
    return t.clamp(1e-3, 1.0).to(device)


def sample_discrete_timesteps(batch: int, generator=None, shift: float = 1.0, device="cpu"):
    """OneTrainer-style discrete rule: returns (sigma = (idx+1)/1000, model_t = idx/1000)."""
    t = torch.sigmoid(torch.randn(batch, generator=generator))
    t = shift * t / (1.0 + (shift - 1.0) * t)
    idx = (t * 1000.0).long().clamp(0, 999)
    return ((idx + 1).float() / 1000.0).to(device), (idx.float() / 1000.0).to(device)


def lr_at(step: int, base_lr: float, total_steps: int, kind: str = "constant", warmup: int = 0, min_ratio: float = 0.0,
          cycles: int = 1, power: float = 1.0) -> float:
    if warmup > 0 and step < warmup:
        return base_lr * (step + 1) / warmup
    n = max(1, total_steps - warmup)
    p = min(1.0, max(0.0, (step - warmup) / n))
    if kind == "constant":
        f = 1.0
    elif kind == "linear":
        f = 1.0 - p
    elif kind == "cosine":
        f = 0.5 * (1.0 + math.cos(math.pi * p))
    elif kind == "cosine_with_restarts":
        f = 0.5 * (1.0 + math.cos(math.pi * ((p * cycles) % 1.0))) if p < 1.0 else 0.0
    elif kind == "polynomial":
        f = (1.0 - p) ** power
    elif kind == "rex":
        f = (1.0 - p) / (0.5 + 0.5 * (1.0 - p))
    else:
        raise ValueError(kind)
    return base_lr * (min_ratio + (1.0 - min_ratio) * f)


def ema_decay_at(step: int, max_decay: float = 0.9999, inv_gamma: float = 1.0, power: float = 2.0 / 3.0,
                 update_after: int = 0) -> float:
    s = max(0, step - update_after - 1)
    if s <= 0:
        return 0.0
    return min(max_decay, max(0.0, 1.0 - (1.0 + s / inv_gamma) ** (-power)))
