"""DDPM-family (epsilon-prediction) Euler sampler of SDXL / SD1.5 and the matching training noise schedule.

Scaled-linear betas 0.00085 -> 0.012 over 1000 steps, "leading" timestep spacing with offset 1,
sigma = sqrt((1 - abar) / abar), initial noise x sqrt(sigma_0^2 + 1), model input x / sqrt(sigma^2 + 1),
x += eps * (sigma' - sigma), textbook CFG (serenitymojo/sampling/sdxl_euler.mojo:13-134, sd15_euler.mojo).
Training: noisy = sqrt(abar_t) x0 + sqrt(1 - abar_t) eps, target eps (TRAINING_PLAN_sdxl.md:297-315).
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from .. import ops


def scaled_linear_betas(n: int = 1000, beta_start: float = 0.00085, beta_end: float = 0.012) -> torch.Tensor:
    return torch.linspace(beta_start ** 0.5, beta_end ** 0.5, n, dtype=torch.float64) ** 2


def alphas_cumprod(n: int = 1000, beta_start: float = 0.00085, beta_end: float = 0.012) -> torch.Tensor:
    return torch.cumprod(1.0 - scaled_linear_betas(n, beta_start, beta_end), 0)


class SDXLEulerScheduler:
    def __init__(self, num_steps: int, num_train: int = 1000, beta_start: float = 0.00085, beta_end: float = 0.012,
                 steps_offset: int = 1):
        ac = alphas_cumprod(num_train, beta_start, beta_end)
        ratio = num_train // num_steps
        ts = [(i * ratio) + steps_offset for i in range(num_steps)][::-1]          # leading spacing, descending
        self.timesteps: List[int] = [min(t, num_train - 1) for t in ts]
        sig = [math.sqrt((1.0 - float(ac[t])) / float(ac[t])) for t in self.timesteps]
        self.sigmas: List[float] = sig + [0.0]

    @property
    def init_noise_sigma(self) -> float:
        return math.sqrt(self.sigmas[0] ** 2 + 1.0)

    def scale_model_input(self, x: torch.Tensor, i: int) -> torch.Tensor:
        return x / math.sqrt(self.sigmas[i] ** 2 + 1.0)

    def step(self, x: torch.Tensor, eps: torch.Tensor, i: int) -> torch.Tensor:
        return x + eps.to(x.dtype) * (self.sigmas[i + 1] - self.sigmas[i])


@torch.no_grad()
def euler_eps_sample(model_fn: Callable[[torch.Tensor, int], torch.Tensor], noise: torch.Tensor,
                     sched: SDXLEulerScheduler, uncond_fn: Optional[Callable] = None, cfg_scale: float = 1.0,
                     callback=None) -> torch.Tensor:
    """model_fn(x_scaled, timestep) -> eps. Latent state fp32; CFG: eps_u + s (eps_c - eps_u)."""
    x = noise.float() * sched.init_noise_sigma
    for i, t in enumerate(sched.timesteps):
        xin = sched.scale_model_input(x, i)
        ec = model_fn(xin, t).float()
        if uncond_fn is not None and cfg_scale != 1.0:
            eu = uncond_fn(xin, t).float()
            ec = eu + cfg_scale * (ec - eu)
        x = sched.step(x, ec, i)
        if callback is not None:
            callback(i, x)
    return x


def ddpm_add_noise(x0: torch.Tensor, eps: torch.Tensor, t: torch.Tensor, ac: Optional[torch.Tensor] = None):
    """noisy = sqrt(abar_t) x0 + sqrt(1 - abar_t) eps; returns (noisy, target=eps)."""
    ac = alphas_cumprod() if ac is None else ac
    a = ac.to(x0.device)[t.long()].float().reshape(-1, *([1] * (x0.dim() - 1)))
    return a.sqrt() * x0.float() + (1.0 - a).sqrt() * eps.float(), eps.float()
