"""LTX-2 samplers: distilled sigma tables, Euler with denoise-return final step, and res_2s (second-order exponential
Runge-Kutta with phi-functions, optional SDE noise injection).

Behaviour: serenitymojo/sampling/ltx2_sampling.mojo:56-697 (schedules :123-198; res_2s coefficients and combination
:430-560; SDE coefficients :560-697), pipeline use serenitymojo/pipeline/ltx2_t2v_av_hq.mojo:17-24.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import torch

from .flow_match import ltx2_linear_quadratic_sigmas, ltx2_token_shift_sigmas

# distilled tables (stage 1: 8 steps, stage 2 refinement: 3 steps)
DISTILLED_STAGE1 = [1.0, 0.99375, 0.9875, 0.98125, 0.975, 0.909375, 0.725, 0.421875, 0.0]
DISTILLED_STAGE2 = [0.909375, 0.725, 0.421875, 0.0]


def phi(k: int, z: float) -> float:
    """phi_1(z) = (e^z - 1)/z, phi_2(z) = (e^z - 1 - z)/z^2 (series near 0)."""
    if abs(z) < 1e-6:
        return 1.0 / math.factorial(k) + z / math.factorial(k + 1)
    if k == 1:
        return math.expm1(z) / z
    if k == 2:
        return (math.expm1(z) - z) / (z * z)
    raise ValueError(k)


def res2s_coefficients(sigma: float, sigma_next: float, c2: float = 0.5):
    """h = log(sigma/sigma_next); a21 = c2 phi_1(-h c2); b2 = phi_2(-h)/c2; b1 = phi_1(-h) - b2; sub_sigma = sqrt(s s')."""
    if sigma_next <= 0.0:
        raise ValueError("res_2s needs sigma_next > 0 (the last step is a denoise return)")
    h = math.log(sigma / sigma_next)
    a21 = c2 * phi(1, -h * c2)
    b2 = phi(2, -h) / c2
    b1 = phi(1, -h) - b2
    return h, a21, b1, b2, math.sqrt(sigma * sigma_next)


def sde_coefficients(sigma_next: float, eta: float = 0.5):
    """sigma_up = min(eta sigma', 0.9999 sigma'); residual = sqrt(sigma'^2 - sigma_up^2); alpha_ratio = (1 - sigma') +
    residual; sigma_down = residual / alpha_ratio."""
    up = min(sigma_next * eta, sigma_next * 0.9999)
    resid = math.sqrt(max(sigma_next * sigma_next - up * up, 0.0))
    alpha_ratio = (1.0 - sigma_next) + resid
    return alpha_ratio, resid / alpha_ratio, up


@torch.no_grad()
def euler_ltx2_sample(v_fn: Callable[[torch.Tensor, float], torch.Tensor], x: torch.Tensor, sigmas: Sequence[float]):
    """Interior steps x += v (s' - s); the final step returns the denoised sample x - v s."""
    x = x.float()
    n = len(sigmas) - 1
    for i in range(n):
        s, sn = float(sigmas[i]), float(sigmas[i + 1])
        v = v_fn(x, s).float()
        x = x - v * s if (i == n - 1 or sn <= 0.0) else x + v * (sn - s)
    return x


@torch.no_grad()
def res2s_sample(v_fn: Callable[[torch.Tensor, float], torch.Tensor], x: torch.Tensor, sigmas: Sequence[float],
                 eta: float = 0.0, generator: Optional[torch.Generator] = None):
    """Two model evaluations per step; denoised = x - v sigma. With eta > 0 the step ends with the SDE noise mix
    x <- alpha_ratio (x_det rescaled to sigma_down) + sigma_up * noise."""
    x = x.float()
    n = len(sigmas) - 1
    for i in range(n):
        s, sn = float(sigmas[i]), float(sigmas[i + 1])
        d1 = x - v_fn(x, s).float() * s
        if sn <= 0.0:
            return d1
        target = sn
        if eta > 0.0:
            alpha_ratio, s_down, s_up = sde_coefficients(sn, eta)
            target = s_down
        h, a21, b1, b2, sub = res2s_coefficients(s, target)
        x_mid = x + (h * a21) * (d1 - x)
        d2 = x_mid - v_fn(x_mid, sub).float() * sub
        x_next = x + h * (b1 * (d1 - x) + b2 * (d2 - x))
        if eta > 0.0:
            noise = torch.randn(x.shape, generator=generator, device="cpu").to(x.device) if generator is not None \
                else torch.randn_like(x)
            x_next = alpha_ratio * x_next + s_up * noise
        x = x_next
    return x
