"""Per-family flow-matching schedules and step rules that are not variations of the FLUX / SD3 tables: Ideogram-4
(logit-normal), Cosmos-Predict2.5 (rectified flow on the UniPC grid), ACE-Step (audio), Lens (empirical exponential
shift), Krea-2 (resolution-aware exponential shift, cond-anchored guidance) and HiDream-O1 (fixed 28-step "flash" table
with re-noising, or an N-step shifted table). Scalar math in float64 on the host; the step rules take tensors.

Behaviour: serenitymojo/sampling/ideogram4_schedule.mojo:8-83, cosmos_rf.mojo:14-148, acestep_flow_match.mojo:30-73,
lens_flowmatch.mojo:8-171, krea2_sampler.mojo:8-161, hidream_o1_scheduler.mojo:8-185.
"""
from __future__ import annotations

import math
from statistics import NormalDist
from typing import List, Optional

import torch

from .flow_match import shifted_sigmas

_NORMAL = NormalDist()


# ---- Ideogram-4 ---------------------------------------------------------------------------------------------------------
def ideogram4_logitnormal(t: float, mean: float, std: float = 1.0, logsnr_min: float = -15.0, logsnr_max: float = 18.0) -> float:
    """Noise level for the uniform step position t in [0, 1]: 1 - sigmoid(mean + std * Phi^-1(t)), clamped to the levels
    whose log-SNR lies in [logsnr_min, logsnr_max]."""
    if t <= 0.0:
        z = -1.0e30
    elif t >= 1.0:
        z = 1.0e30
    else:
        z = _NORMAL.inv_cdf(t)
    y = mean + std * z
    level = 1.0 - (1.0 / (1.0 + math.exp(-y)) if y > -700 else 0.0)
    lo, hi = 1.0 / (1.0 + math.exp(0.5 * logsnr_max)), 1.0 / (1.0 + math.exp(0.5 * logsnr_min))
    return min(max(level, lo), hi)


def ideogram4_schedule_mean(height: int, width: int, known_mean: float = 1.0, known_h: int = 512, known_w: int = 512) -> float:
    return known_mean + 0.5 * math.log((height * width) / (known_h * known_w))


def ideogram4_levels(num_steps: int, height: int, width: int, std: float = 1.0) -> List[float]:
    """num_steps + 1 noise levels for the uniform intervals i / num_steps at a resolution (ascending in t: the sampler
    walks them from the noisy end)."""
    mean = ideogram4_schedule_mean(height, width)
    return [ideogram4_logitnormal(i / num_steps, mean, std) for i in range(num_steps + 1)]


# ---- Cosmos-Predict2.5 ---------------------------------------------------------------------------------------------------
def cosmos_rf_sigmas(num_steps: int = 35, shift: float = 5.0, num_train_timesteps: int = 1000) -> List[float]:
    """linspace((N - 1) / N, 0, steps + 1) without its last point, flow-shifted, then a final 0: the first value is
    0.9998 at shift 5, not 1."""
    if num_steps <= 0:
        raise ValueError("cosmos_rf_sigmas: num_steps must be positive")
    smax = (num_train_timesteps - 1) / num_train_timesteps
    raw = [smax * (1.0 - i / num_steps) for i in range(num_steps)]
    return [shift * s / (1.0 + (shift - 1.0) * s) for s in raw] + [0.0]


def cosmos_timesteps(sigmas: List[float], num_train_timesteps: int = 1000) -> List[float]:
    return [s * num_train_timesteps for s in sigmas[:-1]]


# ---- ACE-Step ------------------------------------------------------------------------------------------------------------
def acestep_sigmas(num_steps: int = 8, shift: float = 3.0) -> List[float]:
    """linspace(1, 0, steps + 1) with the static shift; the turbo model takes 8 steps without guidance."""
    return shifted_sigmas(num_steps, shift)


def acestep_euler_step(x: torch.Tensor, v: torch.Tensor, t_curr: float, t_prev: float) -> torch.Tensor:
    return x - v * (t_curr - t_prev)


# ---- Lens ----------------------------------------------------------------------------------------------------------------
def lens_image_seq_len(width: int, height: int) -> int:
    if width <= 0 or height <= 0 or width % 16 or height % 16:
        raise ValueError("lens_image_seq_len: positive multiples of 16")
    return (height // 16) * (width // 16)


def lens_empirical_mu(image_seq_len: int, num_steps: int) -> float:
    a1, b1, a2, b2 = 8.73809524e-05, 1.89833333, 0.00016927, 0.45666666
    if image_seq_len > 4300:
        return a2 * image_seq_len + b2
    m200, m10 = a2 * image_seq_len + b2, a1 * image_seq_len + b1
    a = (m200 - m10) / 190.0
    return a * num_steps + (m200 - 200.0 * a)


def lens_sigmas(num_steps: int, image_seq_len: int) -> List[float]:
    """num_steps values: linspace(1, 1 / N, N) through the exponential shift with the empirical mu (the last step's
    target, 0, is not part of the list)."""
    mu = lens_empirical_mu(image_seq_len, num_steps)
    raw = [1.0] if num_steps == 1 else [1.0 + (1.0 / num_steps - 1.0) * i / (num_steps - 1) for i in range(num_steps)]
    e = math.exp(mu)
    return [e * s / (e * s + (1.0 - s)) for s in raw]


# ---- Krea-2 --------------------------------------------------------------------------------------------------------------
def krea2_packed_seq_len(height: int, width: int) -> int:
    if height <= 0 or width <= 0 or height % 16 or width % 16:
        raise ValueError("krea2_packed_seq_len: positive multiples of 16")
    return (height // 16) * (width // 16)


def krea2_mu(seq_len: float, y1: float = 0.5, y2: float = 1.15, min_res: int = 256, max_res: int = 1280) -> float:
    x1, x2 = (min_res // 16) ** 2, (max_res // 16) ** 2
    slope = (y2 - y1) / (x2 - x1)
    return slope * seq_len + (y1 - slope * x1)


def krea2_timesteps(seq_len: int, steps: int, mu: Optional[float] = None, sigma: float = 1.0) -> List[float]:
    """steps + 1 times from 1 to 0: exp(mu) / (exp(mu) + (1 / t - 1) ** sigma) over linspace(1, 0); ``mu`` pins the shift
    (the distilled checkpoint was trained at 1.15)."""
    if steps <= 0:
        raise ValueError("krea2_timesteps: steps must be positive")
    e = math.exp(krea2_mu(seq_len) if mu is None else mu)
    out = []
    for i in range(steps + 1):
        t = 1.0 - i / steps
        out.append(1.0 if t >= 1.0 else 0.0 if t <= 0.0 else e / (e + (1.0 / t - 1.0) ** sigma))
    return out


def krea2_cfg(v_cond: torch.Tensor, v_uncond: torch.Tensor, scale: float) -> torch.Tensor:
    """Cond-anchored: v_cond + scale (v_cond - v_uncond)."""
    return v_cond + scale * (v_cond - v_uncond)


# ---- HiDream-O1 ----------------------------------------------------------------------------------------------------------
HIDREAM_DEV_TIMESTEPS = (999, 987, 974, 960, 945, 929, 913, 895, 877, 857, 836, 814, 790, 764, 737, 707, 675, 640, 602, 560,
                         515, 464, 409, 347, 278, 199, 110, 8)


class HiDreamO1Scheduler:
    """``dev()``: the fixed 28-step table; every step re-noises the denoised estimate (stochastic).
    ``full(n, shift)``: n shifted steps from t = 1000 to t = 1, plain Euler."""

    def __init__(self, timesteps: List[float], sigmas: List[float], shift: float, flash: bool):
        self.timesteps, self.sigmas, self.shift, self.flash = timesteps, sigmas, shift, flash

    @staticmethod
    def dev() -> "HiDreamO1Scheduler":
        ts = [float(t) for t in HIDREAM_DEV_TIMESTEPS]
        return HiDreamO1Scheduler(ts, [t / 1000.0 for t in ts] + [0.0], 1.0, True)

    @staticmethod
    def full(n: int, shift: float) -> "HiDreamO1Scheduler":
        t0 = [1000.0] if n == 1 else [1000.0 + (1.0 - 1000.0) * i / (n - 1) for i in range(n)]
        sig = [shift * (t / 1000.0) / (1.0 + (shift - 1.0) * (t / 1000.0)) for t in t0]
        return HiDreamO1Scheduler([s * 1000.0 for s in sig], sig + [0.0], shift, False)

    def step(self, model_output: torch.Tensor, i: int, sample: torch.Tensor, noise: Optional[torch.Tensor] = None,
             s_noise: float = 1.0, noise_clip_std: float = 0.0) -> torch.Tensor:
        sigma, nxt = self.sigmas[i], self.sigmas[i + 1]
        mo = model_output.to(sample.dtype)
        if not self.flash:
            return sample + (nxt - sigma) * mo
        denoised = sample - sigma * mo
        n = noise.to(sample.dtype)
        if noise_clip_std > 0.0:
            clip = noise_clip_std * float(n.float().std(unbiased=False))
            n = n.clamp(-clip, clip)
        return nxt * s_noise * n + (1.0 - nxt) * denoised


# ---- PiD / PixelDiT distilled super-resolution decoder ---------------------------------------------------------------------
PID_STUDENT_TIMES = (0.999, 0.866, 0.634, 0.342, 0.0)      # the released 4-step student schedule
PID_TIMESCALE = 1000.0


def pid_distill_sample(model_fn, x: torch.Tensor, noise_fn, times=PID_STUDENT_TIMES) -> torch.Tensor:
    """Few-step stochastic sampling of a distilled velocity model in pixel space: at every step the clean estimate
    ``x - t v`` is re-noised to the next time with fresh noise, ``(1 - t') x0 + t' eps``; the result is clamped to [-1, 1].
    ``model_fn(x, t * 1000)`` returns the velocity, ``noise_fn()`` a standard normal tensor of x's shape
    (serenitymojo/sampling/pid_distill.mojo:1-199)."""
    for t, t_next in zip(times[:-1], times[1:]):
        x0 = x - t * model_fn(x, t * PID_TIMESCALE).to(x.dtype)
        x = (1.0 - t_next) * x0 + t_next * noise_fn().to(x.dtype) if t_next > 0.0 else x0
    return x.clamp(-1.0, 1.0)


# ---- Lance T2V ---------------------------------------------------------------------------------------------------------------
def lance_times(num_steps: int, shift: float) -> List[float]:
    if num_steps <= 0 or shift <= 0:
        raise ValueError("lance_times: num_steps and shift must be positive")
    return shifted_sigmas(num_steps, shift)


def lance_cfg_renorm(v_cond: torch.Tensor, v_uncond: torch.Tensor, scale: float, renorm_min: float = 0.0,
                     renorm_max: float = 1.0) -> torch.Tensor:
    """Textbook guidance followed by a global renormalisation: the guided velocity is scaled by
    clamp(||v_cond|| / (||v_cfg|| + 1e-8), renorm_min, renorm_max), norms over the whole tensor, no host read-back
    (serenitymojo/sampling/lance_t2v.mojo:41-352)."""
    v = v_uncond + scale * (v_cond - v_uncond)
    ratio = (v_cond.float().square().sum().sqrt() / (v.float().square().sum().sqrt() + 1e-8)).clamp(renorm_min, renorm_max)
    return (v.float() * ratio).to(v.dtype)


def lance_denoise_step(x: torch.Tensor, v: torch.Tensor, t_curr: float, t_next: float) -> torch.Tensor:
    return x - (t_curr - t_next) * v
