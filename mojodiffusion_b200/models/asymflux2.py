"""AsymFLUX.2: a pixel-space (Oklab) flow model whose transformer predicts an "asymmetric" velocity.

The backbone is an unchanged FLUX.2 Klein transformer fed 16 x 16 pixel patches (3 * 16 * 16 = 768 channels). Its output
``u_a`` is not the flow velocity: inside the column space of a fixed projection ``P`` [D, R] the velocity is a calibrated
blend of ``u_a`` and the data term, outside it a plain rescale:

    sigma = t / num_timesteps,  k = 1 / (s + (1 - s) sigma),  the transformer sees x_t * k at time t * k
    sub(z) = z P P^T,  comp(z) = z - sub(z)
    u = s k sub(u_a) + (1 - s k) / sigma * sub(x_t)  +  (comp(x_t) + s comp(u_a)) / sigma

Written with one projection: ``u = (x_t + s u_a) / sigma + sub((s k - s / sigma) u_a - (s k / sigma) x_t)``, all in fp32.
The sampler adds guidance with the component parallel to the denoised image removed, and keeps the denoised image
inside the sRGB gamut by clamping it through Oklab -> sRGB -> Oklab.

Behaviour: serenitymojo/models/asymflux2/asymflow.mojo:45-183, serenitymojo/pipeline/asymflux2_klein9b_gen.mojo:317-640.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn as nn

from .mmdit import pack_latents, unpack_latents

PATCH = 16
SIGMA_MIN = 1e-4
OKLAB_MEAN = (0.56, 0.0, 0.01)
OKLAB_STD = 0.16
_LRGB_TO_LMS = ((0.4122214708, 0.5363325363, 0.0514459929),
                (0.2119034982, 0.6806995451, 0.1073969566),
                (0.0883024619, 0.2817188376, 0.6299787005))
_LMS_TO_OKLAB = ((0.2104542553, 0.7936177850, -0.0040720468),
                 (1.9779984951, -2.4285922050, 0.4505937099),
                 (0.0259040371, 0.7827717662, -0.8086757660))


@dataclass
class AsymFlowCalibration:
    s: float            # the adapter's scale buffer
    k: float            # 1 / (s + (1 - s) sigma)
    cal_timestep: float
    sigma: float


def compute_calibration(timestep: float, scale_buffer: float, num_timesteps: float = 1.0) -> AsymFlowCalibration:
    sigma = timestep / num_timesteps
    k = 1.0 / (scale_buffer + (1.0 - scale_buffer) * sigma)
    return AsymFlowCalibration(scale_buffer, k, timestep * k, sigma)


def _clamp_sigma(sigma: float, sigma_min: float) -> float:
    return sigma if (sigma != sigma or sigma >= sigma_min) else sigma_min      # NaN stays NaN


def asymflow_velocity(u_a: torch.Tensor, x_t: torch.Tensor, cal: AsymFlowCalibration, p: torch.Tensor,
                      sigma_min: float = SIGMA_MIN) -> torch.Tensor:
    """Full velocity [B, hw, D] in fp32 from the transformer output ``u_a`` and the packed noisy pixels ``x_t``;
    ``p`` is the [D, R] projection buffer."""
    u_a, x_t, p = u_a.float(), x_t.float(), p.float()
    inv = 1.0 / _clamp_sigma(cal.sigma, sigma_min)
    sk = cal.s * cal.k
    low = (sk - cal.s * inv) * u_a - (sk * inv) * x_t
    return (x_t + cal.s * u_a) * inv + (low @ p) @ p.t()


# ---- Oklab <-> sRGB on [B, 3, H, W] fp32 (normalised Oklab: (value - mean) / std per channel) ---------------------------
def _mat(rows, ref: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    m = torch.tensor(rows, dtype=torch.float64)
    return (torch.linalg.inv(m) if inverse else m).to(ref.device, torch.float32)


def _apply(m: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    return torch.einsum("ij,bjhw->bihw", m, x)


def oklab_decode(z: torch.Tensor) -> torch.Tensor:
    """Normalised Oklab -> sRGB in [-1, 1] (linear RGB clamped to the gamut)."""
    z = z.float()
    mean = torch.tensor(OKLAB_MEAN, device=z.device).view(1, 3, 1, 1)
    lms = _apply(_mat(_LMS_TO_OKLAB, z, True), z * OKLAB_STD + mean) ** 3
    lin = _apply(_mat(_LRGB_TO_LMS, z, True), lms).clamp(0.0, 1.0)
    srgb = torch.where(lin <= 0.0031308, lin * 12.92, 1.055 * lin.clamp_min(1e-12) ** (1.0 / 2.4) - 0.055)
    return srgb * 2.0 - 1.0


def oklab_encode(rgb: torch.Tensor) -> torch.Tensor:
    """sRGB in [-1, 1] -> normalised Oklab."""
    s = rgb.float() * 0.5 + 0.5
    lin = torch.where(s <= 0.04045, s / 12.92, ((s.clamp_min(0.0) + 0.055) / 1.055) ** 2.4)
    lms = _apply(_mat(_LRGB_TO_LMS, s), lin).clamp_min(0.0)
    ok = _apply(_mat(_LMS_TO_OKLAB, s), torch.sign(lms) * lms.abs() ** (1.0 / 3.0))
    mean = torch.tensor(OKLAB_MEAN, device=s.device).view(1, 3, 1, 1)
    return (ok - mean) / OKLAB_STD


def clamp_denoised_oklab(x_t: torch.Tensor, velocity: torch.Tensor, sigma: float, sigma_min: float = SIGMA_MIN) -> torch.Tensor:
    """Velocity whose denoised image ``x_t - sigma * velocity`` has been pulled into the sRGB gamut."""
    den = oklab_encode(oklab_decode(x_t - velocity * sigma).clamp(-1.0, 1.0))
    return (x_t - den) / _clamp_sigma(sigma, sigma_min)


def guidance_bias(pos: torch.Tensor, neg: torch.Tensor, scale: float, ortho: float, parallel_dir: torch.Tensor) -> torch.Tensor:
    """(scale - 1)(pos - neg) with ``ortho`` x its projection on ``parallel_dir`` removed (per sample)."""
    bias = (pos - neg) * (scale - 1.0)
    if ortho == 0.0:
        return bias
    dims = tuple(range(1, bias.dim()))
    coef = (bias * parallel_dir).mean(dims, keepdim=True) / (parallel_dir * parallel_dir).mean(dims, keepdim=True).clamp_min(1e-6)
    return bias - parallel_dir * (coef * ortho)


def dynamic_shift(height: int, width: int) -> float:
    """Resolution-dependent time shift: 17 at 1024 x 1024, 34 at 2048 x 2048, linear in sqrt(pixels)."""
    lo, hi = math.sqrt(1024.0 * 1024.0), math.sqrt(2048.0 * 2048.0)
    return (math.sqrt(height * width) - lo) * (34.0 - 17.0) / (hi - lo) + 17.0


def sigma_schedule(steps: int, shift: float) -> List[float]:
    out = []
    for i in range(steps):
        raw = 1.0 - i / steps
        out.append(shift * raw / (1.0 + (shift - 1.0) * raw))
    return out + [0.0]


class AsymFlux2(nn.Module):
    """A FLUX.2 transformer with ``in_channels = 3 * 16 * 16`` plus the adapter's ``proj_buffer`` [768, R] and scalar
    ``scale_buffer``; ``forward`` returns the full pixel-space velocity."""

    def __init__(self, transformer: nn.Module, proj_buffer: torch.Tensor, scale_buffer: float, num_timesteps: float = 1.0):
        super().__init__()
        self.transformer = transformer
        self.register_buffer("proj_buffer", proj_buffer.float())
        self.scale_buffer = float(scale_buffer)
        self.num_timesteps = float(num_timesteps)

    @torch.no_grad()
    def forward(self, x_t: torch.Tensor, txt: torch.Tensor, timestep: float) -> torch.Tensor:
        """x_t: [B, 3, H, W] normalised Oklab (any dtype); returns the velocity [B, 3, H, W] in fp32."""
        B, _, H, W = x_t.shape
        hw = (H // PATCH, W // PATCH)
        packed = pack_latents(x_t.float(), PATCH)
        cal = compute_calibration(timestep, self.scale_buffer, self.num_timesteps)
        dt = next(self.transformer.parameters()).dtype
        t = torch.full((B,), cal.cal_timestep, device=x_t.device, dtype=torch.float32)
        u_a = self.transformer((packed * cal.k).to(dt), txt, t, hw=hw)
        return unpack_latents(asymflow_velocity(u_a, packed, cal, self.proj_buffer), hw[0], hw[1], PATCH)

    @torch.no_grad()
    def sample(self, noise: torch.Tensor, txt: torch.Tensor, neg_txt: Optional[torch.Tensor] = None, steps: int = 28,
               cfg_scale: float = 4.0, cfg_ortho: float = 1.0, shift: Optional[float] = None) -> torch.Tensor:
        """Euler sampling from pixel noise [B, 3, H, W]; returns sRGB in [-1, 1]."""
        x = noise.float()
        sig = sigma_schedule(steps, dynamic_shift(x.shape[-2], x.shape[-1]) if shift is None else shift)
        for i in range(steps):
            s0, s1 = sig[i], sig[i + 1]
            u = self.forward(x, txt, s0)
            if cfg_scale != 1.0 and neg_txt is not None:
                u = u + guidance_bias(u, self.forward(x, neg_txt, s0), cfg_scale, cfg_ortho, x - u * s0)
            x = x + clamp_denoised_oklab(x, u, s0) * (s1 - s0)
        return oklab_decode(x)
