"""Small training features that are off by default and leave the step bit-identical when off: offset noise, input
perturbation, multi-resolution (pyramid) noise, caption dropout, timestep bias, gradient accumulation bookkeeping and
a gradient-coverage audit (serenitymojo/training/noise_modifiers.mojo:1-40, caption_dropout.mojo:1-50,
timestep_bias.mojo:1-70, grad_accum.mojo, grad_coverage.mojo)."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, List, Optional

import torch


# ---- noise modifiers (order: offset, then input perturbation, then multires) ------------------------------
def apply_offset_noise(noise: torch.Tensor, weight: float, prob: float, generator: Optional[torch.Generator] = None,
                       channel_dim: int = -1) -> torch.Tensor:
    """With probability ``prob`` adds weight * randn per (sample, channel), broadcast over positions."""
    if weight <= 0 or prob <= 0:
        return noise
    if float(torch.rand((), generator=generator)) >= prob:
        return noise
    shape = [1] * noise.dim()
    shape[0] = noise.shape[0]
    shape[channel_dim] = noise.shape[channel_dim]
    off = torch.randn(shape, generator=generator).to(noise.device, noise.dtype)
    return noise + weight * off


def apply_input_perturbation(noise: torch.Tensor, gamma: float, generator: Optional[torch.Generator] = None):
    if gamma <= 0:
        return noise
    return noise + gamma * torch.randn(noise.shape, generator=generator).to(noise.device, noise.dtype)


def apply_multires_noise(noise: torch.Tensor, iterations: int, discount: float = 0.3,
                         generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """Pyramid noise for [B, C, H, W] tensors (other ranks pass through): adds upsampled coarser noise, each level
    scaled by discount^i, then renormalises to unit std."""
    if iterations <= 0 or noise.dim() != 4:
        return noise
    B, C, H, W = noise.shape
    out = noise.float()
    for i in range(1, iterations + 1):
        h, w = max(1, H // (2 ** i)), max(1, W // (2 ** i))
        coarse = torch.randn(B, C, h, w, generator=generator).to(noise.device)
        out = out + torch.nn.functional.interpolate(coarse, size=(H, W), mode="bilinear", align_corners=False) * discount ** i
        if h == 1 or w == 1:
            break
    return (out / out.std()).to(noise.dtype)


# ---- caption dropout -----------------------------------------------------------------------------------------
def should_drop_caption(prob: float, generator: Optional[torch.Generator] = None) -> bool:
    if prob <= 0:
        return False                      # no draw at all: the random stream is unchanged when the feature is off
    return float(torch.rand((), generator=generator)) < prob


def drop_caption(text: torch.Tensor, uncond: Optional[torch.Tensor], prob: float, generator=None) -> torch.Tensor:
    if not should_drop_caption(prob, generator):
        return text
    return torch.zeros_like(text) if uncond is None else uncond.to(text.device, text.dtype).expand_as(text)


# ---- timestep bias ---------------------------------------------------------------------------------------------
TSB_NONE, TSB_LATER, TSB_EARLIER, TSB_RANGE = 0, 1, 2, 3
_TSB_NAMES = {"none": 0, "later": 1, "earlier": 2, "range": 3}


def apply_timestep_bias(t: torch.Tensor, total: float = 1.0, strategy=TSB_NONE, multiplier: float = 0.0,
                        range_min: float = 0.0, range_max: float = 1.0) -> torch.Tensor:
    if isinstance(strategy, str):
        strategy = _TSB_NAMES[strategy.lower()]
    c = lambda x: min(max(x, 0.0), 1.0)
    if strategy == TSB_NONE:
        return t
    if strategy == TSB_LATER:
        return t + c(multiplier) * (total - t)
    if strategy == TSB_EARLIER:
        return t * (1.0 - c(multiplier))
    lo = c(range_min)
    hi = max(c(range_max), lo)
    return (lo + (t / total).clamp(0, 1) * (hi - lo)) * total


# ---- gradient accumulation -------------------------------------------------------------------------------------
@dataclass
class GradAccumulator:
    """Counts micro-steps; ``should_step`` is true on every ``steps``-th call. The loss scale for each micro-step is
    1 / steps so the accumulated gradient equals the gradient of the mean loss over the group."""
    steps: int = 1
    micro: int = 0

    @property
    def loss_scale(self) -> float:
        return 1.0 / max(1, self.steps)

    def tick(self) -> bool:
        self.micro += 1
        if self.micro >= max(1, self.steps):
            self.micro = 0
            return True
        return False


# ---- gradient coverage -----------------------------------------------------------------------------------------
@dataclass
class GradCoverage:
    """Audit that every trainable tensor receives a finite, non-zero gradient (after the first optimizer step, when
    zero-initialised factors have left zero). ``check`` returns the names that are dead or non-finite."""
    dead: List[str] = field(default_factory=list)
    nonfinite: List[str] = field(default_factory=list)

    def check(self, named: Iterable, step: int, min_step: int = 1) -> "GradCoverage":
        self.dead, self.nonfinite = [], []
        if step < min_step:
            return self
        for n, p in named:
            if not p.requires_grad:
                continue
            g = p.grad
            if g is None or not bool((g != 0).any()):
                self.dead.append(n)
            elif not bool(torch.isfinite(g).all()):
                self.nonfinite.append(n)
        return self

    @property
    def ok(self) -> bool:
        return not self.dead and not self.nonfinite
