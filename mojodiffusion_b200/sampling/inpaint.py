"""img2img / inpaint / outpaint helpers, LanPaint inner loop, variation-seed noise and reference-latent packing
(serenitymojo/sampling/inpaint.mojo:65-133, img2img_refpack.mojo:42-108, variation_noise.mojo:41,
klein_reference_latent_bridge.mojo)."""
from __future__ import annotations

import math
from typing import Callable, Optional, Tuple

import torch


def img2img_start(latent: torch.Tensor, noise: torch.Tensor, sigmas, strength: float):
    """Start a flow-matching run part-way: returns (x_start, first_index) with x = (1 - s) latent + s noise."""
    n = len(sigmas) - 1
    first = min(max(int(round(n * (1.0 - strength))), 0), n - 1)
    s = float(sigmas[first])
    return (1.0 - s) * latent.float() + s * noise.float(), first


def inpaint_blend(x: torch.Tensor, known_latent: torch.Tensor, noise: torch.Tensor, mask: torch.Tensor, sigma: float):
    """mask = 1 where content is generated; elsewhere the known latent re-noised to the current sigma is pasted."""
    known = (1.0 - sigma) * known_latent.float() + sigma * noise.float()
    return mask * x.float() + (1.0 - mask) * known


@torch.no_grad()
def lanpaint_inner(x, score_fn: Callable[[torch.Tensor], torch.Tensor], known_latent, mask, sigma: float,
                   n_steps: int = 5, step_size: float = 0.15, friction: float = 15.0, lam: float = 4.0,
                   generator: Optional[torch.Generator] = None):
    """Overdamped Langevin refinement of the masked region before each outer step: the drift mixes the model score
    with an attraction (strength lam) of the known region towards the observed latent."""
    x = x.float()
    for _ in range(n_steps):
        drift = score_fn(x).float()
        known_t = (1.0 - sigma) * known_latent.float()
        drift = drift + lam * (1.0 - mask) * (known_t - x * (1.0 - sigma)) / max(sigma * sigma, 1e-4)
        noise = torch.randn(x.shape, generator=generator).to(x.device) if generator is not None else torch.randn_like(x)
        dt = step_size / friction
        x = x + dt * drift + math.sqrt(2.0 * dt) * sigma * noise * 0.1
    return x


def slerp(a: torch.Tensor, b: torch.Tensor, t: float) -> torch.Tensor:
    af, bf = a.float().flatten(), b.float().flatten()
    dot = torch.clamp(torch.dot(af / af.norm(), bf / bf.norm()), -1.0, 1.0)
    omega = torch.acos(dot)
    if float(omega.abs()) < 1e-6:
        return ((1 - t) * a.float() + t * b.float())
    so = torch.sin(omega)
    return (torch.sin((1 - t) * omega) / so) * a.float() + (torch.sin(t * omega) / so) * b.float()


def variation_noise(shape, seed: int, variation_seed: int, strength: float) -> torch.Tensor:
    """SwarmUI-style variation: spherical interpolation between the base-seed noise and the variation-seed noise."""
    a = torch.randn(shape, generator=torch.Generator().manual_seed(seed))
    if strength <= 0.0:
        return a
    b = torch.randn(shape, generator=torch.Generator().manual_seed(variation_seed))
    return slerp(a, b, strength)


def pack_reference_tokens(img_tokens: torch.Tensor, img_ids: torch.Tensor, ref_tokens: torch.Tensor,
                          ref_hw: Tuple[int, int], index: int = 1):
    """Append reference-image tokens to the sequence; their ids carry `index` on axis 0 so RoPE separates them."""
    h, w = ref_hw
    ids = torch.zeros(h * w, 3, dtype=img_ids.dtype, device=img_ids.device)
    ids[:, 0] = float(index)
    ids[:, 1] = torch.arange(h, device=img_ids.device, dtype=img_ids.dtype)[:, None].expand(h, w).reshape(-1)
    ids[:, 2] = torch.arange(w, device=img_ids.device, dtype=img_ids.dtype)[None, :].expand(h, w).reshape(-1)
    return torch.cat((img_tokens, ref_tokens), dim=1), torch.cat((img_ids, ids), dim=0)


def quantize_resolution(width: int, height: int, multiple: int = 16) -> Tuple[int, int]:
    """Round to the model's pixel multiple with banker's rounding (serenitymojo/sampling/base_sampler.mojo:34-93)."""
    def bank(v):
        q = v / multiple
        f = math.floor(q)
        d = q - f
        if d > 0.5 or (d == 0.5 and f % 2 == 1):
            f += 1
        return max(multiple, int(f) * multiple)
    return bank(width), bank(height)
