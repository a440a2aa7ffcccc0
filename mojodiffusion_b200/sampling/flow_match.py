"""Flow-matching sigma schedules and the Euler sampler loop.

Schedules (host-side scalar math, returned as python floats / fp64 tensors):
* ``shifted_sigmas``      sigma_i = shift*t/(1+(shift-1)t), t = 1 - i/N  (serenitymojo/sampling/flow_match.mojo:42-66)
* ``flux1_sigmas``        BFL time shift with mu = lerp((256,0.5),(4096,1.15))(image_seq_len)
                          (serenitymojo/sampling/flux1_dev.mojo:94-141)
* ``flux2_klein_mu``      empirical mu of FLUX.2 / Klein (serenitymojo/sampling/flux2_klein.mojo:24-46)
* ``qwen_image_sigmas``   linspace(1, 1/N) -> exponential shift with mu(seq_len) -> stretch to terminal 0.02 -> 0
                          (serenitymojo/sampling/flow_match.mojo:120-255)
* ``ltx2_linear_quadratic_sigmas``  (serenitymojo/sampling/ltx2_sampling.mojo:123-198)
* ``sd3_sigmas``          static shift 3.0 schedule (serenitymojo/sampling/sd3_flow_match.mojo)

``euler_flow_sample`` runs the denoise loop: fp32 latent state, bf16 model input, one fused CFG + Euler kernel per
step (serenitymojo/sampling/flow_match.mojo:69-91; loop body serenitymojo/serve/flux_backend.mojo:482-512).
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import torch

from .. import ops

CFG_NONE, CFG_TEXTBOOK, CFG_COND_ANCHORED = 0, 1, 2


def shifted_sigmas(num_steps: int, shift: float = 1.0) -> List[float]:
    out = []
    for i in range(num_steps + 1):
        t = 1.0 - i / num_steps
        out.append(shift * t / (1.0 + (shift - 1.0) * t))
    return out


def _lin(x1, y1, x2, y2):
    m = (y2 - y1) / (x2 - x1)
    b = y1 - m * x1
    return lambda x: m * x + b


def flux1_mu(image_seq_len: int, base_shift: float = 0.5, max_shift: float = 1.15) -> float:
    return _lin(256, base_shift, 4096, max_shift)(image_seq_len)


def time_shift(mu: float, sigma: float, t: float) -> float:
    if t <= 0.0:
        return 0.0
    return math.exp(mu) / (math.exp(mu) + (1.0 / t - 1.0) ** sigma)


def flux1_sigmas(num_steps: int, image_seq_len: int, shift: bool = True) -> List[float]:
    """N+1 values from exactly 1 to exactly 0."""
    ts = [1.0 - i / num_steps for i in range(num_steps + 1)]
    if not shift:
        return ts
    mu = flux1_mu(image_seq_len)
    out = [time_shift(mu, 1.0, t) for t in ts]
    out[0], out[-1] = 1.0, 0.0
    return out


def flux2_klein_mu(image_seq_len: int, num_steps: int) -> float:
    a1, b1 = 8.73809524e-05, 1.89833333
    a2, b2 = 0.00016927, 0.45666666
    if image_seq_len > 4300:
        return a2 * image_seq_len + b2
    m_200 = a2 * image_seq_len + b2
    m_10 = a1 * image_seq_len + b1
    a = (m_200 - m_10) / 190.0
    b = m_200 - 200.0 * a
    return a * num_steps + b


def flux2_klein_sigmas(num_steps: int, image_seq_len: int) -> List[float]:
    mu = flux2_klein_mu(image_seq_len, num_steps)
    ts = [1.0 - i / num_steps for i in range(num_steps + 1)]
    out = [time_shift(mu, 1.0, t) for t in ts]
    out[0], out[-1] = 1.0, 0.0
    return out


def qwen_image_mu(seq_len: int, base_len=256, max_len=8192, base_shift=0.5, max_shift=0.9) -> float:
    m = (max_shift - base_shift) / (max_len - base_len)
    return seq_len * m + (base_shift - m * base_len)


def qwen_image_sigmas(num_steps: int, seq_len: int, shift_terminal: float = 0.02) -> List[float]:
    sig = [1.0 + i * (1.0 / num_steps - 1.0) / (num_steps - 1) for i in range(num_steps)] if num_steps > 1 else [1.0]
    mu = qwen_image_mu(seq_len)
    sig = [math.exp(mu) / (math.exp(mu) + (1.0 / s - 1.0)) for s in sig]
    one_minus = [1.0 - s for s in sig]
    scale = one_minus[-1] / (1.0 - shift_terminal)
    sig = [1.0 - o / scale for o in one_minus]
    return sig + [0.0]


def sd3_sigmas(num_steps: int, shift: float = 3.0) -> List[float]:
    return shifted_sigmas(num_steps, shift)


def ltx2_linear_quadratic_sigmas(num_steps: int, threshold_noise: float = 0.025,
                                 linear_steps: Optional[int] = None) -> List[float]:
    if num_steps == 1:
        return [1.0, 0.0]
    ls = linear_steps if linear_steps is not None else num_steps // 2
    lin = [i * threshold_noise / ls for i in range(ls)]
    tnsd = ls - threshold_noise * num_steps
    qs = num_steps - ls
    qc = tnsd / (ls * qs ** 2)
    lc = threshold_noise / ls - 2.0 * tnsd / (qs ** 2)
    const = qc * (ls ** 2)
    quad = [qc * (i ** 2) + lc * i + const for i in range(ls, num_steps)]
    sched = lin + quad + [1.0]
    return [1.0 - x for x in sched]


def ltx2_token_shift_sigmas(num_steps: int, num_tokens: int, base_shift: float = 0.95, max_shift: float = 2.05,
                            terminal: Optional[float] = 0.1) -> List[float]:
    """Token-count dependent exponential shift with optional stretch to a terminal sigma."""
    mu = _lin(1024, base_shift, 4096, max_shift)(num_tokens)
    ts = [1.0 - i / num_steps for i in range(num_steps + 1)]
    sig = [time_shift(mu, 1.0, t) if t > 0 else 0.0 for t in ts]
    if terminal is not None:
        nz = [s for s in sig if s != 0.0]
        one_minus = [1.0 - s for s in nz]
        scale = one_minus[-1] / (1.0 - terminal)
        nz = [1.0 - o / scale for o in one_minus]
        sig = nz + [0.0] * (len(sig) - len(nz))
    return sig


@torch.no_grad()
def euler_flow_sample(model_fn: Callable[[torch.Tensor, float], torch.Tensor], x: torch.Tensor,
                      sigmas: Sequence[float], uncond_fn: Optional[Callable] = None, cfg_scale: float = 1.0,
                      cfg_mode: int = CFG_NONE, callback: Optional[Callable[[int, torch.Tensor], None]] = None,
                      final_denoise: bool = False) -> torch.Tensor:
    """Euler integration of dx/dsigma = v.

    ``model_fn(x_model_dtype, sigma) -> v`` (and ``uncond_fn`` for classifier-free guidance). The latent state
    ``x`` is kept in fp32 across steps and handed to the model in bf16 (GPU) / its own dtype (CPU). With
    ``final_denoise`` the last step returns ``x - v * sigma`` (LTX-2 convention).
    """
    x = x.float().contiguous()
    on_gpu = x.is_cuda
    xb = x.to(torch.bfloat16) if on_gpu else x
    n = len(sigmas) - 1
    for i in range(n):
        s, s_next = float(sigmas[i]), float(sigmas[i + 1])
        vc = model_fn(xb, s)
        vu = uncond_fn(xb, s) if (uncond_fn is not None and cfg_mode != CFG_NONE) else None
        dt = (0.0 - s) if (final_denoise and i == n - 1) else (s_next - s)
        if on_gpu:
            ops.cfg_euler(x, vc.to(torch.bfloat16), vu.to(torch.bfloat16) if vu is not None else None, dt, cfg_scale,
                          cfg_mode if vu is not None else CFG_NONE, x_bf16=xb)
        else:
            ops.cfg_euler(x, vc, vu, dt, cfg_scale, cfg_mode if vu is not None else CFG_NONE)
            xb = x
        if callback is not None:
            callback(i, x)
    return x
