"""Loss functions and weights selected at run time from the train config ("levers"): MSE / Huber / smooth-L1, masked
variants, min-SNR-gamma and debiased weights in the flow-matching parametrisation, combined MSE+MAE+Huber.
With every lever at its default the result is exactly the plain MSE (serenitymojo/training/levers.mojo:13-22,55-247;
weights serenitymojo/training/loss_weight.mojo: snr(sigma) = ((1 - sigma) / sigma)^2; host losses
serenitymojo/ops/loss_fns.mojo:93-325)."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


def snr_from_sigma(sigma: torch.Tensor) -> torch.Tensor:
    s = sigma.float().clamp(1e-6, 1.0)
    return ((1.0 - s) / s) ** 2


def min_snr_weight(sigma: torch.Tensor, gamma: float, v_prediction: bool = True) -> torch.Tensor:
    snr = snr_from_sigma(sigma)
    cap = torch.minimum(snr, torch.full_like(snr, gamma))
    return cap / (snr + 1.0) if v_prediction else cap / snr.clamp_min(1e-8)


def debiased_weight(sigma: torch.Tensor, v_prediction: bool = True) -> torch.Tensor:
    snr = snr_from_sigma(sigma).clamp_max(1e3)
    return (1.0 / torch.sqrt(snr + 1.0 if v_prediction else snr)).clamp_min(1e-8)


def _elementwise(pred, target, kind: str, huber_delta: float, smooth_l1_beta: float):
    d = pred.float() - target.float()
    if kind == "mse":
        return d * d
    if kind == "mae":
        return d.abs()
    if kind == "huber":
        a = d.abs()
        return torch.where(a <= huber_delta, 0.5 * d * d, huber_delta * (a - 0.5 * huber_delta))
    if kind == "smooth_l1":
        a = d.abs()
        return torch.where(a < smooth_l1_beta, 0.5 * d * d / smooth_l1_beta, a - 0.5 * smooth_l1_beta)
    raise ValueError(kind)


def diffusion_loss(pred, target, sigma: Optional[torch.Tensor] = None, loss_fn: str = "mse", mask: Optional[torch.Tensor] = None,
                   min_snr_gamma: float = 0.0, debiased: bool = False, huber_delta: float = 1.0,
                   smooth_l1_beta: float = 1.0, mse_w: float = 1.0, mae_w: float = 0.0, huber_w: float = 0.0):
    """Scalar loss. Fast path: plain unmasked, unweighted MSE runs the fused CUDA reduction (with its analytic gradient)."""
    plain = loss_fn == "mse" and mask is None and min_snr_gamma <= 0 and not debiased and mae_w == 0 and huber_w == 0 \
        and mse_w == 1.0
    if plain:
        return ops.mse_loss(pred, target)
    if loss_fn == "combined":
        e = mse_w * _elementwise(pred, target, "mse", huber_delta, smooth_l1_beta)
        if mae_w:
            e = e + mae_w * _elementwise(pred, target, "mae", huber_delta, smooth_l1_beta)
        if huber_w:
            e = e + huber_w * _elementwise(pred, target, "huber", huber_delta, smooth_l1_beta)
    else:
        e = _elementwise(pred, target, loss_fn, huber_delta, smooth_l1_beta)
    B = e.shape[0]
    if mask is not None:
        m = mask.float().expand_as(e)
        per = (e * m).reshape(B, -1).sum(1) / m.reshape(B, -1).sum(1).clamp_min(1.0)
    else:
        per = e.reshape(B, -1).mean(1)
    if sigma is not None and min_snr_gamma > 0:
        per = per * min_snr_weight(sigma, min_snr_gamma).to(per.device)
    if sigma is not None and debiased:
        per = per * debiased_weight(sigma).to(per.device)
    return per.mean()
