"""Guidance rules used by the samplers (reference: serenitymojo/sampling/flow_match.mojo:69-91,120-255,
serenitymojo/sampling/ltx2_guidance.mojo:44-331, serenitymojo/models/dit/ltx2_nag.mojo)."""
from __future__ import annotations

from typing import Optional, Sequence

import torch


def cfg_textbook(vc, vu, s: float):
    return vu + s * (vc - vu)


def cfg_cond_anchored(vc, vu, s: float):
    return vc + s * (vc - vu)


def cfg_true_with_norm_rescale(vc, vu, s: float, dim: int = -1, eps: float = 1e-8):
    """Qwen-Image true-CFG: combine, then rescale every token so its norm equals the conditional prediction's."""
    comb = vu + s * (vc - vu)
    cn = vc.float().norm(dim=dim, keepdim=True)
    nn_ = comb.float().norm(dim=dim, keepdim=True)
    return (comb.float() * (cn / (nn_ + eps))).to(vc.dtype)


def cfg_star_rescale(vc, vu, s: float, eps: float = 1e-8):
    """CFG-star: project the unconditional branch onto the conditional one before combining
    (alpha = <vc, vu> / |vu|^2 per sample)."""
    b = vc.shape[0]
    c, u = vc.float().reshape(b, -1), vu.float().reshape(b, -1)
    alpha = (c * u).sum(1, keepdim=True) / (u.pow(2).sum(1, keepdim=True) + eps)
    u2 = (alpha * u).reshape(vc.shape)
    return (u2 + s * (vc.float() - u2)).to(vc.dtype)


def cfg_rescale_std(guided, vc, phi: float = 0.7):
    """Rescale the guided prediction towards the conditional branch's per-sample std (guidance_rescale)."""
    b = vc.shape[0]
    sc = vc.float().reshape(b, -1).std(1).reshape(b, *([1] * (vc.dim() - 1)))
    sg = guided.float().reshape(b, -1).std(1).reshape(b, *([1] * (vc.dim() - 1)))
    resc = guided.float() * (sc / (sg + 1e-8))
    return (phi * resc + (1 - phi) * guided.float()).to(guided.dtype)


def stg_combine(v_cond, v_uncond, v_perturbed, cfg_scale: float, stg_scale: float, rescale: float = 0.0):
    """Spatio-temporal guidance: CFG plus a push away from the skip-layer (perturbed) prediction."""
    out = v_uncond + cfg_scale * (v_cond - v_uncond) + stg_scale * (v_cond - v_perturbed)
    return cfg_rescale_std(out, v_cond, rescale) if rescale > 0 else out


def stg_skip_mask(num_layers: int, skip_layers: Sequence[int]) -> torch.Tensor:
    m = torch.ones(num_layers)
    for i in skip_layers:
        m[i] = 0.0
    return m


def nag_attention_guidance(z_pos, z_neg, scale: float, tau: float = 2.5, alpha: float = 0.25):
    """Normalised attention guidance on attention outputs: extrapolate, clamp the per-token L1 norm ratio to tau,
    blend back with alpha."""
    z = z_pos.float() + scale * (z_pos.float() - z_neg.float())
    n_pos = z_pos.float().abs().sum(-1, keepdim=True)
    n_z = z.abs().sum(-1, keepdim=True)
    ratio = n_z / (n_pos + 1e-8)
    z = torch.where(ratio > tau, z * (tau / (ratio + 1e-8)), z)
    return (alpha * z + (1 - alpha) * z_pos.float()).to(z_pos.dtype)


def multimodal_guider(v_text, v_uncond, v_no_audio: Optional[torch.Tensor], s_text: float, s_cross: float = 0.0):
    """Separate scales for the text condition and for a cross-modal (audio <-> video) condition."""
    out = v_uncond + s_text * (v_text - v_uncond)
    if v_no_audio is not None and s_cross != 0.0:
        out = out + s_cross * (v_text - v_no_audio)
    return out
