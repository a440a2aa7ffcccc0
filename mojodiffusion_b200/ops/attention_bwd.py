"""Attention backward entry used by the autograd function in ``ops.functional``.

dV = P^T dO, dP = dO V^T, dS = P * (dP - rowsum(dO * O)), dQ = dS K * scale, dK = dS^T Q * scale, with P rebuilt
from the saved log-sum-exp so no [S, S] tensor is kept between forward and backward
(reference math: serenitymojo/ops/attention_backward.mojo:249-349; cuDNN path serenitymojo/ops/cshim/cudnn_sdpa_bwd.cpp:325).
"""
from __future__ import annotations

import torch

from . import native


def backward_math(q, k, v, o, lse, do, scale, kv_len=None):
    """Decomposed fp32 backward, processed in head groups so the score block stays below ~2 GiB."""
    B, Sq, H, Dh = q.shape
    Skv = k.shape[1]
    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    per_head = max(1, B * Sq * Skv * 4)
    hg = max(1, min(H, (1 << 31) // per_head))
    delta = (do.float() * o.float()).sum(-1)  # [B, Sq, H]
    mask = None
    if kv_len is not None:
        mask = (torch.arange(Skv, device=q.device)[None, :] >= kv_len[:, None])[:, None, None, :]
    for h0 in range(0, H, hg):
        h1 = min(H, h0 + hg)
        qf, kf, vf = q[:, :, h0:h1].float(), k[:, :, h0:h1].float(), v[:, :, h0:h1].float()
        dof = do[:, :, h0:h1].float()
        s = torch.einsum("bqhd,bkhd->bhqk", qf, kf) * scale
        if mask is not None:
            s = s.masked_fill(mask, float("-inf"))
        p = torch.exp(s - lse[:, h0:h1, :, None])
        dv[:, :, h0:h1] = torch.einsum("bhqk,bqhd->bkhd", p, dof).to(dv.dtype)
        dp = torch.einsum("bqhd,bkhd->bhqk", dof, vf)
        ds = p * (dp - delta[:, :, h0:h1].permute(0, 2, 1)[..., None])
        dq[:, :, h0:h1] = (torch.einsum("bhqk,bkhd->bqhd", ds, kf) * scale).to(dq.dtype)
        dk[:, :, h0:h1] = (torch.einsum("bhqk,bqhd->bkhd", ds, qf) * scale).to(dk.dtype)
    return dq, dk, dv


def backward(q, k, v, o, lse, do, scale, kv_len=None, outs=None):
    """``outs``: optional (dq, dk, dv) views to fill (e.g. the column ranges of one packed gradient buffer)."""
    if q.is_cuda and native.available() and hasattr(torch.ops.mdb200, "attention_bwd"):
        if do.stride(-1) != 1:
            do = do.contiguous()
        return torch.ops.mdb200.attention_bwd(q, k, v, o, lse, do, scale, kv_len, list(outs) if outs is not None else [])
    dq, dk, dv = backward_math(q, k, v, o, lse, do, scale, kv_len)
    if outs is not None:
        outs[0].copy_(dq), outs[1].copy_(dk), outs[2].copy_(dv)
        return outs
    return dq, dk, dv
