"""Nucleus-Image: a 17B sparse mixture-of-experts image DiT (image-only residual stream, text as extra keys / values).

32 blocks of width 2048 (16 query heads, 4 key / value heads of 128: grouped-query attention). Per block the text features
(RMS-normalised once, 4096 wide) get their own projection to the model width and enter attention only as added keys and
values (own K / V projections, own key norm, rotary positions continuing after the image grid); queries are image tokens.
Modulation per block is (scale1, gate1, scale2, gate2) from ``Linear(silu(temb))``; gates are clamped to +-2 and passed
through tanh. Blocks 0-2 have a dense SwiGLU feed-forward, blocks 3-31 an expert-choice mixture of 64 experts (capacity
factor 4 for blocks 3-4, 2 afterwards, gates renormalised per token and scaled by 2.5) plus a shared dense expert. The
router sees the concatenation of the time embedding and the un-modulated normalised hidden state. Rotary: interleaved
pairs, axes (16, 56, 56), centred ("signed") height / width positions.

Behaviour and checkpoint keys: serenitymojo/models/dit/nucleus_dit.mojo:8-860, serenitymojo/models/dit/nucleus_moe.mojo:27-110.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import moe
from .layers import Linear, RMSNorm, init_module_weights, timestep_embedding


@dataclass
class NucleusConfig:
    depth: int = 32
    heads: int = 16
    kv_heads: int = 4
    head_dim: int = 128
    hidden: int = 2048
    joint_dim: int = 4096
    num_experts: int = 64
    moe_inner: int = 1344
    route_scale: float = 2.5
    patch: int = 2
    in_channels: int = 64
    out_channels: int = 16
    theta: float = 10000.0
    eps: float = 1e-6
    axes_dim: Tuple[int, int, int] = (16, 56, 56)
    dense_layers: int = 3
    name: str = "nucleus-image"

    @property
    def dense_inner(self) -> int:
        return int(self.hidden * 4.0 * 2.0 / 3.0) // 128 * 128

    def capacity_factor(self, layer: int) -> float:
        if layer < self.dense_layers:
            return 0.0
        return 4.0 if layer < self.dense_layers + 2 else 2.0


def tiny_nucleus_config() -> NucleusConfig:
    return NucleusConfig(depth=5, heads=4, kv_heads=2, head_dim=64, hidden=256, joint_dim=96, num_experts=4, moe_inner=128,
                         in_channels=16, out_channels=4, axes_dim=(16, 24, 24), dense_layers=2, name="tiny-nucleus")


def _signed(n: int) -> torch.Tensor:
    neg = n - n // 2
    return torch.cat((torch.arange(-neg, 0), torch.arange(n // 2))).float()


def nucleus_rope(f: int, h: int, w: int, n_txt: int, cfg: NucleusConfig, device=None):
    """(image cos, sin [f h w, head_dim / 2], text cos, sin [n_txt, head_dim / 2]) in fp32. Height / width positions are
    centred; every axis of a text token carries max(h, w) // 2 + its index."""
    pos = torch.stack(torch.meshgrid(torch.arange(f).float(), _signed(h), _signed(w), indexing="ij"), -1).reshape(-1, 3).double()
    tpos = (max(h // 2, w // 2) + torch.arange(n_txt)).double()[:, None].expand(n_txt, 3)
    out = []
    for p in (pos, tpos):
        parts = []
        for a, d in enumerate(cfg.axes_dim):
            inv = 1.0 / (cfg.theta ** (torch.arange(d // 2).double() / (d // 2)))
            parts.append(p[:, a:a + 1] * inv[None])
        ang = torch.cat(parts, -1)
        out += [ang.cos().float().to(device), ang.sin().float().to(device)]
    return tuple(out)


class _Attn(nn.Module):
    def __init__(self, cfg: NucleusConfig, dtype, device):
        super().__init__()
        D, kv = cfg.hidden, cfg.kv_heads * cfg.head_dim
        self.to_q = Linear(D, cfg.heads * cfg.head_dim, False, dtype, device)
        self.to_k = Linear(D, kv, False, dtype, device)
        self.to_v = Linear(D, kv, False, dtype, device)
        self.add_k_proj = Linear(D, kv, False, dtype, device)
        self.add_v_proj = Linear(D, kv, False, dtype, device)
        self.norm_q = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)
        self.norm_k = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)
        self.norm_added_k = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)
        self.to_out = nn.ModuleList([Linear(cfg.heads * cfg.head_dim, D, False, dtype, device)])


class _Ffn(nn.Module):
    """SwiGLU with the up rows first and the gate rows second in ``net.0.proj`` (silu(gate) * up)."""

    def __init__(self, dim, inner, dtype, device):
        super().__init__()
        self.net = nn.ModuleList([nn.ModuleDict({"proj": Linear(dim, 2 * inner, False, dtype, device)}), nn.Identity(),
                                  Linear(inner, dim, False, dtype, device)])

    def forward(self, x):
        return self.net[2](ops.linear_glu(x, self.net[0]["proj"].weight, None, "silu", True))


class _Experts(nn.Module):
    def __init__(self, cfg: NucleusConfig, dtype, device):
        super().__init__()
        self.gate_up_proj = nn.Parameter(torch.empty(cfg.num_experts, cfg.hidden, 2 * cfg.moe_inner, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(cfg.num_experts, cfg.moe_inner, cfg.hidden, dtype=dtype, device=device))


class _MoE(nn.Module):
    def __init__(self, cfg: NucleusConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.gate = Linear(2 * cfg.hidden, cfg.num_experts, False, dtype, device)
        self.experts = _Experts(cfg, dtype, device)
        self.shared_expert = _Ffn(cfg.hidden, cfg.moe_inner, dtype, device)

    def forward(self, modulated, unmodulated, temb, capacity_factor: float):
        cfg = self.cfg
        B, S, D = modulated.shape
        capacity = max(1, math.ceil(capacity_factor * S / cfg.num_experts))
        router_in = torch.cat((temb[:, None].expand(B, S, D), unmodulated), -1)
        scores = torch.softmax(self.gate(router_in).float(), -1).to(torch.bfloat16).float()      # bf16-rounded affinities
        idx, gate = moe.expert_choice_route(scores.transpose(1, 2), capacity, cfg.route_scale)
        routed = moe.expert_choice_ffn(modulated.reshape(B * S, D), idx, gate, self.experts.gate_up_proj, self.experts.down_proj)
        return self.shared_expert(modulated) + routed.reshape(B, S, D)


class NucleusBlock(nn.Module):
    def __init__(self, cfg: NucleusConfig, layer: int, dtype, device):
        super().__init__()
        self.cfg, self.layer = cfg, layer
        D = cfg.hidden
        self.img_mod = nn.ModuleList([nn.Identity(), Linear(D, 4 * D, True, dtype, device)])
        self.encoder_proj = Linear(cfg.joint_dim, D, True, dtype, device)
        self.attn = _Attn(cfg, dtype, device)
        self.img_mlp = _Ffn(D, cfg.dense_inner, dtype, device) if layer < cfg.dense_layers else _MoE(cfg, dtype, device)

    def forward(self, x, enc_normed, temb, rope):
        cfg, a = self.cfg, self.attn
        B, S, D = x.shape
        H, KV, Dh = cfg.heads, cfg.kv_heads, cfg.head_dim
        icos, isin, tcos, tsin = rope
        m = self.img_mod[1](ops.activation(temb, "silu"))
        scale1, scale2 = m[:, :D], m[:, 2 * D:3 * D]
        gate1, gate2 = m[:, D:2 * D].clamp(-2.0, 2.0), m[:, 3 * D:].clamp(-2.0, 2.0)
        ctx = self.encoder_proj(enc_normed)
        h = ops.norm_modulate(x, scale=scale1, eps=cfg.eps)
        q = _rope_pairs(a.norm_q(a.to_q(h).unflatten(-1, (H, Dh))), icos, isin)
        k = torch.cat((_rope_pairs(a.norm_k(a.to_k(h).unflatten(-1, (KV, Dh))), icos, isin),
                       _rope_pairs(a.norm_added_k(a.add_k_proj(ctx).unflatten(-1, (KV, Dh))), tcos, tsin)), 1)
        v = torch.cat((a.to_v(h), a.add_v_proj(ctx)), 1).unflatten(-1, (KV, Dh))
        rep = H // KV
        o = ops.attention(q, k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)).flatten(-2)
        x = ops.gate_residual(x, a.to_out[0](o), gate1, S, tanh_gate=True)
        un = ops.norm_modulate(x, eps=cfg.eps)
        h = ops.norm_modulate(x, scale=scale2, eps=cfg.eps)
        y = self.img_mlp(h) if self.layer < cfg.dense_layers else self.img_mlp(h, un, temb, cfg.capacity_factor(self.layer))
        return ops.gate_residual(x, y, gate2, S, tanh_gate=True)


def _rope_pairs(x, cos, sin):
    """Interleaved-pair rotation of [B, S, H, Dh] by per-token tables [S, Dh / 2]."""
    c, s = cos[None, :, None].to(x.dtype), sin[None, :, None].to(x.dtype)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)


class _TimeTextEmbed(nn.Module):
    def __init__(self, D, eps, dtype, device):
        super().__init__()
        self.timestep_embedder = nn.ModuleDict({"linear_1": Linear(D, D, True, dtype, device), "linear_2": Linear(D, D, True, dtype, device)})
        self.norm = RMSNorm(D, eps, dtype, device)


class _NormOut(nn.Module):
    def __init__(self, D, dtype, device):
        super().__init__()
        self.linear = Linear(D, 2 * D, True, dtype, device)


class NucleusDiT(nn.Module):
    """forward(tokens [B, f h w, 64] (2 x 2 patches of 16 latent channels), text [B, S_txt, 4096], t [B] in [0, 1],
    grid (f, h, w)) -> [B, f h w, patch^2 * out_channels]."""

    def __init__(self, cfg: NucleusConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert sum(cfg.axes_dim) == cfg.head_dim and cfg.heads % cfg.kv_heads == 0
        self.img_in = Linear(cfg.in_channels, D, True, dtype, device)
        self.txt_norm = RMSNorm(cfg.joint_dim, cfg.eps, dtype, device)
        self.time_text_embed = _TimeTextEmbed(D, cfg.eps, dtype, device)
        self.transformer_blocks = nn.ModuleList([NucleusBlock(cfg, i, dtype, device) for i in range(cfg.depth)])
        self.norm_out = _NormOut(D, dtype, device)
        self.proj_out = Linear(D, cfg.patch ** 2 * cfg.out_channels, False, dtype, device)
        self.gradient_checkpointing = False

    def forward(self, tokens, text, timesteps, grid: Tuple[int, int, int]):
        cfg = self.cfg
        dt = self.img_in.weight.dtype
        D = cfg.hidden
        x = self.img_in(tokens.to(dt))
        enc = self.txt_norm(text.to(dt))
        te = self.time_text_embed
        emb = te.timestep_embedder
        temb = te.norm(emb["linear_2"](emb["linear_1"](timestep_embedding(timesteps, D).to(dt), act="silu")))
        rope = nucleus_rope(*grid, text.shape[1], cfg, tokens.device)
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.transformer_blocks:
            if ckpt:
                x = torch.utils.checkpoint.checkpoint(blk, x, enc, temb, rope, use_reentrant=False, preserve_rng_state=False)
            else:
                x = blk(x, enc, temb, rope)
        m = self.norm_out.linear(ops.activation(temb, "silu"))
        return self.proj_out(ops.norm_modulate(x, scale=m[:, :D], shift=m[:, D:], eps=cfg.eps))

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
