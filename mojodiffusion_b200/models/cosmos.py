"""Cosmos-Predict2.5 (2B) DiT: self-attention + text cross-attention + MLP blocks with adaLN-LoRA modulation.

The latent (16 channels) is extended by a conditioning-frame mask and a padding mask channel (18), patchified 1 x 2 x 2
(72 values per token) and embedded without bias. Text features (100 352 wide) are projected to 1024. The sinusoid of the
timestep is RMS-normalised into ``emb``; an MLP on the same sinusoid gives a shared ``adaln_lora`` [3D]. Each of the three
sub-blocks computes (shift, scale, gate) = chunk3(W2 W1 silu(emb) + adaln_lora) with a rank-256 bottleneck, and applies
``x += gate * f(LN(x) (1 + scale) + shift)``. Attention: bias-free projections, per-head RMSNorm on q and k, half-split
three-axis rotary (44, 42, 42 of 128) with NTK-scaled per-axis bases (height and width ratio 3), cross-attention without
rotary. The final layer uses a two-chunk modulation plus the first 2D of ``adaln_lora`` and un-patchifies with the channel
as the slowest index of the token vector. Modulation is per (sample, latent frame), so frames may carry their own timestep.

Behaviour and checkpoint keys: serenitymojo/models/dit/cosmos_predict25_dit.mojo:8-696. The feed-forward uses the exact
(erf) GELU of the published network; the residual stream stays in the activation dtype, added by the GEMM epilogue.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops.conv import patchify_3d
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class CosmosConfig:
    in_channels: int = 16
    out_channels: int = 16
    model_channels: int = 2048
    heads: int = 16
    head_dim: int = 128
    depth: int = 28
    mlp_ratio: int = 4
    adaln_lora_dim: int = 256
    text_in_dim: int = 100352
    text_dim: int = 1024
    patch_spatial: int = 2
    patch_temporal: int = 1
    rope_ratio: Tuple[float, float, float] = (1.0, 3.0, 3.0)      # (t, h, w) NTK extrapolation ratios
    eps: float = 1e-6
    name: str = "cosmos-predict2.5-2b"

    @property
    def axes_dim(self) -> Tuple[int, int, int]:
        dh = self.head_dim // 6 * 2
        return (self.head_dim - 2 * dh, dh, dh)


def tiny_cosmos_config() -> CosmosConfig:
    return CosmosConfig(in_channels=4, out_channels=4, model_channels=128, heads=2, head_dim=64, depth=2, adaln_lora_dim=16,
                        text_in_dim=96, text_dim=48, name="tiny-cosmos")


def cosmos_rope_table(f: int, h: int, w: int, cfg: CosmosConfig, device=None):
    """cos / sin [f h w, head_dim / 2] (fp32): per axis a, base 10000 * ratio_a ** (dim_a / (dim_a - 2))."""
    ids = torch.stack(torch.meshgrid(torch.arange(f), torch.arange(h), torch.arange(w), indexing="ij"), -1).reshape(-1, 3).double()
    parts = []
    for a, (d, r) in enumerate(zip(cfg.axes_dim, cfg.rope_ratio)):
        theta = 10000.0 * r ** (d / (d - 2))
        freq = theta ** (-torch.arange(0, d, 2).double() / d)
        parts.append(ids[:, a:a + 1] * freq[None])
    ang = torch.cat(parts, -1)
    return ang.cos().float().to(device), ang.sin().float().to(device)


class _AdaLN(nn.ModuleDict):
    """silu -> Linear(D, r) -> Linear(r, n D), both without bias (entries "1" and "2", the checkpoint's indices)."""

    def __init__(self, D, r, n, dtype, device):
        super().__init__({"1": Linear(D, r, False, dtype, device), "2": Linear(r, n * D, False, dtype, device)})

    def forward(self, emb):
        return self["2"](self["1"](ops.activation(emb, "silu")))


class _Attn(nn.Module):
    def __init__(self, cfg: CosmosConfig, kv_dim: int, dtype, device):
        super().__init__()
        D = cfg.model_channels
        self.q_proj = Linear(D, D, False, dtype, device)
        self.k_proj = Linear(kv_dim, D, False, dtype, device)
        self.v_proj = Linear(kv_dim, D, False, dtype, device)
        self.output_proj = Linear(D, D, False, dtype, device)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)


class _Mlp(nn.Module):
    def __init__(self, cfg: CosmosConfig, dtype, device):
        super().__init__()
        D = cfg.model_channels
        self.layer1 = Linear(D, cfg.mlp_ratio * D, False, dtype, device)
        self.layer2 = Linear(cfg.mlp_ratio * D, D, False, dtype, device)


class CosmosBlock(nn.Module):
    def __init__(self, cfg: CosmosConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        D, r = cfg.model_channels, cfg.adaln_lora_dim
        self.adaln_modulation_self_attn = _AdaLN(D, r, 3, dtype, device)
        self.adaln_modulation_cross_attn = _AdaLN(D, r, 3, dtype, device)
        self.adaln_modulation_mlp = _AdaLN(D, r, 3, dtype, device)
        self.self_attn = _Attn(cfg, D, dtype, device)
        self.cross_attn = _Attn(cfg, cfg.text_dim, dtype, device)
        self.mlp = _Mlp(cfg, dtype, device)

    def forward(self, x, emb, adaln_lora, text, cos, sin, rows_per_group: int):
        cfg = self.cfg
        D, H, Dh = cfg.model_channels, cfg.heads, cfg.head_dim
        B = x.shape[0]

        def mod(layer):
            m = layer(emb) + adaln_lora                                   # [B Tp, 3D]
            return m[:, :D], m[:, D:2 * D], m[:, 2 * D:]

        x2 = x.reshape(-1, D)                                             # rows grouped by (sample, frame)
        sh, sc, g = mod(self.adaln_modulation_self_attn)
        a = self.self_attn
        u = ops.norm_modulate(x2, scale=sc, shift=sh, rows_per_group=rows_per_group, eps=cfg.eps).reshape(x.shape)
        qkv = packed_projection(u, (a.q_proj, a.k_proj, a.v_proj))
        o = ops.qkv_attention(qkv, H, Dh, a.q_norm.weight, a.k_norm.weight, cos, sin, interleaved=False, eps=cfg.eps)
        x2 = a.output_proj(o.reshape(-1, D), residual=x2, gate=g, rows_per_group=rows_per_group)
        sh, sc, g = mod(self.adaln_modulation_cross_attn)
        c = self.cross_attn
        u = ops.norm_modulate(x2, scale=sc, shift=sh, rows_per_group=rows_per_group, eps=cfg.eps).reshape(x.shape)
        q = c.q_norm(c.q_proj(u).unflatten(-1, (H, Dh)))
        k = c.k_norm(c.k_proj(text).unflatten(-1, (H, Dh)))
        v = c.v_proj(text).unflatten(-1, (H, Dh))
        x2 = c.output_proj(ops.attention(q, k, v).reshape(-1, D), residual=x2, gate=g, rows_per_group=rows_per_group)
        sh, sc, g = mod(self.adaln_modulation_mlp)
        u = ops.norm_modulate(x2, scale=sc, shift=sh, rows_per_group=rows_per_group, eps=cfg.eps)
        x2 = self.mlp.layer2(self.mlp.layer1(u, act="gelu"), residual=x2, gate=g, rows_per_group=rows_per_group)
        return x2.reshape(x.shape)


class _TEmbedder(nn.Module):
    def __init__(self, D, dtype, device):
        super().__init__()
        self.linear_1 = Linear(D, D, False, dtype, device)
        self.linear_2 = Linear(D, 3 * D, False, dtype, device)


class _Final(nn.Module):
    def __init__(self, cfg: CosmosConfig, dtype, device):
        super().__init__()
        D = cfg.model_channels
        self.adaln_modulation = _AdaLN(D, cfg.adaln_lora_dim, 2, dtype, device)
        self.linear = Linear(D, cfg.patch_spatial ** 2 * cfg.patch_temporal * cfg.out_channels, False, dtype, device)


class CosmosDiT(nn.Module):
    """forward(latent [B, 16, T, H, W], text [B, S, text_in_dim], timesteps [B] or [B, T / patch_temporal],
    cond_mask / padding_mask [B, 1, T, H, W] or None) -> [B, 16, T, H, W]."""

    def __init__(self, cfg: CosmosConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.model_channels
        patch_in = (cfg.in_channels + 2) * cfg.patch_temporal * cfg.patch_spatial ** 2
        self.x_embedder = nn.ModuleDict({"proj": nn.ModuleDict({"1": Linear(patch_in, D, False, dtype, device)})})
        self.crossattn_proj = nn.ModuleDict({"0": Linear(cfg.text_in_dim, cfg.text_dim, True, dtype, device)})
        self.t_embedder = nn.ModuleDict({"1": _TEmbedder(D, dtype, device)})
        self.t_embedding_norm = RMSNorm(D, cfg.eps, dtype, device)
        self.blocks = nn.ModuleList([CosmosBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        self.final_layer = _Final(cfg, dtype, device)
        self.gradient_checkpointing = False

    def forward(self, z, text, timesteps, cond_mask: Optional[torch.Tensor] = None, padding_mask: Optional[torch.Tensor] = None):
        cfg = self.cfg
        B, C, T, Hh, Ww = z.shape
        ps, pt, D = cfg.patch_spatial, cfg.patch_temporal, cfg.model_channels
        tp, hp, wp = T // pt, Hh // ps, Ww // ps
        dt = self.final_layer.linear.weight.dtype
        zeros = z.new_zeros(B, 1, T, Hh, Ww)
        x_in = torch.cat((z, zeros if cond_mask is None else cond_mask.to(z.dtype), zeros if padding_mask is None else padding_mask.to(z.dtype)), 1)
        x = self.x_embedder["proj"]["1"](patchify_3d(x_in, pt, ps, ps).to(dt))                 # [B, N, D]
        txt = self.crossattn_proj["0"](text.to(dt))
        tt = timesteps.float().reshape(B, -1).expand(B, tp).reshape(-1)                          # one per (sample, frame)
        sample = timestep_embedding(tt, D, 10000.0, time_factor=1.0).to(dt)                      # [B tp, D]
        te = self.t_embedder["1"]
        adaln_lora = te.linear_2(te.linear_1(sample, act="silu"))                                # [B tp, 3D]
        emb = self.t_embedding_norm(sample)
        cos, sin = cosmos_rope_table(tp, hp, wp, cfg, z.device)
        hpwp = hp * wp
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.blocks:
            if ckpt:
                x = torch.utils.checkpoint.checkpoint(blk, x, emb, adaln_lora, txt, cos, sin, hpwp, use_reentrant=False, preserve_rng_state=False)
            else:
                x = blk(x, emb, adaln_lora, txt, cos, sin, hpwp)
        m = self.final_layer.adaln_modulation(emb) + adaln_lora[:, :2 * D]
        u = ops.norm_modulate(x.reshape(-1, D), scale=m[:, D:], shift=m[:, :D], rows_per_group=hpwp, eps=cfg.eps)
        out = self.final_layer.linear(u)                                                          # [B N, p1 p2 t' c]
        out = out.reshape(B, tp, hp, wp, ps, ps, pt, cfg.out_channels).permute(0, 7, 1, 6, 2, 4, 3, 5)
        return out.reshape(B, cfg.out_channels, T, Hh, Ww)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)

