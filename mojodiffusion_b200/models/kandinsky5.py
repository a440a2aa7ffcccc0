"""Kandinsky-5.0 video DiT (T2V Lite): text encoder blocks, then visual decoder blocks with self + cross attention.

Text features (3584 wide) go through a linear + LayerNorm and two encoder blocks (self-attention with 1-D rotary over the
token index, exact-GELU feed-forward). Video latents (33 channels: latent + condition + mask) are patchified 1 x 2 x 2 and
run through 32 decoder blocks: self-attention with interleaved three-axis rotary (16, 24, 24), cross-attention to the
encoded text (QK-RMSNorm, no rotary), feed-forward. Every sub-layer is ``x + gate * f(LN(x) * (1 + scale) + shift)`` with
per-sample (shift, scale, gate) from ``Linear(silu(time_embed))``; the time embedding is the sinusoid MLP plus a projected,
LayerNormed pooled text vector (768 wide). Width 1792 = 28 heads x 64, feed-forward 7168, no biases in the feed-forward.

Behaviour and checkpoint keys: serenitymojo/models/dit/kandinsky5_dit.mojo:8-691.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops.conv import patchify_3d, unpatchify_3d
from .layers import LayerNorm, Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class Kandinsky5Config:
    in_visual_dim: int = 33
    out_visual_dim: int = 16
    in_text_dim: int = 3584
    in_text_dim2: int = 768
    time_dim: int = 512
    model_dim: int = 1792
    ff_dim: int = 7168
    num_text_blocks: int = 2
    num_visual_blocks: int = 32
    axes_dim: Tuple[int, int, int] = (16, 24, 24)
    patch: Tuple[int, int, int] = (1, 2, 2)
    eps: float = 1e-6
    max_period: float = 10000.0
    name: str = "kandinsky-5-t2v-lite"

    @property
    def head_dim(self) -> int:
        return sum(self.axes_dim)

    @property
    def heads(self) -> int:
        return self.model_dim // self.head_dim


def tiny_kandinsky5_config() -> Kandinsky5Config:
    return Kandinsky5Config(in_visual_dim=5, out_visual_dim=2, in_text_dim=48, in_text_dim2=24, time_dim=32, model_dim=128,
                            ff_dim=256, num_text_blocks=1, num_visual_blocks=2, axes_dim=(16, 24, 24), name="tiny-kandinsky5")


class _Modulation(nn.Module):
    def __init__(self, time_dim, n, dtype, device):
        super().__init__()
        self.out_layer = Linear(time_dim, n, True, dtype, device)

    def forward(self, time_embed):
        return self.out_layer(ops.activation(time_embed, "silu"))


class _Attention(nn.Module):
    def __init__(self, cfg: Kandinsky5Config, dtype, device):
        super().__init__()
        D = cfg.model_dim
        self.to_query = Linear(D, D, True, dtype, device)
        self.to_key = Linear(D, D, True, dtype, device)
        self.to_value = Linear(D, D, True, dtype, device)
        self.query_norm = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)
        self.key_norm = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)
        self.out_layer = Linear(D, D, True, dtype, device)


class _FeedForward(nn.Module):
    def __init__(self, cfg: Kandinsky5Config, dtype, device):
        super().__init__()
        self.in_layer = Linear(cfg.model_dim, cfg.ff_dim, False, dtype, device)
        self.out_layer = Linear(cfg.ff_dim, cfg.model_dim, False, dtype, device)

    def forward(self, x, residual, gate, rows):
        return self.out_layer(self.in_layer(x, act="gelu"), residual=residual, gate=gate, rows_per_group=rows)


def _self_attention(a: _Attention, cfg, x, cos, sin):
    qkv = packed_projection(x, (a.to_query, a.to_key, a.to_value))
    return ops.qkv_attention(qkv, cfg.heads, cfg.head_dim, a.query_norm.weight, a.key_norm.weight, cos, sin,
                             interleaved=True, eps=cfg.eps)


class Kandinsky5EncoderBlock(nn.Module):
    def __init__(self, cfg: Kandinsky5Config, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.text_modulation = _Modulation(cfg.time_dim, 6 * cfg.model_dim, dtype, device)
        self.self_attention = _Attention(cfg, dtype, device)
        self.feed_forward = _FeedForward(cfg, dtype, device)

    def forward(self, x, time_embed, cos, sin):
        cfg, D, S = self.cfg, self.cfg.model_dim, x.shape[1]
        m = self.text_modulation(time_embed)
        sh1, sc1, g1, sh2, sc2, g2 = (m[:, j * D:(j + 1) * D] for j in range(6))
        h = _self_attention(self.self_attention, cfg, ops.norm_modulate(x, scale=sc1, shift=sh1, eps=cfg.eps), cos, sin)
        x = self.self_attention.out_layer(h, residual=x, gate=g1, rows_per_group=S)
        return self.feed_forward(ops.norm_modulate(x, scale=sc2, shift=sh2, eps=cfg.eps), x, g2, S)


class Kandinsky5DecoderBlock(nn.Module):
    def __init__(self, cfg: Kandinsky5Config, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.visual_modulation = _Modulation(cfg.time_dim, 9 * cfg.model_dim, dtype, device)
        self.self_attention = _Attention(cfg, dtype, device)
        self.cross_attention = _Attention(cfg, dtype, device)
        self.feed_forward = _FeedForward(cfg, dtype, device)

    def forward(self, x, text, time_embed, cos, sin):
        cfg, D, S = self.cfg, self.cfg.model_dim, x.shape[1]
        H, Dh = cfg.heads, cfg.head_dim
        m = self.visual_modulation(time_embed)
        sh1, sc1, g1, sh2, sc2, g2, sh3, sc3, g3 = (m[:, j * D:(j + 1) * D] for j in range(9))
        h = _self_attention(self.self_attention, cfg, ops.norm_modulate(x, scale=sc1, shift=sh1, eps=cfg.eps), cos, sin)
        x = self.self_attention.out_layer(h, residual=x, gate=g1, rows_per_group=S)
        c = self.cross_attention
        q = c.query_norm(c.to_query(ops.norm_modulate(x, scale=sc2, shift=sh2, eps=cfg.eps)).unflatten(-1, (H, Dh)))
        k = c.key_norm(c.to_key(text).unflatten(-1, (H, Dh)))
        v = c.to_value(text).unflatten(-1, (H, Dh))
        h = ops.attention(q, k, v).flatten(-2)
        x = c.out_layer(h, residual=x, gate=g2, rows_per_group=S)
        return self.feed_forward(ops.norm_modulate(x, scale=sc3, shift=sh3, eps=cfg.eps), x, g3, S)


class _InNorm(nn.Module):
    def __init__(self, din, dout, eps, dtype, device):
        super().__init__()
        self.in_layer = Linear(din, dout, True, dtype, device)
        self.norm = LayerNorm(dout, eps, True, dtype, device)

    def forward(self, x):
        return self.norm(self.in_layer(x))


class _TimeEmbeddings(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        self.in_layer = Linear(cfg.model_dim, cfg.time_dim, True, dtype, device)
        self.out_layer = Linear(cfg.time_dim, cfg.time_dim, True, dtype, device)


class _VisualIn(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        pt, ph, pw = cfg.patch
        self.in_layer = Linear(cfg.in_visual_dim * pt * ph * pw, cfg.model_dim, True, dtype, device)


class _Out(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        pt, ph, pw = cfg.patch
        self.modulation = _Modulation(cfg.time_dim, 2 * cfg.model_dim, dtype, device)
        self.out_layer = Linear(cfg.model_dim, cfg.out_visual_dim * pt * ph * pw, True, dtype, device)


class Kandinsky5DiT(nn.Module):
    """forward(latent [B, 33, F, H, W], text [B, T, 3584], pooled [B, 768], timestep [B] in the model's own units) ->
    [B, 16, F, H, W]."""

    def __init__(self, cfg: Kandinsky5Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.text_embeddings = _InNorm(cfg.in_text_dim, cfg.model_dim, cfg.eps, dtype, device)
        self.pooled_text_embeddings = _InNorm(cfg.in_text_dim2, cfg.time_dim, cfg.eps, dtype, device)
        self.time_embeddings = _TimeEmbeddings(cfg, dtype, device)
        self.visual_embeddings = _VisualIn(cfg, dtype, device)
        self.text_transformer_blocks = nn.ModuleList([Kandinsky5EncoderBlock(cfg, dtype, device) for _ in range(cfg.num_text_blocks)])
        self.visual_transformer_blocks = nn.ModuleList([Kandinsky5DecoderBlock(cfg, dtype, device) for _ in range(cfg.num_visual_blocks)])
        self.out_layer = _Out(cfg, dtype, device)
        self.gradient_checkpointing = False

    def forward(self, z, text, pooled, timesteps):
        cfg = self.cfg
        B, C, F_, Hh, Ww = z.shape
        pt, ph, pw = cfg.patch
        f, h, w = F_ // pt, Hh // ph, Ww // pw
        dt = self.visual_embeddings.in_layer.weight.dtype
        dev = z.device
        te = self.time_embeddings
        temb = timestep_embedding(timesteps, cfg.model_dim, cfg.max_period, time_factor=1.0).to(dt)
        time_embed = te.out_layer(te.in_layer(temb, act="silu")) + self.pooled_text_embeddings(pooled.to(dt))
        txt = self.text_embeddings(text.to(dt))
        T = txt.shape[1]
        tcos, tsin = ops.rope_table(torch.arange(T, device=dev, dtype=torch.float32)[:, None].contiguous(), [cfg.head_dim], cfg.max_period)
        ids = torch.stack(torch.meshgrid(torch.arange(f, device=dev), torch.arange(h, device=dev), torch.arange(w, device=dev),
                                         indexing="ij"), -1).reshape(-1, 3).float().contiguous()
        vcos, vsin = ops.rope_table(ids, list(cfg.axes_dim), cfg.max_period)
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        run = (lambda blk, *a: torch.utils.checkpoint.checkpoint(blk, *a, use_reentrant=False, preserve_rng_state=False)) if ckpt \
            else (lambda blk, *a: blk(*a))
        for blk in self.text_transformer_blocks:
            txt = run(blk, txt, time_embed, tcos, tsin)
        x = self.visual_embeddings.in_layer(patchify_3d(z, pt, ph, pw).to(dt))
        for blk in self.visual_transformer_blocks:
            x = run(blk, x, txt, time_embed, vcos, vsin)
        D = cfg.model_dim
        m = self.out_layer.modulation(time_embed)
        out = self.out_layer.out_layer(ops.norm_modulate(x, scale=m[:, D:], shift=m[:, :D], eps=cfg.eps))
        return unpatchify_3d(out, (f, h, w), cfg.out_visual_dim, pt, ph, pw)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
