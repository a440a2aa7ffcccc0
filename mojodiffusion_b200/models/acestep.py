"""ACE-Step 1.5 audio DiT: a 1-D diffusion transformer over acoustic latents with lyric / timbre / text conditioning.

The noisy latent [B, T, 64] is concatenated with context latents [B, T, 128], padded to an even length and embedded by a
stride-2 1-D convolution (two frames per token). 24 layers of width 2048 (16 query heads, 8 key / value heads of 128):
self-attention with QK-RMSNorm, half-split rotary over the token index (theta 1e6) and adaLN (shift, scale, gate); even
layers restrict every token to a bidirectional window of +-128 tokens, odd layers attend to everything; cross-attention to
the projected condition sequence (QK-RMSNorm, no rotary, plain residual); SwiGLU MLP with adaLN. The six modulation
vectors are a learned per-layer table plus a projection of the time embedding, which is the sum of the embeddings of t and
of t - r (two timestep MLPs: the model is trained on intervals). Output: RMSNorm + 2-way adaLN + stride-2 transposed
convolution back to [B, T, 64].

Behaviour and checkpoint keys: serenitymojo/models/dit/acestep_dit.mojo:8-771. Windowed layers longer than the window run
``scaled_dot_product_attention`` with a band mask (the tcgen05 attention kernel has key-length masks only).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, timestep_embedding


@dataclass
class AceStepConfig:
    hidden: int = 2048
    heads: int = 16
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 6144
    depth: int = 24
    in_channels: int = 192          # 128 context + 64 acoustic
    acoustic_dim: int = 64
    patch: int = 2
    theta: float = 1.0e6
    eps: float = 1e-6
    sliding_window: int = 128
    name: str = "ace-step-1.5-turbo"


def tiny_acestep_config() -> AceStepConfig:
    return AceStepConfig(hidden=128, heads=4, kv_heads=2, head_dim=32, intermediate=256, depth=2, in_channels=24,
                         acoustic_dim=8, sliding_window=4, name="tiny-ace-step")


def _rope_half(x, cos, sin):
    """Half-split rotation of [B, S, H, Dh] by tables [S, Dh / 2]."""
    c, s = cos[None, :, None].to(x.dtype), sin[None, :, None].to(x.dtype)
    a, b = x.chunk(2, -1)
    return torch.cat((a * c - b * s, b * c + a * s), -1)


class _Attn(nn.Module):
    def __init__(self, cfg: AceStepConfig, dtype, device):
        super().__init__()
        D, kv = cfg.hidden, cfg.kv_heads * cfg.head_dim
        self.q_proj = Linear(D, cfg.heads * cfg.head_dim, False, dtype, device)
        self.k_proj = Linear(D, kv, False, dtype, device)
        self.v_proj = Linear(D, kv, False, dtype, device)
        self.o_proj = Linear(cfg.heads * cfg.head_dim, D, False, dtype, device)
        self.q_norm = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)
        self.k_norm = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)

    def forward(self, cfg, x, kv_src, rope=None, window: int = 0):
        H, KV, Dh = cfg.heads, cfg.kv_heads, cfg.head_dim
        q = self.q_norm(self.q_proj(x).unflatten(-1, (H, Dh)))
        k = self.k_norm(self.k_proj(kv_src).unflatten(-1, (KV, Dh)))
        v = self.v_proj(kv_src).unflatten(-1, (KV, Dh))
        if rope is not None:
            q, k = _rope_half(q, *rope), _rope_half(k, *rope)
        k, v = k.repeat_interleave(H // KV, 2), v.repeat_interleave(H // KV, 2)
        S = x.shape[1]
        if window > 0 and S > window:
            i = torch.arange(S, device=x.device)
            band = (i[:, None] - i[None, :]).abs() <= window
            o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2),
                                                                 attn_mask=band).transpose(1, 2)
        else:
            o = ops.attention(q, k, v)
        return self.o_proj(o.flatten(-2))


class _Mlp(nn.Module):
    def __init__(self, cfg: AceStepConfig, dtype, device):
        super().__init__()
        self.gate_proj = Linear(cfg.hidden, cfg.intermediate, False, dtype, device)
        self.up_proj = Linear(cfg.hidden, cfg.intermediate, False, dtype, device)
        self.down_proj = Linear(cfg.intermediate, cfg.hidden, False, dtype, device)

    def forward(self, x):
        return self.down_proj(ops.activation(self.gate_proj(x), "silu") * self.up_proj(x))


class AceStepLayer(nn.Module):
    def __init__(self, cfg: AceStepConfig, layer: int, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.window = cfg.sliding_window if (layer + 1) % 2 == 1 else 0           # even layers are windowed
        D = cfg.hidden
        self.scale_shift_table = nn.Parameter(torch.zeros(1, 6, D, dtype=dtype, device=device))
        self.self_attn_norm = RMSNorm(D, cfg.eps, dtype, device)
        self.cross_attn_norm = RMSNorm(D, cfg.eps, dtype, device)
        self.mlp_norm = RMSNorm(D, cfg.eps, dtype, device)
        self.self_attn = _Attn(cfg, dtype, device)
        self.cross_attn = _Attn(cfg, dtype, device)
        self.mlp = _Mlp(cfg, dtype, device)

    def forward(self, x, timestep_proj, enc, rope):
        cfg, S = self.cfg, x.shape[1]
        m = self.scale_shift_table + timestep_proj                                  # [B, 6, D]
        sh1, sc1, g1, sh2, sc2, g2 = (m[:, j] for j in range(6))
        u = self.self_attn_norm(x, scale=sc1, shift=sh1)
        x = ops.gate_residual(x, self.self_attn(cfg, u, u, rope, self.window), g1, S)
        x = x + self.cross_attn(cfg, self.cross_attn_norm(x), enc)
        return ops.gate_residual(x, self.mlp(self.mlp_norm(x, scale=sc2, shift=sh2)), g2, S)


class _TimeEmbed(nn.Module):
    def __init__(self, D, dtype, device):
        super().__init__()
        self.linear_1 = Linear(256, D, True, dtype, device)
        self.linear_2 = Linear(D, D, True, dtype, device)
        self.time_proj = Linear(D, 6 * D, True, dtype, device)

    def forward(self, t):
        dt = self.linear_1.weight.dtype
        temb = self.linear_2(self.linear_1(timestep_embedding(t, 256).to(dt), act="silu"))
        return temb, self.time_proj(ops.activation(temb, "silu")).unflatten(-1, (6, -1))


class _Decoder(nn.Module):
    def __init__(self, cfg: AceStepConfig, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.time_embed = _TimeEmbed(D, dtype, device)
        self.time_embed_r = _TimeEmbed(D, dtype, device)
        self.proj_in = nn.ModuleList([nn.Identity(), nn.Conv1d(cfg.in_channels, D, cfg.patch, cfg.patch, dtype=dtype, device=device)])
        self.condition_embedder = Linear(D, D, True, dtype, device)
        self.layers = nn.ModuleList([AceStepLayer(cfg, i, dtype, device) for i in range(cfg.depth)])
        self.scale_shift_table = nn.Parameter(torch.zeros(1, 2, D, dtype=dtype, device=device))
        self.norm_out = RMSNorm(D, cfg.eps, dtype, device)
        self.proj_out = nn.ModuleList([nn.Identity(), nn.ConvTranspose1d(D, cfg.acoustic_dim, cfg.patch, cfg.patch, dtype=dtype, device=device)])


class AceStepDiT(nn.Module):
    """forward(x_t [B, T, 64], context [B, T, 128], condition [B, L, hidden], t [B], r [B] or None) -> velocity [B, T, 64].
    ``t`` and ``r`` lie in [0, 1]; the second embedding sees ``t - r``."""

    def __init__(self, cfg: AceStepConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.decoder = _Decoder(cfg, dtype, device)
        self.gradient_checkpointing = False

    def forward(self, x_t, context, condition, t, r: Optional[torch.Tensor] = None):
        cfg, d = self.cfg, self.decoder
        B, T, _ = x_t.shape
        ps, D = cfg.patch, cfg.hidden
        w_in, w_out = d.proj_in[1], d.proj_out[1]
        dt = w_in.weight.dtype
        r = t if r is None else r
        temb_t, proj_t = d.time_embed(t)
        temb_r, proj_r = d.time_embed_r(t - r)
        temb, timestep_proj = temb_t + temb_r, proj_t + proj_r
        xin = torch.cat((context, x_t), -1).to(dt)
        pad = (-T) % ps
        if pad:
            xin = torch.nn.functional.pad(xin, (0, 0, 0, pad))
        S = (T + pad) // ps
        # stride = kernel convolution as a GEMM over [B, S, ps * Cin] rows (token vector ordered (frame, channel))
        x = ops.linear(xin.reshape(B, S, ps * cfg.in_channels), w_in.weight.permute(0, 2, 1).reshape(D, -1), w_in.bias)
        enc = d.condition_embedder(condition.to(dt))
        half = cfg.head_dim // 2
        inv = 1.0 / (cfg.theta ** (torch.arange(half, dtype=torch.float64) * 2 / cfg.head_dim))
        ang = torch.arange(S, dtype=torch.float64)[:, None] * inv[None]
        rope = (ang.cos().float().to(x.device), ang.sin().float().to(x.device))
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for layer in d.layers:
            if ckpt:
                x = torch.utils.checkpoint.checkpoint(layer, x, timestep_proj, enc, rope, use_reentrant=False, preserve_rng_state=False)
            else:
                x = layer(x, timestep_proj, enc, rope)
        m = d.scale_shift_table + temb[:, None]
        x = d.norm_out(x, scale=m[:, 1], shift=m[:, 0])
        # transposed convolution with stride = kernel: every token expands to ps frames
        y = ops.linear(x, w_out.weight.permute(2, 1, 0).reshape(ps * cfg.acoustic_dim, D), w_out.bias.repeat(ps))
        return y.reshape(B, S * ps, cfg.acoustic_dim)[:, :T]

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
