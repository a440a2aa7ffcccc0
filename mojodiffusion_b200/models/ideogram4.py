"""Ideogram-4 DiT: a single-stream transformer over one joint sequence of text and image tokens.

Every position carries an indicator (0 padding, 2 image, 3 text). Image tokens enter through ``input_proj`` (128 latent
channels), text tokens through RMSNorm + ``llm_cond_proj`` of stacked language-model features (53 248 wide); a learned
two-row embedding marks image positions. 34 blocks of width 4608 (18 heads x 256): adaLN from a 512-wide conditioning
vector gives (1 + scale) before attention / MLP and a tanh gate after them, each sub-layer is RMS-normalised on the way in
AND on the way out, QK-RMSNorm (eps 1e-5) + half-split rotary with an interleaved three-axis table (theta 5e6, sections
24 / 20 / 20), SwiGLU feed-forward 12 288 wide, no biases inside the blocks. The final layer is LayerNorm without affine
times (1 + scale) and a linear back to 128 channels.

Behaviour: serenitymojo/models/dit/ideogram4_dit.mojo:60-371, serenitymojo/models/dit/ideogram4_mrope.mojo:1-60,
serenitymojo/models/ideogram4/config.mojo. Checkpoint keys are the reference's, except that ``feed_forward.w1`` and
``feed_forward.w3`` are stored stacked as ``feed_forward.w13`` (one gated GEMM); ``remap_ideogram4_keys`` converts.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Tuple

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights

IND_PAD, IND_IMAGE, IND_TEXT = 0, 2, 3


@dataclass
class Ideogram4Config:
    in_channels: int = 128
    llm_dim: int = 53248
    hidden: int = 4608
    heads: int = 18
    head_dim: int = 256
    depth: int = 34
    mlp_hidden: int = 12288
    adaln_dim: int = 512
    theta: float = 5.0e6
    mrope_section: Tuple[int, int, int] = (24, 20, 20)
    name: str = "ideogram-4"


def tiny_ideogram4_config() -> Ideogram4Config:
    return Ideogram4Config(in_channels=16, llm_dim=96, hidden=128, heads=2, head_dim=64, depth=2, mlp_hidden=256,
                           adaln_dim=32, mrope_section=(6, 5, 5), name="tiny-ideogram4")


def mrope_table(position_ids: torch.Tensor, head_dim: int, section: Tuple[int, int, int], theta: float):
    """cos / sin [L, head_dim / 2] (fp32) for positions [L, 3] = (t, h, w). Frequency slot d uses the h position when
    d % 3 == 1 and d < 3 * section[1], the w position when d % 3 == 2 and d < 3 * section[2], else the t position; the
    angle is reduced in float64 (positions reach 65 536)."""
    half = head_dim // 2
    d = torch.arange(half)
    axis = torch.zeros(half, dtype=torch.long)
    axis[(d % 3 == 1) & (d < section[1] * 3)] = 1
    axis[(d % 3 == 2) & (d < section[2] * 3)] = 2
    inv = torch.exp(-(d.float() / half) * math.log(theta))                       # fp32 inverse frequencies
    pos = position_ids.detach().float().cpu()[:, axis]                            # [L, half]
    ang = (pos * inv).double()
    ang = ang - torch.floor(ang / (2 * math.pi) + 0.5) * (2 * math.pi)
    return ang.cos().float().to(position_ids.device), ang.sin().float().to(position_ids.device)


def scalar_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    """Sin-first sinusoid of 1e4 * t with frequencies exp(-i ln(1e4) / (half - 1)) -> [B, dim] fp32."""
    half = dim // 2
    freq = torch.exp(-torch.arange(half, dtype=torch.float32, device=t.device) * (math.log(1.0e4) / (half - 1)))
    ang = (t.float()[:, None] * 1.0e4 * freq[None]).double()
    ang = ang - torch.floor(ang / (2 * math.pi) + 0.5) * (2 * math.pi)
    return torch.cat((ang.sin(), ang.cos()), -1).float()


class _Attention(nn.Module):
    def __init__(self, cfg: Ideogram4Config, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.qkv = Linear(D, 3 * D, False, dtype, device)
        self.o = Linear(D, D, False, dtype, device)
        self.norm_q = RMSNorm(cfg.head_dim, 1e-5, dtype, device)
        self.norm_k = RMSNorm(cfg.head_dim, 1e-5, dtype, device)


class _FeedForward(nn.Module):
    def __init__(self, cfg: Ideogram4Config, dtype, device):
        super().__init__()
        self.w13 = Linear(cfg.hidden, 2 * cfg.mlp_hidden, False, dtype, device)      # [w1 ; w3]: silu(w1 x) * (w3 x)
        self.w2 = Linear(cfg.mlp_hidden, cfg.hidden, False, dtype, device)


class Ideogram4Block(nn.Module):
    def __init__(self, cfg: Ideogram4Config, dtype, device):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        self.adaln_modulation = Linear(cfg.adaln_dim, 4 * D, True, dtype, device)
        self.attention_norm1 = RMSNorm(D, 1e-5, dtype, device)
        self.attention_norm2 = RMSNorm(D, 1e-5, dtype, device)
        self.ffn_norm1 = RMSNorm(D, 1e-5, dtype, device)
        self.ffn_norm2 = RMSNorm(D, 1e-5, dtype, device)
        self.attention = _Attention(cfg, dtype, device)
        self.feed_forward = _FeedForward(cfg, dtype, device)

    def forward(self, x, adaln_input, cos, sin):
        cfg, a, f = self.cfg, self.attention, self.feed_forward
        D = cfg.hidden
        S = x.shape[1]
        mod = self.adaln_modulation(adaln_input)                                   # [B, 4D]: scale, gate, scale, gate
        h = self.attention_norm1(x, scale=mod[:, 0:D])
        h = ops.qkv_attention(a.qkv(h), cfg.heads, cfg.head_dim, a.norm_q.weight, a.norm_k.weight, cos, sin,
                              interleaved=False, eps=1e-5)
        x = ops.gate_residual(x, self.attention_norm2(a.o(h)), mod[:, D:2 * D], S, tanh_gate=True)
        h = self.ffn_norm1(x, scale=mod[:, 2 * D:3 * D])
        h = f.w2(ops.linear_glu(h, f.w13.weight, None, "silu", False))
        return ops.gate_residual(x, self.ffn_norm2(h), mod[:, 3 * D:4 * D], S, tanh_gate=True)


class _TEmbedding(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        self.mlp_in = Linear(dim, dim, True, dtype, device)
        self.mlp_out = Linear(dim, dim, True, dtype, device)


class _Final(nn.Module):
    def __init__(self, cfg: Ideogram4Config, dtype, device):
        super().__init__()
        self.adaln_modulation = Linear(cfg.adaln_dim, cfg.hidden, True, dtype, device)
        self.linear = Linear(cfg.hidden, cfg.in_channels, True, dtype, device)


class Ideogram4DiT(nn.Module):
    """forward(x [B, L, 128], llm [B, L, llm_dim], t [B], indicator [B, L], position_ids [L, 3]) -> [B, L, 128] (fp32).
    Positions whose indicator is not ``IND_IMAGE`` ignore ``x``; those that are not ``IND_TEXT`` ignore ``llm``."""

    def __init__(self, cfg: Ideogram4Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert cfg.heads * cfg.head_dim == D
        self.input_proj = Linear(cfg.in_channels, D, True, dtype, device)
        self.t_embedding = _TEmbedding(D, dtype, device)
        self.adaln_proj = Linear(D, cfg.adaln_dim, True, dtype, device)
        self.llm_cond_norm = RMSNorm(cfg.llm_dim, 1e-6, dtype, device)
        self.llm_cond_proj = Linear(cfg.llm_dim, D, True, dtype, device)
        self.embed_image_indicator = nn.Embedding(2, D, dtype=dtype, device=device)
        self.layers = nn.ModuleList([Ideogram4Block(cfg, dtype, device) for _ in range(cfg.depth)])
        self.final_layer = _Final(cfg, dtype, device)
        self.gradient_checkpointing = False

    def conditioning(self, t: torch.Tensor) -> torch.Tensor:
        dt = self.input_proj.weight.dtype
        te = self.t_embedding
        c = te.mlp_out(te.mlp_in(scalar_embedding(t, self.cfg.hidden).to(dt), act="silu"))
        return self.adaln_proj(c, act="silu")                                       # [B, adaln_dim]

    def embed(self, x, llm, indicator):
        dt = self.input_proj.weight.dtype
        img = (indicator == IND_IMAGE)
        txt = (indicator == IND_TEXT)
        im, tm = img[..., None].to(dt), txt[..., None].to(dt)
        h = self.input_proj(x.to(dt) * im) * im
        h = h + self.llm_cond_proj(self.llm_cond_norm(llm.to(dt) * tm)) * tm
        return h + self.embed_image_indicator(img.long())

    def forward(self, x, llm, t, indicator, position_ids):
        cfg = self.cfg
        adaln_input = self.conditioning(t)
        cos, sin = mrope_table(position_ids, cfg.head_dim, cfg.mrope_section, cfg.theta)
        h = self.embed(x, llm, indicator)
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.layers:
            if ckpt:
                h = torch.utils.checkpoint.checkpoint(blk, h, adaln_input, cos, sin, use_reentrant=False, preserve_rng_state=False)
            else:
                h = blk(h, adaln_input, cos, sin)
        return self.final_layer.linear(self.prefinal_hidden(h, adaln_input)).float()

    def prefinal_hidden(self, h, adaln_input):
        """LayerNorm (no affine, 1e-6) times (1 + scale): the input of the final linear, which is the seam the reference's
        final-linear LoRA trainer attaches to."""
        scale = self.final_layer.adaln_modulation(ops.activation(adaln_input, "silu"))
        return ops.norm_modulate(h, scale=scale, eps=1e-6, rms=False)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)


def remap_ideogram4_keys(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Reference checkpoint names -> this module's: ``feed_forward.w1`` / ``w3`` stacked into ``feed_forward.w13``."""
    out, w1 = {}, {}
    for k, v in sd.items():
        if k.endswith("feed_forward.w1.weight"):
            w1[k[:-len("w1.weight")]] = v
        elif not k.endswith("feed_forward.w3.weight"):
            out[k] = v
    for p, a in w1.items():
        out[p + "w13.weight"] = torch.cat((a, sd[p + "w3.weight"]), 0)
    return out
