"""ERNIE-Image 8B: a single-stream DiT over [image tokens | text tokens] with ONE shared adaLN modulation for all layers.

    latent [B, 128, h, w] (Klein-VAE packed latents, patch 1) -> x_embedder (1x1 convolution = linear) -> image tokens
    text   [B, T, 3072] (Mistral-3B hidden states)          -> text_proj (no bias)
    temb = MLP(sin-first sinusoid(sigma * 1000));  (shift, scale, gate) x (attention, MLP) = adaLN_modulation(SiLU(temb))
    36 x block:  h = RMSNorm(x) * (1 + scale) + shift -> q, k, v (no bias) -> per-head RMSNorm of q / k -> 3-axis
                 half-split RoPE (axes 32 / 48 / 48, theta 256) -> attention -> to_out -> x + gate * .
                 h = RMSNorm(x) * (1 + scale) + shift -> GELU(gate_proj h) * up_proj h -> linear_fc2 -> x + gate * .
    final: RMS/LayerNorm with its own 2-way modulation -> linear -> image tokens only

Sampler: shifted sigmas (shift 3) Euler, textbook CFG 4.0, 50 steps. Key names follow the checkpoint
(``x_embedder.proj``, ``time_embedding.linear_{1,2}``, ``text_proj``, ``adaLN_modulation.1``, ``layers.{i}.adaLN_sa_ln``,
``layers.{i}.self_attention.{to_q,to_k,to_v,to_out.0,norm_q,norm_k}``, ``layers.{i}.adaLN_mlp_ln``,
``layers.{i}.mlp.{gate_proj,up_proj,linear_fc2}``, ``final_norm.linear``, ``final_linear``)
(serenitymojo/models/dit/ernie_image.mojo:280-366, ernie_contract.mojo:30-70, serenitymojo/sampling/ernie_sampling.mojo).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
from torch import nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class ErnieConfig:
    in_channels: int = 128
    hidden: int = 4096
    heads: int = 32
    head_dim: int = 128
    depth: int = 36
    ffn_hidden: int = 12288
    text_dim: int = 3072
    axes_dim: Tuple[int, int, int] = (32, 48, 48)
    theta: float = 256.0
    eps: float = 1e-6
    name: str = "ernie-image-8b"


def ernie_config() -> ErnieConfig:
    return ErnieConfig()


def tiny_ernie_config() -> ErnieConfig:
    return ErnieConfig(in_channels=16, hidden=256, heads=4, head_dim=64, depth=2, ffn_hidden=512, text_dim=96, axes_dim=(16, 24, 24),
                       name="tiny-ernie")


class _SelfAttention(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.cfg = cfg
        self.to_q, self.to_k, self.to_v = [Linear(D, D, False, dtype, device) for _ in range(3)]
        self.to_out = nn.ModuleList([Linear(D, D, False, dtype, device)])
        self.norm_q = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)
        self.norm_k = RMSNorm(cfg.head_dim, cfg.eps, dtype, device)

    def forward(self, x, cos, sin, kv_len=None):
        cfg = self.cfg
        B, S, D = x.shape
        qkv = packed_projection(x, (self.to_q, self.to_k, self.to_v))
        qkv = ops.qk_norm_rope(qkv, cfg.heads, cfg.head_dim, self.norm_q.weight, self.norm_k.weight, cos, sin, eps=cfg.eps, interleaved=False)
        q, k, v = [qkv[..., i * D:(i + 1) * D].unflatten(-1, (cfg.heads, cfg.head_dim)) for i in range(3)]
        return ops.attention(q, k, v, kv_len=kv_len).reshape(B, S, D)


class _MLP(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        self.gate_proj = Linear(cfg.hidden, cfg.ffn_hidden, False, dtype, device)
        self.up_proj = Linear(cfg.hidden, cfg.ffn_hidden, False, dtype, device)
        self.linear_fc2 = Linear(cfg.ffn_hidden, cfg.hidden, False, dtype, device)

    def forward(self, x, residual, gate, rows):
        h = ops.glu(packed_projection(x, (self.gate_proj, self.up_proj)), "gelu_erf")
        return self.linear_fc2(h, residual=residual, gate=gate, rows_per_group=rows)


class ErnieBlock(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        self.adaLN_sa_ln = RMSNorm(cfg.hidden, cfg.eps, dtype, device)
        self.self_attention = _SelfAttention(cfg, dtype, device)
        self.adaLN_mlp_ln = RMSNorm(cfg.hidden, cfg.eps, dtype, device)
        self.mlp = _MLP(cfg, dtype, device)

    def forward(self, x, mods, cos, sin, kv_len=None):
        S = x.shape[1]
        shift_a, scale_a, gate_a, shift_m, scale_m, gate_m = mods
        h = self.self_attention(self.adaLN_sa_ln(x, scale=scale_a, shift=shift_a), cos, sin, kv_len)
        x = self.self_attention.to_out[0](h, residual=x, gate=gate_a, rows_per_group=S)
        return self.mlp(self.adaLN_mlp_ln(x, scale=scale_m, shift=shift_m), x, gate_m, S)


class ErnieImage(nn.Module):
    """forward(img [B, S_img, C], text [B, T, text_dim], sigma [B] in (0, 1], hw, text_len) -> velocity [B, S_img, C]."""

    def __init__(self, cfg: ErnieConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert cfg.heads * cfg.head_dim == D and sum(cfg.axes_dim) == cfg.head_dim
        xe = nn.Module()
        xe.proj = Linear(cfg.in_channels, D, True, dtype, device)           # checkpoint weight [D, C, 1, 1] loads as [D, C]
        self.x_embedder = xe
        te = nn.Module()
        te.linear_1, te.linear_2 = Linear(D, D, True, dtype, device), Linear(D, D, True, dtype, device)
        self.time_embedding = te
        self.text_proj = Linear(cfg.text_dim, D, False, dtype, device)
        self.adaLN_modulation = nn.ModuleDict({"1": Linear(D, 6 * D, True, dtype, device)})
        self.layers = nn.ModuleList([ErnieBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        fn = nn.Module()
        fn.linear = Linear(D, 2 * D, True, dtype, device)
        self.final_norm = fn
        self.final_linear = Linear(D, cfg.in_channels, True, dtype, device)
        self.gradient_checkpointing = False

    @staticmethod
    def make_ids(h: int, w: int, n_txt: int, device=None) -> torch.Tensor:
        """Image tokens first at (0, row, col); text token i at (i, 0, 0) after them."""
        ids = torch.zeros(h * w + n_txt, 3, dtype=torch.float32, device=device)
        ids[:h * w, 1] = torch.arange(h, device=device, dtype=torch.float32)[:, None].expand(h, w).reshape(-1)
        ids[:h * w, 2] = torch.arange(w, device=device, dtype=torch.float32)[None, :].expand(h, w).reshape(-1)
        ids[h * w:, 0] = torch.arange(n_txt, device=device, dtype=torch.float32)
        return ids

    def forward(self, img, text, sigma, hw: Optional[Tuple[int, int]] = None, text_len: Optional[torch.Tensor] = None):
        cfg = self.cfg
        B, S_img, _ = img.shape
        T = text.shape[1]
        D = cfg.hidden
        if hw is None:
            side = int(round(S_img ** 0.5))
            hw = (side, S_img // side)
        dt = self.text_proj.weight.dtype
        cos, sin = ops.rope_table(self.make_ids(hw[0], hw[1], T, img.device), cfg.axes_dim, cfg.theta)
        e = timestep_embedding(sigma, D, time_factor=1000.0, cos_first=False).to(dt)
        temb = self.time_embedding.linear_2(self.time_embedding.linear_1(e, act="silu"))
        m = self.adaLN_modulation["1"](ops.activation(temb, "silu"))
        mods = [m[:, i * D:(i + 1) * D] for i in range(6)]
        x = torch.cat((self.x_embedder.proj(img.to(dt)), self.text_proj(text.to(dt))), dim=1)
        kv_len = (S_img + text_len).to(torch.int32) if text_len is not None else None
        for blk in self.layers:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(blk, x, mods, cos, sin, kv_len, use_reentrant=False, preserve_rng_state=False)
            else:
                x = blk(x, mods, cos, sin, kv_len)
        f = self.final_norm.linear(ops.activation(temb, "silu"))
        y = ops.norm_modulate(x[:, :S_img], scale=f[:, :D], shift=f[:, D:], eps=cfg.eps)
        return self.final_linear(y)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)


def ernie_sigmas(steps: int = 50, shift: float = 3.0):
    from ..sampling.flow_match import shifted_sigmas
    return shifted_sigmas(steps, shift)


def ernie_lora_targets(depth: int):
    out = []
    for i in range(depth):
        b = f"layers.{i}."
        out += [b + "self_attention." + n for n in ("to_q", "to_k", "to_v", "to_out.0")] + [b + "mlp." + n for n in ("gate_proj", "up_proj", "linear_fc2")]
    return out
