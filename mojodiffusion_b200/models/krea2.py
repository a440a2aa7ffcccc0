"""Krea-2 single-stream MMDiT: text tokens (fused from twelve stacked Qwen3-VL hidden states) and 2 x 2-patchified image
latents run as ONE sequence through 28 identical blocks of width 6144.

* every RMSNorm is fp32-internal with weight ``1 + scale`` (``scale`` starts at zero) and eps 1e-5;
* attention: 48 query heads over 12 key / value heads (each shared by four query heads) of 128, QK-RMSNorm per head,
  interleaved-pair rotary embedding from a three-axis table (axes 32 / 48 / 48 of the head = global, row, column; base
  1e3; angles reduced in float64), and a sigmoid gate: ``wo(attention * sigmoid(gate(x)))``; no biases;
* SwiGLU feed-forward 16 384 wide (``int(2 * features / 3) * multiplier`` rounded up to 128);
* modulation: ``tproj(t)`` gives one [6 * features] vector shared by ALL blocks; each block adds its own learned ``mod.lin``
  and splits it into (scale, shift, gate) for the attention branch and for the feed-forward branch;
* text path: two blocks attending over the 12 LAYERS of every token, a Linear(12 -> 1) collapse of the layer axis, two
  blocks attending over the tokens (no rotary, 20 heads of 128, plain residuals), then RMSNorm + a two-layer GELU-tanh MLP
  up to the model width;
* timestep: cos-first sinusoid of ``1000 t`` (256 wide) -> Linear -> GELU-tanh -> Linear = ``t``; blocks read
  ``tproj(t)``, the last layer reads ``t`` itself through a learned two-row (scale, shift) offset.

Behaviour: serenitymojo/models/dit/krea2_dit.mojo:10-135 (rotary table), :329-470 (norm, SwiGLU), :477-550 (modulations),
:626-800 (attention), :812-867 (block), :869-993 (embedders and heads), :1075-1246 (text fusion), :1304-1520 (forward);
serenitymojo/pipeline/krea2_pipeline.mojo:153-200 (positions, patchify), :225-262 (sampling loop). Parameter names are the
checkpoint's own (``blocks.N.attn.wq.weight``, ``blocks.N.mod.lin``, ``txtfusion.layerwise_blocks.N...``, ``last.linear``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import native
from .layers import Linear, init_module_weights, packed_projection, timestep_embedding


@dataclass
class Krea2Config:
    features: int = 6144
    tdim: int = 256
    txtdim: int = 2560
    heads: int = 48
    kvheads: int = 12
    multiplier: int = 4
    layers: int = 28
    patch: int = 2
    channels: int = 16
    txtheads: int = 20
    txtkvheads: int = 20
    txtlayers: int = 12
    theta: float = 1.0e3
    eps: float = 1e-5
    name: str = "krea-2"

    @property
    def head_dim(self) -> int:
        return self.features // self.heads

    @property
    def rope_axes(self) -> Tuple[int, int, int]:
        unit = self.head_dim // 16
        return (self.head_dim - 12 * unit, 6 * unit, 6 * unit)

    @property
    def patch_dim(self) -> int:
        return self.channels * self.patch * self.patch

    @property
    def in_channels(self) -> int:
        """Width of one packed image token (the name the shared sampler and adapters read)."""
        return self.patch_dim


def tiny_krea2_config() -> Krea2Config:
    return Krea2Config(features=128, tdim=32, txtdim=64, heads=4, kvheads=2, multiplier=2, layers=2, channels=4, txtheads=2,
                       txtkvheads=2, txtlayers=3, name="tiny-krea2")


def swiglu_width(features: int, multiplier: int) -> int:
    return 128 * ((int(2 * features // 3) * multiplier + 127) // 128)


def krea2_rope_table(pos: torch.Tensor, axes: Tuple[int, ...], theta: float):
    """cos / sin [L, sum(axes) / 2] (fp32) for positions [L, len(axes)]: axis a owns ``axes[a] / 2`` consecutive frequency
    slots with omega_i = theta ** (-2 i / axes[a]); the angle is reduced modulo 2 pi in float64 before the fp32 trig."""
    p = pos.detach().double().cpu()
    cols = []
    for a, d in enumerate(axes):
        omega = 1.0 / (float(theta) ** (torch.arange(0, d, 2, dtype=torch.float64) / d))
        cols.append(p[:, a:a + 1] * omega[None])
    ang = torch.cat(cols, -1)
    ang = ang - torch.floor(ang / (2 * math.pi) + 0.5) * (2 * math.pi)
    return ang.float().cos().to(pos.device), ang.float().sin().to(pos.device)


def krea2_positions(text_len: int, gh: int, gw: int, device=None) -> torch.Tensor:
    """[text_len + gh * gw, 3] fp32: text rows all zero, image token (r, c) -> (0, r, c) in row-major order."""
    pos = torch.zeros(text_len + gh * gw, 3, dtype=torch.float32, device=device)
    pos[text_len:, 1] = torch.arange(gh, dtype=torch.float32, device=device)[:, None].expand(gh, gw).reshape(-1)
    pos[text_len:, 2] = torch.arange(gw, dtype=torch.float32, device=device)[None, :].expand(gh, gw).reshape(-1)
    return pos


def patchify(latent: torch.Tensor, p: int = 2) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H / p) (W / p), C p p] with per-token feature order (channel, row in patch, column in patch)."""
    B, C, H, W = latent.shape
    return latent.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // p) * (W // p), C * p * p)


def unpatchify(tokens: torch.Tensor, gh: int, gw: int, p: int = 2) -> torch.Tensor:
    B, _, F = tokens.shape
    C = F // (p * p)
    return tokens.reshape(B, gh, gw, C, p, p).permute(0, 3, 1, 4, 2, 5).reshape(B, C, gh * p, gw * p)


def _rope_pairs(x, cos, sin):
    c, s = cos[None, :, None].to(x.dtype), sin[None, :, None].to(x.dtype)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)


class ScaleNorm(nn.Module):
    """RMSNorm whose weight is ``1 + scale`` (serenitymojo/models/dit/krea2_dit.mojo:329-343)."""

    def __init__(self, dim: int, eps: float, dtype, device):
        super().__init__()
        self.eps = eps
        self.scale = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))

    def forward(self, x, scale=None, shift=None, rows_per_group=None):
        return ops.norm_modulate(x, weight=(self.scale.float() + 1.0).to(x.dtype), scale=scale, shift=shift, rows_per_group=rows_per_group,
                                 eps=self.eps, rms=True)


class _QKNorm(nn.Module):
    def __init__(self, dim, eps, dtype, device):
        super().__init__()
        self.qnorm = ScaleNorm(dim, eps, dtype, device)
        self.knorm = ScaleNorm(dim, eps, dtype, device)


class Krea2Attention(nn.Module):
    def __init__(self, width: int, heads: int, kvheads: int, eps: float, dtype, device):
        super().__init__()
        self.heads, self.kvheads, self.head_dim = heads, kvheads, width // heads
        kv = kvheads * self.head_dim
        self.wq = Linear(width, width, False, dtype, device)
        self.wk = Linear(width, kv, False, dtype, device)
        self.wv = Linear(width, kv, False, dtype, device)
        self.gate = Linear(width, width, False, dtype, device)
        self.wo = Linear(width, width, False, dtype, device)
        self.qknorm = _QKNorm(self.head_dim, eps, dtype, device)

    def _forward_packed(self, x, rope):
        """Inference on the device kernels: q | k | v land in one buffer (each GEMM stores into its column range), the
        per-head norm + rotary kernel runs in place on the query heads and on the key heads (two half-ranges per launch),
        attention writes next to the gate projection and one gated-unit kernel forms ``sigmoid(gate) * attention``."""
        H, KV, Dh = self.heads, self.kvheads, self.head_dim
        B, S, D = x.shape
        qkv = packed_projection(x, (self.wq, self.wk, self.wv))
        wq = (self.qknorm.qnorm.scale.float() + 1.0).to(x.dtype)
        wk = (self.qknorm.knorm.scale.float() + 1.0).to(x.dtype)
        cos, sin = rope if rope is not None else (None, None)
        eps = self.qknorm.qnorm.eps
        ops.qk_norm_rope(qkv, H // 2, Dh, wq, wq, cos, sin, eps, True, q_off=0, k_off=(H // 2) * Dh)
        ops.qk_norm_rope(qkv, KV // 2, Dh, wk, wk, cos, sin, eps, True, q_off=D, k_off=D + (KV // 2) * Dh)
        q = qkv[..., :D].unflatten(-1, (H, Dh))
        k = qkv[..., D:D + KV * Dh].unflatten(-1, (KV, Dh))
        v = qkv[..., D + KV * Dh:].unflatten(-1, (KV, Dh))
        if KV != H:
            k, v = k.repeat_interleave(H // KV, 2), v.repeat_interleave(H // KV, 2)
        pair = torch.empty(B, S, 2 * D, dtype=x.dtype, device=x.device)
        self.gate(x, out=pair[..., :D])
        ops.attention(q, k, v, out=pair[..., D:].unflatten(-1, (H, Dh)))
        return self.wo(ops.glu(pair, "sigmoid"))

    def forward(self, x, rope=None):
        H, KV, Dh = self.heads, self.kvheads, self.head_dim
        if (native.use_native(x) and not torch.is_grad_enabled() and Dh in (64, 128) and H % 2 == 0 and KV % 2 == 0
                and x.dim() == 3):
            return self._forward_packed(x, rope)
        q = self.qknorm.qnorm(self.wq(x).unflatten(-1, (H, Dh)))
        k = self.qknorm.knorm(self.wk(x).unflatten(-1, (KV, Dh)))
        v = self.wv(x).unflatten(-1, (KV, Dh))
        if rope is not None:
            q, k = _rope_pairs(q, *rope), _rope_pairs(k, *rope)
        if KV != H:
            k, v = k.repeat_interleave(H // KV, 2), v.repeat_interleave(H // KV, 2)
        o = ops.attention(q, k, v).flatten(-2)
        return self.wo(o * torch.sigmoid(self.gate(x)))


class _SwiGLU(nn.Module):
    def __init__(self, width: int, multiplier: int, dtype, device):
        super().__init__()
        inner = swiglu_width(width, multiplier)
        self.gate = Linear(width, inner, False, dtype, device)
        self.up = Linear(width, inner, False, dtype, device)
        self.down = Linear(inner, width, False, dtype, device)

    def forward(self, x):
        if native.use_native(x) and not torch.is_grad_enabled():
            return self.down(ops.glu(packed_projection(x, (self.gate, self.up)), "silu"))
        return self.down(self.gate(x, act="silu") * self.up(x))


class _Mod(nn.Module):
    def __init__(self, shape, dtype, device):
        super().__init__()
        self.lin = nn.Parameter(torch.zeros(*shape, dtype=dtype, device=device))


class Krea2Block(nn.Module):
    def __init__(self, cfg: Krea2Config, dtype, device):
        super().__init__()
        D = cfg.features
        self.mod = _Mod((6 * D,), dtype, device)
        self.prenorm = ScaleNorm(D, cfg.eps, dtype, device)
        self.postnorm = ScaleNorm(D, cfg.eps, dtype, device)
        self.attn = Krea2Attention(D, cfg.heads, cfg.kvheads, cfg.eps, dtype, device)
        self.mlp = _SwiGLU(D, cfg.multiplier, dtype, device)

    def forward(self, x, vec, rope):
        D, S = x.shape[-1], x.shape[1]
        m = vec + self.mod.lin                                                     # [B, 6D]
        h = self.prenorm(x, scale=m[:, 0:D], shift=m[:, D:2 * D])
        x = ops.gate_residual(x, self.attn(h, rope), m[:, 2 * D:3 * D], S)
        h = self.postnorm(x, scale=m[:, 3 * D:4 * D], shift=m[:, 4 * D:5 * D])
        return ops.gate_residual(x, self.mlp(h), m[:, 5 * D:6 * D], S)


class TextFusionBlock(nn.Module):
    def __init__(self, cfg: Krea2Config, dtype, device):
        super().__init__()
        D = cfg.txtdim
        self.prenorm = ScaleNorm(D, cfg.eps, dtype, device)
        self.postnorm = ScaleNorm(D, cfg.eps, dtype, device)
        self.attn = Krea2Attention(D, cfg.txtheads, cfg.txtkvheads, cfg.eps, dtype, device)
        self.mlp = _SwiGLU(D, cfg.multiplier, dtype, device)

    def forward(self, x):
        x = x + self.attn(self.prenorm(x))
        return x + self.mlp(self.postnorm(x))


class TextFusion(nn.Module):
    """[B, Lt, layers, d] -> [B, Lt, d] (serenitymojo/models/dit/krea2_dit.mojo:1193-1246)."""

    def __init__(self, cfg: Krea2Config, dtype, device):
        super().__init__()
        self.layerwise_blocks = nn.ModuleList([TextFusionBlock(cfg, dtype, device) for _ in range(2)])
        self.projector = Linear(cfg.txtlayers, 1, False, dtype, device)
        self.refiner_blocks = nn.ModuleList([TextFusionBlock(cfg, dtype, device) for _ in range(2)])

    def forward(self, context):
        B, L, n, d = context.shape
        x = context.reshape(B * L, n, d)
        for blk in self.layerwise_blocks:
            x = blk(x)
        x = self.projector(x.transpose(1, 2).contiguous()).reshape(B, L, d)
        for blk in self.refiner_blocks:
            x = blk(x)
        return x


class _Last(nn.Module):
    def __init__(self, cfg: Krea2Config, dtype, device):
        super().__init__()
        self.norm = ScaleNorm(cfg.features, cfg.eps, dtype, device)
        self.modulation = _Mod((2, cfg.features), dtype, device)
        self.linear = Linear(cfg.features, cfg.patch_dim, True, dtype, device)


class Krea2DiT(nn.Module):
    """forward(img [B, N, channels * patch^2], context [B, Lt, txtlayers, txtdim], t [B], pos [Lt + N, 3]) ->
    velocity on the image tokens [B, N, channels * patch^2]. Every sample of a batch has the same (unpadded) text length,
    which is how the reference samples: a prompt runs at its natural token count."""

    def __init__(self, cfg: Krea2Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.features
        self.first = Linear(cfg.patch_dim, D, True, dtype, device)
        self.tmlp = nn.ModuleDict({"0": Linear(cfg.tdim, D, True, dtype, device), "2": Linear(D, D, True, dtype, device)})
        self.tproj = nn.ModuleDict({"1": Linear(D, 6 * D, True, dtype, device)})
        self.txtfusion = TextFusion(cfg, dtype, device)
        self.txtmlp = nn.ModuleDict({"0": ScaleNorm(cfg.txtdim, cfg.eps, dtype, device),
                                     "1": Linear(cfg.txtdim, D, True, dtype, device), "3": Linear(D, D, True, dtype, device)})
        self.blocks = nn.ModuleList([Krea2Block(cfg, dtype, device) for _ in range(cfg.layers)])
        self.last = _Last(cfg, dtype, device)
        self.gradient_checkpointing = False

    def time_vectors(self, t: torch.Tensor):
        dt = self.first.weight.dtype
        tv = self.tmlp["2"](self.tmlp["0"](timestep_embedding(t, self.cfg.tdim).to(dt), act="gelu_tanh"))
        return tv, self.tproj["1"](ops.activation(tv, "gelu_tanh"))

    def text_tokens(self, context: torch.Tensor) -> torch.Tensor:
        dt = self.first.weight.dtype
        c = self.txtfusion(context.to(dt))
        return self.txtmlp["3"](self.txtmlp["1"](self.txtmlp["0"](c), act="gelu_tanh"))

    def forward(self, img, context, t, pos):
        cfg = self.cfg
        dt = self.first.weight.dtype
        tv, vec = self.time_vectors(t)
        txt = self.text_tokens(context)
        Lt = txt.shape[1]
        x = torch.cat((txt, self.first(img.to(dt))), 1)
        rope = krea2_rope_table(pos.to(x.device), cfg.rope_axes, cfg.theta)
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.blocks:
            if ckpt:
                x = torch.utils.checkpoint.checkpoint(blk, x, vec, rope, use_reentrant=False, preserve_rng_state=False)
            else:
                x = blk(x, vec, rope)
        m = tv[:, None, :] + self.last.modulation.lin[None]                        # [B, 2, D]: scale, shift
        h = self.last.norm(x[:, Lt:], scale=m[:, 0], shift=m[:, 1])
        return self.last.linear(h)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        init_module_weights(self, seed, std)
        with torch.no_grad():
            for n, p in self.named_parameters():
                if n.endswith(".scale"):                                           # the norm weight is 1 + scale
                    p.zero_()
        return self


@torch.no_grad()
def krea2_sample(model: Krea2DiT, context: torch.Tensor, uncond_context: Optional[torch.Tensor], height: int, width: int,
                 steps: int = 20, cfg_scale: float = 4.5, seed: int = 0, latent: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Euler integration of the flow from t = 1 to 0 on an fp32 latent [1, channels, height / 8, width / 8]; the model is fed
    the latent rounded to its dtype; with an unconditional context the velocity is ``v_c + cfg_scale * (v_c - v_u)``
    (serenitymojo/pipeline/krea2_pipeline.mojo:225-262)."""
    from ..sampling.family_schedules import krea2_cfg, krea2_packed_seq_len, krea2_timesteps
    cfg = model.cfg
    dev, dt = model.first.weight.device, model.first.weight.dtype
    lh, lw = height // 8, width // 8
    gh, gw = lh // cfg.patch, lw // cfg.patch
    if latent is None:
        latent = ops.randn((1, cfg.channels, lh, lw), seed, 0, torch.float32, dev)
    latent = latent.float()
    ts = krea2_timesteps(krea2_packed_seq_len(height, width), steps)
    pos_c = krea2_positions(context.shape[1], gh, gw, dev)
    pos_u = krea2_positions(uncond_context.shape[1], gh, gw, dev) if uncond_context is not None else None
    for i in range(steps):
        t = torch.tensor([ts[i]], dtype=torch.float32, device=dev)
        tok = patchify(latent, cfg.patch).to(dt)
        v = model(tok, context, t, pos_c)
        if uncond_context is not None:
            v = krea2_cfg(v, model(tok, uncond_context, t, pos_u), cfg_scale)
        latent = latent + (ts[i + 1] - ts[i]) * unpatchify(v.float(), gh, gw, cfg.patch)
    return latent
