"""Boogu-Image DiT (Lumina-2 lineage): width 3360, 28 query / 7 key-value heads of 120, SwiGLU 13 568 wide, no biases inside
the blocks; 2 context-refiner blocks on the caption, 2 noise-refiner blocks on the image, 8 DOUBLE-stream blocks, then 32
single-stream blocks over [caption, image].

* conditioning: cos-first sinusoid of ``1000 t`` (256) -> Linear -> SiLU -> Linear = temb (1024); caption = RMSNorm(4096) +
  Linear; image tokens = Linear of 2 x 2 patches in (row, column, channel) order of a 16-channel latent;
* "norm-zero" modulation: ``Linear(silu(temb))`` gives four chunks (scale_msa, gate_msa, scale_mlp, gate_mlp); the output is
  ``RMSNorm(x) * (1 + scale_msa)``. A modulated block computes
  ``x += tanh(gate_msa) * norm2(attn(.))``, ``x += tanh(gate_mlp) * ffn_norm2(ffn(ffn_norm1(x) * (1 + scale_mlp)))``;
  an unmodulated block (context refiner) has plain RMSNorms and plain residuals; every RMSNorm has eps 1e-5;
* attention: per-head QK-RMSNorm, interleaved-pair rotation with three axes of 40 (theta 1e4), key / value heads repeated
  four times. Caption token i sits at (i, i, i); image token (r, c) at (caption length, r, c);
* double-stream block: five norm-zero modulations (img_norm1 / 2 / 3, instruct_norm1 / 2). Joint attention with per-stream
  q / k / v projections over [caption, image], per-stream output projections, then a shared ``to_out``; the image stream also
  has a self-attention fed by img_norm3 whose chunk 1 gates it; the feed-forward input is
  ``(1 + scale_mlp) * norm2_out + shift`` where scale_mlp comes from norm1 and shift is chunk 1 of norm2;
* output: LayerNorm without affine (eps 1e-6) times ``1 + Linear(silu(temb))``, Linear to 64, image rows unpatchified.

Behaviour: serenitymojo/models/dit/boogu_dit.mojo:10-46 (embedders), :191-284 (positions), :286-352 (single block), :540-610
(double block), :963-1000 (output), :1202-1240 (forward order). Parameter names are the checkpoint's.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, timestep_embedding


@dataclass
class BooguConfig:
    hidden: int = 3360
    heads: int = 28
    kv_heads: int = 7
    head_dim: int = 120
    ffn_inner: int = 13568
    in_channels: int = 16
    patch: int = 2
    instruction_dim: int = 4096
    time_embed_dim: int = 1024
    axes_dim: Tuple[int, int, int] = (40, 40, 40)
    theta: float = 1.0e4
    n_context_refiner: int = 2
    n_noise_refiner: int = 2
    n_double: int = 8
    n_single: int = 32
    eps: float = 1e-5
    name: str = "boogu-image-0.1"

    @property
    def patch_dim(self):
        return self.patch * self.patch * self.in_channels


def tiny_boogu_config() -> BooguConfig:
    return BooguConfig(hidden=96, heads=4, kv_heads=2, head_dim=24, ffn_inner=160, in_channels=4, instruction_dim=40, time_embed_dim=32,
                       axes_dim=(8, 8, 8), n_context_refiner=1, n_noise_refiner=1, n_double=2, n_single=2, name="tiny-boogu")


def boogu_patchify(latent: torch.Tensor, p: int = 2) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H / p)(W / p), p p C] with the channel fastest."""
    B, C, H, W = latent.shape
    return latent.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 3, 5, 1).reshape(B, (H // p) * (W // p), p * p * C)


def boogu_unpatchify(tokens: torch.Tensor, h: int, w: int, p: int = 2) -> torch.Tensor:
    B, _, Fd = tokens.shape
    C = Fd // (p * p)
    return tokens.reshape(B, h, w, p, p, C).permute(0, 5, 1, 3, 2, 4).reshape(B, C, h * p, w * p)


def boogu_positions(cap_len: int, h: int, w: int, device=None) -> torch.Tensor:
    pos = torch.zeros(cap_len + h * w, 3, dtype=torch.float32, device=device)
    pos[:cap_len] = torch.arange(cap_len, dtype=torch.float32, device=device)[:, None]
    pos[cap_len:, 0] = float(cap_len)
    pos[cap_len:, 1] = torch.arange(h, dtype=torch.float32, device=device).repeat_interleave(w)
    pos[cap_len:, 2] = torch.arange(w, dtype=torch.float32, device=device).repeat(h)
    return pos


def _rope_pairs(x, cos, sin):
    c, s = cos[None, :, None].to(x.dtype), sin[None, :, None].to(x.dtype)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)


def _attend(q, k, v, rep: int):
    """[B, S, H, Dh] x [B, S, KV, Dh]: the tcgen05 kernel for head widths 64 / 128, library attention otherwise."""
    k, v = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
    if q.shape[-1] in (64, 128) or not q.is_cuda:
        return ops.attention(q, k, v)
    return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)


class _NormZero(nn.Module):
    def __init__(self, c: BooguConfig, dtype, device):
        super().__init__()
        self.linear = Linear(c.time_embed_dim, 4 * c.hidden, True, dtype, device)
        self.norm = RMSNorm(c.hidden, c.eps, dtype, device)

    def forward(self, x, temb_silu):
        D = x.shape[-1]
        e = self.linear(temb_silu)
        return self.norm(x, scale=e[:, :D]), e[:, D:2 * D], e[:, 2 * D:3 * D], e[:, 3 * D:]


class _SelfAttn(nn.Module):
    def __init__(self, c: BooguConfig, dtype, device):
        super().__init__()
        self.c = c
        D, KVD = c.hidden, c.kv_heads * c.head_dim
        self.to_q = Linear(D, D, False, dtype, device)
        self.to_k = Linear(D, KVD, False, dtype, device)
        self.to_v = Linear(D, KVD, False, dtype, device)
        self.to_out = nn.ModuleList([Linear(D, D, False, dtype, device)])
        self.norm_q, self.norm_k = RMSNorm(c.head_dim, c.eps, dtype, device), RMSNorm(c.head_dim, c.eps, dtype, device)

    def forward(self, x, cos, sin):
        c = self.c
        B, S, D = x.shape
        q = _rope_pairs(self.norm_q(self.to_q(x).unflatten(-1, (c.heads, c.head_dim))), cos, sin)
        k = _rope_pairs(self.norm_k(self.to_k(x).unflatten(-1, (c.kv_heads, c.head_dim))), cos, sin)
        v = self.to_v(x).unflatten(-1, (c.kv_heads, c.head_dim))
        return self.to_out[0](_attend(q, k, v, c.heads // c.kv_heads).reshape(B, S, D))


class _FeedForward(nn.Module):
    def __init__(self, c: BooguConfig, dtype, device):
        super().__init__()
        self.linear_1 = Linear(c.hidden, c.ffn_inner, False, dtype, device)
        self.linear_2 = Linear(c.ffn_inner, c.hidden, False, dtype, device)
        self.linear_3 = Linear(c.hidden, c.ffn_inner, False, dtype, device)

    def forward(self, x):
        return self.linear_2(self.linear_1(x, act="silu") * self.linear_3(x))


class BooguBlock(nn.Module):
    def __init__(self, c: BooguConfig, modulation: bool, dtype, device):
        super().__init__()
        self.modulation = modulation
        self.norm1 = _NormZero(c, dtype, device) if modulation else RMSNorm(c.hidden, c.eps, dtype, device)
        self.attn = _SelfAttn(c, dtype, device)
        self.norm2 = RMSNorm(c.hidden, c.eps, dtype, device)
        self.ffn_norm1 = RMSNorm(c.hidden, c.eps, dtype, device)
        self.ffn_norm2 = RMSNorm(c.hidden, c.eps, dtype, device)
        self.feed_forward = _FeedForward(c, dtype, device)

    def forward(self, x, temb_silu, cos, sin):
        S = x.shape[1]
        if not self.modulation:
            x = x + self.norm2(self.attn(self.norm1(x), cos, sin))
            return x + self.ffn_norm2(self.feed_forward(self.ffn_norm1(x)))
        h, gate_msa, scale_mlp, gate_mlp = self.norm1(x, temb_silu)
        x = ops.gate_residual(x, self.norm2(self.attn(h, cos, sin)), gate_msa, S, tanh_gate=True)
        h = self.feed_forward(self.ffn_norm1(x, scale=scale_mlp))
        return ops.gate_residual(x, self.ffn_norm2(h), gate_mlp, S, tanh_gate=True)


class _Processor(nn.Module):
    def __init__(self, c: BooguConfig, dtype, device):
        super().__init__()
        D, KVD = c.hidden, c.kv_heads * c.head_dim
        for s in ("img", "instruct"):
            setattr(self, s + "_to_q", Linear(D, D, False, dtype, device))
            setattr(self, s + "_to_k", Linear(D, KVD, False, dtype, device))
            setattr(self, s + "_to_v", Linear(D, KVD, False, dtype, device))
            setattr(self, s + "_out", Linear(D, D, False, dtype, device))


class _JointAttn(nn.Module):
    def __init__(self, c: BooguConfig, dtype, device):
        super().__init__()
        self.c = c
        self.processor = _Processor(c, dtype, device)
        self.to_out = nn.ModuleList([Linear(c.hidden, c.hidden, False, dtype, device)])
        self.norm_q, self.norm_k = RMSNorm(c.head_dim, c.eps, dtype, device), RMSNorm(c.head_dim, c.eps, dtype, device)

    def forward(self, ins, img, cos, sin):
        c, p = self.c, self.processor
        B, Li, D = ins.shape
        cat = lambda a, b: torch.cat((a, b), 1)
        q = cat(p.instruct_to_q(ins), p.img_to_q(img)).unflatten(-1, (c.heads, c.head_dim))
        k = cat(p.instruct_to_k(ins), p.img_to_k(img)).unflatten(-1, (c.kv_heads, c.head_dim))
        v = cat(p.instruct_to_v(ins), p.img_to_v(img)).unflatten(-1, (c.kv_heads, c.head_dim))
        q, k = _rope_pairs(self.norm_q(q), cos, sin), _rope_pairs(self.norm_k(k), cos, sin)
        o = _attend(q, k, v, c.heads // c.kv_heads).flatten(-2)
        o = self.to_out[0](cat(p.instruct_out(o[:, :Li]), p.img_out(o[:, Li:])))
        return o[:, :Li], o[:, Li:]


class BooguDoubleBlock(nn.Module):
    def __init__(self, c: BooguConfig, dtype, device):
        super().__init__()
        for n in ("img_norm1", "img_norm2", "img_norm3", "instruct_norm1", "instruct_norm2"):
            setattr(self, n, _NormZero(c, dtype, device))
        for n in ("img_attn_norm", "img_self_attn_norm", "img_ffn_norm1", "img_ffn_norm2", "instruct_attn_norm", "instruct_ffn_norm1",
                  "instruct_ffn_norm2"):
            setattr(self, n, RMSNorm(c.hidden, c.eps, dtype, device))
        self.img_instruct_attn = _JointAttn(c, dtype, device)
        self.img_self_attn = _SelfAttn(c, dtype, device)
        self.img_feed_forward = _FeedForward(c, dtype, device)
        self.instruct_feed_forward = _FeedForward(c, dtype, device)

    def forward(self, ins, img, temb_silu, cos, sin):
        Li, Lm = ins.shape[1], img.shape[1]
        i1, i_gate_msa, i_scale_mlp, i_gate_mlp = self.img_norm1(img, temb_silu)
        i2, i_shift_mlp, _, _ = self.img_norm2(img, temb_silu)
        i3, i_gate_self, _, _ = self.img_norm3(img, temb_silu)
        t1, t_gate_msa, t_scale_mlp, t_gate_mlp = self.instruct_norm1(ins, temb_silu)
        t2, t_shift_mlp, _, _ = self.instruct_norm2(ins, temb_silu)
        a_ins, a_img = self.img_instruct_attn(t1, i1, cos, sin)
        a_self = self.img_self_attn(i3, cos[Li:], sin[Li:])
        img = ops.gate_residual(img, self.img_attn_norm(a_img), i_gate_msa, Lm, tanh_gate=True)
        img = ops.gate_residual(img, self.img_self_attn_norm(a_self), i_gate_self, Lm, tanh_gate=True)
        h = (1 + i_scale_mlp[:, None]) * i2 + i_shift_mlp[:, None]
        img = ops.gate_residual(img, self.img_ffn_norm2(self.img_feed_forward(self.img_ffn_norm1(h))), i_gate_mlp, Lm, tanh_gate=True)
        ins = ops.gate_residual(ins, self.instruct_attn_norm(a_ins), t_gate_msa, Li, tanh_gate=True)
        h = (1 + t_scale_mlp[:, None]) * t2 + t_shift_mlp[:, None]
        ins = ops.gate_residual(ins, self.instruct_ffn_norm2(self.instruct_feed_forward(self.instruct_ffn_norm1(h))), t_gate_mlp, Li, tanh_gate=True)
        return ins, img


class _TimeCaption(nn.Module):
    def __init__(self, c: BooguConfig, dtype, device):
        super().__init__()
        te = nn.Module()
        te.linear_1 = Linear(256, c.time_embed_dim, True, dtype, device)
        te.linear_2 = Linear(c.time_embed_dim, c.time_embed_dim, True, dtype, device)
        self.timestep_embedder = te
        self.caption_embedder = nn.ModuleDict({"0": RMSNorm(c.instruction_dim, c.eps, dtype, device),
                                               "1": Linear(c.instruction_dim, c.hidden, True, dtype, device)})


class _NormOut(nn.Module):
    def __init__(self, c: BooguConfig, dtype, device):
        super().__init__()
        self.linear_1 = Linear(c.time_embed_dim, c.hidden, True, dtype, device)
        self.linear_2 = Linear(c.hidden, c.patch_dim, True, dtype, device)


class BooguDiT(nn.Module):
    """forward(latent [B, 16, H, W], instruction [B, L, 4096], t [B] in [0, 1]) -> velocity [B, 16, H, W]."""

    def __init__(self, cfg: BooguConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        assert sum(cfg.axes_dim) == cfg.head_dim and cfg.heads * cfg.head_dim == cfg.hidden
        self.x_embedder = Linear(cfg.patch_dim, cfg.hidden, True, dtype, device)
        self.time_caption_embed = _TimeCaption(cfg, dtype, device)
        self.context_refiner = nn.ModuleList([BooguBlock(cfg, False, dtype, device) for _ in range(cfg.n_context_refiner)])
        self.noise_refiner = nn.ModuleList([BooguBlock(cfg, True, dtype, device) for _ in range(cfg.n_noise_refiner)])
        self.double_stream_layers = nn.ModuleList([BooguDoubleBlock(cfg, dtype, device) for _ in range(cfg.n_double)])
        self.single_stream_layers = nn.ModuleList([BooguBlock(cfg, True, dtype, device) for _ in range(cfg.n_single)])
        self.norm_out = _NormOut(cfg, dtype, device)

    def forward(self, latent, instruction, t):
        c, tc = self.cfg, self.time_caption_embed
        B, _, H, W = latent.shape
        h, w = H // c.patch, W // c.patch
        dt = self.x_embedder.weight.dtype
        te = tc.timestep_embedder
        temb = te.linear_2(te.linear_1(timestep_embedding(t, 256).to(dt), act="silu"))
        temb_silu = ops.activation(temb, "silu")
        cap = tc.caption_embedder["1"](tc.caption_embedder["0"](instruction.to(dt)))
        Lc = cap.shape[1]
        cos, sin = ops.rope_table(boogu_positions(Lc, h, w, latent.device), c.axes_dim, c.theta)
        for blk in self.context_refiner:
            cap = blk(cap, None, cos[:Lc], sin[:Lc])
        x = self.x_embedder(boogu_patchify(latent.to(dt), c.patch))
        for blk in self.noise_refiner:
            x = blk(x, temb_silu, cos[Lc:], sin[Lc:])
        for blk in self.double_stream_layers:
            cap, x = blk(cap, x, temb_silu, cos, sin)
        joint = torch.cat((cap, x), 1)
        for blk in self.single_stream_layers:
            joint = blk(joint, temb_silu, cos, sin)
        y = ops.norm_modulate(joint[:, Lc:], scale=self.norm_out.linear_1(temb_silu), eps=1e-6, rms=False)
        return boogu_unpatchify(self.norm_out.linear_2(y), h, w, c.patch)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
