"""Chroma-shaped MMDiT: the FLUX.1 block stack (19 double + 38 single, hidden 3072, 24 heads x 128, RoPE (16,56,56))
with every per-block modulation linear removed. One small "distilled guidance layer" maps, once per step, a table of
344 rows [sinusoid(t*1000, 16) | sinusoid(guidance=0, 16) | sinusoid(row*1000, 32)] through
``in_proj -> 5 x (RMSNorm -> linear -> SiLU -> linear, residual) -> out_proj`` to 344 vectors of width 3072; row r is a
shift, scale or gate: single block i uses rows 3i..3i+2, double block i uses rows 114+6i.. (image) and 228+6i.. (text),
the output norm the last two. No pooled-vector or guidance embedder; text is T5 only.

Parameter names follow the diffusers checkpoint: ``transformer_blocks.{i}.attn.{to_q,to_k,to_v,add_q_proj,add_k_proj,
add_v_proj,to_out.0,to_add_out,norm_q,norm_k,norm_added_q,norm_added_k}``, ``ff.net.{0.proj,2}``, ``ff_context.net.*``,
``single_transformer_blocks.{i}.{attn.to_q,attn.to_k,attn.to_v,attn.norm_q,attn.norm_k,proj_mlp,proj_out}``,
``distilled_guidance_layer.{in_proj,layers.{j}.linear_{1,2},norms.{j},out_proj}``, ``x_embedder``, ``context_embedder``,
``proj_out``.

Facts: serenitymojo/models/dit/chroma_dit.mojo:238-295 (approximator input and layers), :325-360 and :436-450 (row
layout), :507-536 (sinusoids); serenitymojo/models/dit/chroma_contract.mojo:73-92 (sizes)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, packed_projection
from .mmdit import MMDiT


@dataclass
class ChromaConfig:
    in_channels: int = 64
    context_dim: int = 4096
    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    depth_double: int = 19
    depth_single: int = 38
    mlp_hidden: int = 12288
    axes_dim: Tuple[int, ...] = (16, 56, 56)
    theta: float = 10000.0
    approx_in: int = 64
    approx_hidden: int = 5120
    approx_layers: int = 5
    name: str = "chroma1-hd"

    @property
    def mod_rows(self) -> int:
        return 3 * self.depth_single + 12 * self.depth_double + 2


def chroma_config() -> ChromaConfig:
    return ChromaConfig()


def tiny_chroma_config() -> ChromaConfig:
    return ChromaConfig(in_channels=32, context_dim=96, hidden=256, heads=4, head_dim=64, depth_double=2, depth_single=2,
                        mlp_hidden=512, axes_dim=(16, 24, 24), approx_in=32, approx_hidden=128, approx_layers=2,
                        name="tiny-chroma")


def _sinusoid(t: torch.Tensor, dim: int) -> torch.Tensor:
    """[..., dim]: cos over dim/2 frequencies 10000^(-i/(dim/2)), then sin."""
    half = dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    a = t.float()[..., None] * f
    return torch.cat((a.cos(), a.sin()), dim=-1)


class _ApproxLayer(nn.Module):
    def __init__(self, D, dtype, device):
        super().__init__()
        self.linear_1, self.linear_2 = Linear(D, D, True, dtype, device), Linear(D, D, True, dtype, device)


class DistilledGuidanceLayer(nn.Module):
    def __init__(self, cfg: ChromaConfig, dtype, device):
        super().__init__()
        A = cfg.approx_hidden
        self.in_proj = Linear(cfg.approx_in, A, True, dtype, device)
        self.layers = nn.ModuleList([_ApproxLayer(A, dtype, device) for _ in range(cfg.approx_layers)])
        self.norms = nn.ModuleList([RMSNorm(A, 1e-6, dtype, device) for _ in range(cfg.approx_layers)])
        self.out_proj = Linear(A, cfg.hidden, True, dtype, device)

    def forward(self, x):
        h = self.in_proj(x)
        for lay, norm in zip(self.layers, self.norms):
            h = h + lay.linear_2(lay.linear_1(norm(h), act="silu"))
        return self.out_proj(h)


class _JointAttn(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        D, Dh = cfg.hidden, cfg.head_dim
        self.to_q, self.to_k, self.to_v = [Linear(D, D, True, dtype, device) for _ in range(3)]
        self.add_q_proj, self.add_k_proj, self.add_v_proj = [Linear(D, D, True, dtype, device) for _ in range(3)]
        self.to_out = nn.ModuleList([Linear(D, D, True, dtype, device)])
        self.to_add_out = Linear(D, D, True, dtype, device)
        self.norm_q, self.norm_k = RMSNorm(Dh, 1e-6, dtype, device), RMSNorm(Dh, 1e-6, dtype, device)
        self.norm_added_q, self.norm_added_k = RMSNorm(Dh, 1e-6, dtype, device), RMSNorm(Dh, 1e-6, dtype, device)


def _ff(D, F_, dtype, device):
    proj = nn.Module()
    proj.proj = Linear(D, F_, True, dtype, device)
    m = nn.Module()
    m.net = nn.ModuleDict({"0": proj, "2": Linear(F_, D, True, dtype, device)})
    return m


class ChromaDoubleBlock(nn.Module):
    def __init__(self, cfg: ChromaConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.attn = _JointAttn(cfg, dtype, device)
        self.ff = _ff(cfg.hidden, cfg.mlp_hidden, dtype, device)
        self.ff_context = _ff(cfg.hidden, cfg.mlp_hidden, dtype, device)

    def forward(self, img, txt, mi, mt, cos, sin):
        """mi / mt: [B, 6, D] rows (shift1, scale1, gate1, shift2, scale2, gate2) of this block."""
        cfg, a = self.cfg, self.attn
        B, S_img, D = img.shape
        S_txt = txt.shape[1]
        H, Dh = cfg.heads, cfg.head_dim
        img_n = ops.norm_modulate(img, scale=mi[:, 1], shift=mi[:, 0], eps=1e-6)
        txt_n = ops.norm_modulate(txt, scale=mt[:, 1], shift=mt[:, 0], eps=1e-6)
        qkv = torch.cat((packed_projection(txt_n, (a.add_q_proj, a.add_k_proj, a.add_v_proj)),
                         packed_projection(img_n, (a.to_q, a.to_k, a.to_v))), dim=1)                # text first
        o = ops.qkv_attention(qkv, H, Dh, a.norm_q.weight, a.norm_k.weight, cos, sin, split=S_txt,
                              wq_first=a.norm_added_q.weight, wk_first=a.norm_added_k.weight)
        img = a.to_out[0](o[:, S_txt:], residual=img, gate=mi[:, 2], rows_per_group=S_img)
        txt = a.to_add_out(o[:, :S_txt], residual=txt, gate=mt[:, 2], rows_per_group=S_txt)
        h = self.ff.net["0"].proj(ops.norm_modulate(img, scale=mi[:, 4], shift=mi[:, 3], eps=1e-6), act="gelu_tanh")
        img = self.ff.net["2"](h, residual=img, gate=mi[:, 5], rows_per_group=S_img)
        h = self.ff_context.net["0"].proj(ops.norm_modulate(txt, scale=mt[:, 4], shift=mt[:, 3], eps=1e-6), act="gelu_tanh")
        txt = self.ff_context.net["2"](h, residual=txt, gate=mt[:, 5], rows_per_group=S_txt)
        return img, txt


class _SingleAttn(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        D, Dh = cfg.hidden, cfg.head_dim
        self.to_q, self.to_k, self.to_v = [Linear(D, D, True, dtype, device) for _ in range(3)]
        self.norm_q, self.norm_k = RMSNorm(Dh, 1e-6, dtype, device), RMSNorm(Dh, 1e-6, dtype, device)


class ChromaSingleBlock(nn.Module):
    def __init__(self, cfg: ChromaConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        D, F_ = cfg.hidden, cfg.mlp_hidden
        self.attn = _SingleAttn(cfg, dtype, device)
        self.proj_mlp = Linear(D, F_, True, dtype, device)
        self.proj_out = Linear(D + F_, D, True, dtype, device)

    def forward(self, x, m, cos, sin):
        """m: [B, 3, D] rows (shift, scale, gate)."""
        cfg, a = self.cfg, self.attn
        B, S, D = x.shape
        xn = ops.norm_modulate(x, scale=m[:, 1], shift=m[:, 0], eps=1e-6)
        qkv = packed_projection(xn, (a.to_q, a.to_k, a.to_v))
        o = ops.qkv_attention(qkv, cfg.heads, cfg.head_dim, a.norm_q.weight, a.norm_k.weight, cos, sin)
        mlp = self.proj_mlp(xn, act="gelu_tanh")
        return self.proj_out(torch.cat((o, mlp), dim=-1), residual=x, gate=m[:, 2], rows_per_group=S)


class ChromaDiT(nn.Module):
    """forward(img [B,S_img,64], txt [B,S_txt,4096], t [B] in [0,1], hw) -> velocity [B,S_img,64]."""

    def __init__(self, cfg: ChromaConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        self.x_embedder = Linear(cfg.in_channels, D, True, dtype, device)
        self.context_embedder = Linear(cfg.context_dim, D, True, dtype, device)
        self.distilled_guidance_layer = DistilledGuidanceLayer(cfg, dtype, device)
        self.transformer_blocks = nn.ModuleList([ChromaDoubleBlock(cfg, dtype, device) for _ in range(cfg.depth_double)])
        self.single_transformer_blocks = nn.ModuleList([ChromaSingleBlock(cfg, dtype, device) for _ in range(cfg.depth_single)])
        self.proj_out = Linear(D, cfg.in_channels, True, dtype, device)
        self.gradient_checkpointing = False

    def modulation_table(self, timesteps: torch.Tensor) -> torch.Tensor:
        """[B, rows, D]: every shift / scale / gate of the step from the distilled guidance layer."""
        cfg = self.cfg
        B = timesteps.shape[0]
        q = cfg.approx_in // 4
        rows = cfg.mod_rows
        dev = timesteps.device
        tt = _sinusoid(timesteps * 1000.0, q)                                       # [B, q]
        gg = _sinusoid(torch.zeros_like(timesteps), q)
        idx = _sinusoid(torch.arange(rows, device=dev, dtype=torch.float32) * 1000.0, 2 * q)   # [rows, 2q]
        x = torch.cat((tt[:, None].expand(B, rows, q), gg[:, None].expand(B, rows, q), idx[None].expand(B, rows, 2 * q)), -1)
        return self.distilled_guidance_layer(x.to(self.x_embedder.weight.dtype))

    def forward(self, img, txt, timesteps, hw: Optional[Tuple[int, int]] = None):
        cfg = self.cfg
        S_txt, S_img = txt.shape[1], img.shape[1]
        if hw is None:
            side = int(round(S_img ** 0.5))
            hw = (side, S_img // side)
        cos, sin = ops.rope_table(MMDiT.make_ids(hw[0], hw[1], S_txt, img.device), cfg.axes_dim, cfg.theta)
        dt = self.x_embedder.weight.dtype
        mod = self.modulation_table(timesteps)                                       # [B, rows, D]
        img = self.x_embedder(img.to(dt))
        txt = self.context_embedder(txt.to(dt))
        ns, nd = cfg.depth_single, cfg.depth_double
        i0, t0 = 3 * ns, 3 * ns + 6 * nd
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for i, blk in enumerate(self.transformer_blocks):
            mi, mt = mod[:, i0 + 6 * i:i0 + 6 * i + 6], mod[:, t0 + 6 * i:t0 + 6 * i + 6]
            if ckpt:
                img, txt = torch.utils.checkpoint.checkpoint(blk, img, txt, mi, mt, cos, sin, use_reentrant=False, preserve_rng_state=False)
            else:
                img, txt = blk(img, txt, mi, mt, cos, sin)
        x = torch.cat((txt, img), dim=1)
        for i, blk in enumerate(self.single_transformer_blocks):
            m = mod[:, 3 * i:3 * i + 3]
            if ckpt:
                x = torch.utils.checkpoint.checkpoint(blk, x, m, cos, sin, use_reentrant=False, preserve_rng_state=False)
            else:
                x = blk(x, m, cos, sin)
        rows = cfg.mod_rows
        return self.proj_out(ops.norm_modulate(x[:, S_txt:], scale=mod[:, rows - 1], shift=mod[:, rows - 2], eps=1e-6))

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
