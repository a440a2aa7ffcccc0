"""SD3 / SD3.5-shaped MMDiT: joint blocks of a context stream and an image stream with per-block adaLN from
``c = t_embedder(t) + y_embedder(pooled)``, joint attention over [context | image] without rotary embedding (a learned
position table, centre-cropped to the latent grid, is added after patch embedding), per-head RMS QK norm (SD3.5), GELU-tanh
MLP x4; the last context block is ``pre_only`` (it only feeds keys / values); SD3.5-Medium's first 13 image blocks carry a
second, image-only attention (nine modulation vectors).

Sizes: Large = 38 blocks, hidden 2432, 38 heads x 64; Medium = 24 blocks, hidden 1536, 24 heads x 64, dual attention in
blocks 0-12; 16 latent channels, patch 2, context 4096, pooled 2048, position grid 192 (Large) / 384 (Medium). Parameter
names are the checkpoint's after removing ``model.diffusion_model.``: ``joint_blocks.{i}.{x_block,context_block}.
{adaLN_modulation.1, attn.qkv, attn.ln_q, attn.ln_k, attn.proj, mlp.fc1, mlp.fc2, attn2.*}``, ``x_embedder.proj``,
``pos_embed``, ``t_embedder.mlp.{0,2}``, ``y_embedder.mlp.{0,2}``, ``context_embedder``, ``final_layer.*``.

Facts: serenitymojo/models/dit/sd3_mmdit.mojo:1-34 (block rules and keys), :160-215 (position crop), :490-540 (final
layer, unpatchify order); serenitymojo/models/dit/sd3_contract.mojo:11-81 (sizes)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, init_module_weights, timestep_embedding


@dataclass
class SD3Config:
    in_channels: int = 16
    patch: int = 2
    hidden: int = 2432
    heads: int = 38
    head_dim: int = 64
    depth: int = 38
    context_dim: int = 4096
    pooled_dim: int = 2048
    pos_grid: int = 192
    dual_attention_blocks: int = 0
    time_dim: int = 256
    name: str = "sd3.5-large"


def sd35_large_config() -> SD3Config:
    return SD3Config()


def sd35_medium_config() -> SD3Config:
    return SD3Config(hidden=1536, heads=24, depth=24, pos_grid=384, dual_attention_blocks=13, name="sd3.5-medium")


def tiny_sd3_config() -> SD3Config:
    return SD3Config(in_channels=4, hidden=128, heads=2, head_dim=64, depth=3, context_dim=96, pooled_dim=48, pos_grid=16,
                     dual_attention_blocks=1, name="tiny-sd3")


class _NormW(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))


class _Attn(nn.Module):
    def __init__(self, D, Dh, pre_only, dtype, device):
        super().__init__()
        self.qkv = Linear(D, 3 * D, True, dtype, device)
        self.ln_q, self.ln_k = _NormW(Dh, dtype, device), _NormW(Dh, dtype, device)
        if not pre_only:
            self.proj = Linear(D, D, True, dtype, device)


class _Mlp(nn.Module):
    def __init__(self, D, dtype, device):
        super().__init__()
        self.fc1, self.fc2 = Linear(D, 4 * D, True, dtype, device), Linear(4 * D, D, True, dtype, device)


class _Stream(nn.Module):
    def __init__(self, cfg: SD3Config, pre_only: bool, dual: bool, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.pre_only, self.dual = pre_only, dual
        self.n_mod = 2 if pre_only else (9 if dual else 6)
        self.adaLN_modulation = nn.ModuleDict({"1": Linear(D, self.n_mod * D, True, dtype, device)})
        self.attn = _Attn(D, cfg.head_dim, pre_only, dtype, device)
        if dual:
            self.attn2 = _Attn(D, cfg.head_dim, False, dtype, device)
        if not pre_only:
            self.mlp = _Mlp(D, dtype, device)

    def mods(self, c_silu):
        m = self.adaLN_modulation["1"](c_silu)
        D = m.shape[-1] // self.n_mod
        return [m[:, j * D:(j + 1) * D] for j in range(self.n_mod)]


class SD3JointBlock(nn.Module):
    def __init__(self, cfg: SD3Config, last: bool, dual: bool, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.context_block = _Stream(cfg, last, False, dtype, device)
        self.x_block = _Stream(cfg, False, dual, dtype, device)

    def forward(self, ctx, x, c_silu):
        cfg = self.cfg
        H, Dh = cfg.heads, cfg.head_dim
        S_ctx, S_x = ctx.shape[1], x.shape[1]
        cb, xb = self.context_block, self.x_block
        mc, mx = cb.mods(c_silu), xb.mods(c_silu)
        ctx_n = ops.norm_modulate(ctx, scale=mc[1], shift=mc[0], eps=1e-6)
        x_n = ops.norm_modulate(x, scale=mx[1], shift=mx[0], eps=1e-6)
        qkv = torch.cat((cb.attn.qkv(ctx_n), xb.attn.qkv(x_n)), dim=1)                   # context first
        a = ops.qkv_attention(qkv, H, Dh, xb.attn.ln_q.weight, xb.attn.ln_k.weight, None, None, split=S_ctx,
                              wq_first=cb.attn.ln_q.weight, wk_first=cb.attn.ln_k.weight)
        a_ctx, a_x = a[:, :S_ctx], a[:, S_ctx:]
        x_in = x
        x = xb.attn.proj(a_x, residual=x, gate=mx[2], rows_per_group=S_x)
        if xb.dual:
            x2 = ops.norm_modulate(x_in, scale=mx[7], shift=mx[6], eps=1e-6)
            a2 = ops.qkv_attention(xb.attn2.qkv(x2), H, Dh, xb.attn2.ln_q.weight, xb.attn2.ln_k.weight, None, None)
            x = xb.attn2.proj(a2, residual=x, gate=mx[8], rows_per_group=S_x)
        h = xb.mlp.fc1(ops.norm_modulate(x, scale=mx[4], shift=mx[3], eps=1e-6), act="gelu_tanh")
        x = xb.mlp.fc2(h, residual=x, gate=mx[5], rows_per_group=S_x)
        if not cb.pre_only:
            ctx = cb.attn.proj(a_ctx, residual=ctx, gate=mc[2], rows_per_group=S_ctx)
            h = cb.mlp.fc1(ops.norm_modulate(ctx, scale=mc[4], shift=mc[3], eps=1e-6), act="gelu_tanh")
            ctx = cb.mlp.fc2(h, residual=ctx, gate=mc[5], rows_per_group=S_ctx)
        return ctx, x


class _Mlp2(nn.Module):
    def __init__(self, i, D, dtype, device):
        super().__init__()
        self.mlp = nn.ModuleDict({"0": Linear(i, D, True, dtype, device), "2": Linear(D, D, True, dtype, device)})

    def forward(self, v):
        return self.mlp["2"](self.mlp["0"](v, act="silu"))


class _Patch(nn.Module):
    """``x_embedder.proj``: a stride-``p`` convolution = one linear over (channel, row, column)-ordered patches."""

    def __init__(self, cin, p, D, dtype, device):
        super().__init__()
        proj = nn.Module()
        proj.weight = nn.Parameter(torch.empty(D, cin, p, p, dtype=dtype, device=device))
        proj.bias = nn.Parameter(torch.zeros(D, dtype=dtype, device=device))
        self.proj = proj
        self.p = p

    def forward(self, z):
        B, C, Hh, Ww = z.shape
        p = self.p
        t = z.reshape(B, C, Hh // p, p, Ww // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, (Hh // p) * (Ww // p), C * p * p)
        return ops.linear(t.to(self.proj.weight.dtype), self.proj.weight.flatten(1), self.proj.bias)


class _Final(nn.Module):
    def __init__(self, D, out, dtype, device):
        super().__init__()
        self.linear = Linear(D, out, True, dtype, device)
        self.adaLN_modulation = nn.ModuleDict({"1": Linear(D, 2 * D, True, dtype, device)})


class SD3MMDiT(nn.Module):
    """forward(latent [B,16,h,w], context [B,T,4096], t [B] in [0,1], pooled [B,2048]) -> velocity [B,16,h,w]."""

    def __init__(self, cfg: SD3Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert cfg.heads * cfg.head_dim == D
        self.x_embedder = _Patch(cfg.in_channels, cfg.patch, D, dtype, device)
        self.pos_embed = nn.Parameter(torch.zeros(1, cfg.pos_grid * cfg.pos_grid, D, dtype=dtype, device=device))
        self.t_embedder = _Mlp2(cfg.time_dim, D, dtype, device)
        self.y_embedder = _Mlp2(cfg.pooled_dim, D, dtype, device)
        self.context_embedder = Linear(cfg.context_dim, D, True, dtype, device)
        self.joint_blocks = nn.ModuleList([SD3JointBlock(cfg, i == cfg.depth - 1, i < cfg.dual_attention_blocks, dtype, device)
                                           for i in range(cfg.depth)])
        self.final_layer = _Final(D, cfg.patch * cfg.patch * cfg.in_channels, dtype, device)
        self.gradient_checkpointing = False

    def cropped_pos_embed(self, h: int, w: int) -> torch.Tensor:
        """The centre h x w window of the learned position grid, flattened row-major."""
        G = self.cfg.pos_grid
        assert h <= G and w <= G, "latent grid exceeds the position table"
        top, left = (G - h) // 2, (G - w) // 2
        pe = self.pos_embed.reshape(1, G, G, -1)[:, top:top + h, left:left + w]
        return pe.reshape(1, h * w, -1)

    def forward(self, z, context, timesteps, pooled):
        cfg = self.cfg
        B, C, Hh, Ww = z.shape
        p = cfg.patch
        h, w = Hh // p, Ww // p
        dt = self.context_embedder.weight.dtype
        x = self.x_embedder(z) + self.cropped_pos_embed(h, w)
        c = self.t_embedder(timestep_embedding(timesteps, cfg.time_dim).to(dt)) + self.y_embedder(pooled.to(dt))
        c_silu = ops.activation(c, "silu")
        ctx = self.context_embedder(context.to(dt))
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.joint_blocks:
            if ckpt:
                ctx, x = torch.utils.checkpoint.checkpoint(blk, ctx, x, c_silu, use_reentrant=False, preserve_rng_state=False)
            else:
                ctx, x = blk(ctx, x, c_silu)
        D = cfg.hidden
        m = self.final_layer.adaLN_modulation["1"](c_silu)
        out = self.final_layer.linear(ops.norm_modulate(x, scale=m[:, D:], shift=m[:, :D], eps=1e-6))
        # token vector is (row-in-patch, column-in-patch, channel): channel innermost
        out = out.reshape(B, h, w, p, p, C).permute(0, 5, 1, 3, 2, 4)
        return out.reshape(B, C, Hh, Ww)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        init_module_weights(self, seed, std)
        with torch.no_grad():
            g = torch.Generator().manual_seed(seed + 1)
            self.pos_embed.copy_((torch.randn(self.pos_embed.shape, generator=g) * std).to(self.pos_embed.dtype))
            for n, prm in self.named_parameters():
                if n.endswith("ln_q.weight") or n.endswith("ln_k.weight"):
                    prm.fill_(1.0)
        return self
