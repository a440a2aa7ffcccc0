"""Anima (MiniTrainDIT): 28 blocks of self-attention, text cross-attention and MLP, each behind its own low-rank adaLN.

    latent [B, 16, T, H, W] + a zero mask channel -> 2 x 2 patches of 17 channels = 68 -> x_embedder (no bias)
    e = sinusoid(sigma);  hidden = SiLU(linear_1 e);  base = linear_2 hidden [B, 3D];  t_cond = RMSNorm(e)
    per sub-layer: (shift, scale, gate) = W2(W1 SiLU(t_cond)) + base          W1: D -> 256, W2: 256 -> 3D
                   x = x + gate * f(LayerNorm(x) * (1 + scale) + shift)
    self-attention: q / k / v (no bias), per-head RMSNorm, 3-axis half-split RoPE; cross-attention: keys / values from
    the 1024-wide text adapter output, per-head RMSNorm, no RoPE; MLP: D -> 4D -> GELU -> D, no biases
    final layer: 2-way low-rank adaLN, linear D -> 64, un-patchify

The model's timestep is the shifted sigma itself. Sampler: shifted sigmas (shift 3), Euler, textbook CFG, 30 steps. Keys
``net.x_embedder.proj.1``, ``net.t_embedder.1.linear_{1,2}``, ``net.t_embedding_norm``,
``net.blocks.{i}.{self_attn,cross_attn}.{q_proj,k_proj,v_proj,output_proj,q_norm,k_norm}``,
``net.blocks.{i}.mlp.layer{1,2}``, ``net.blocks.{i}.adaln_modulation_{self_attn,cross_attn,mlp}.{1,2}``,
``net.final_layer.{adaln_modulation.{1,2},linear}``
(serenitymojo/models/dit/anima_dit.mojo:5-27,885-1200, serenitymojo/sampling/anima_sampling.mojo).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
from torch import nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class AnimaConfig:
    latent_channels: int = 16
    patch: int = 2
    hidden: int = 2048
    heads: int = 16
    head_dim: int = 128
    depth: int = 28
    mlp_hidden: int = 8192
    adaln_lora_dim: int = 256
    context_dim: int = 1024
    axes_dim: Tuple[int, int, int] = (44, 42, 42)
    theta: float = 10000.0
    name: str = "anima"

    @property
    def patch_in(self) -> int:
        return (self.latent_channels + 1) * self.patch * self.patch

    @property
    def patch_out(self) -> int:
        return self.latent_channels * self.patch * self.patch


def anima_config() -> AnimaConfig:
    return AnimaConfig()


def tiny_anima_config() -> AnimaConfig:
    return AnimaConfig(latent_channels=4, hidden=256, heads=4, head_dim=64, depth=2, mlp_hidden=512, adaln_lora_dim=32, context_dim=96,
                       axes_dim=(16, 24, 24), name="tiny-anima")


def _seq(*mods):
    """Modules under the numeric child names a checkpoint uses (index 0 is a parameter-free activation)."""
    m = nn.Module()
    for i, sub in mods:
        m.add_module(str(i), sub)
    return m


class _Attn(nn.Module):
    def __init__(self, cfg, kv_dim, rope: bool, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.cfg, self.rope = cfg, rope
        self.q_proj = Linear(D, D, False, dtype, device)
        self.k_proj = Linear(kv_dim, D, False, dtype, device)
        self.v_proj = Linear(kv_dim, D, False, dtype, device)
        self.output_proj = Linear(D, D, False, dtype, device)
        self.q_norm = RMSNorm(cfg.head_dim, 1e-6, dtype, device)
        self.k_norm = RMSNorm(cfg.head_dim, 1e-6, dtype, device)

    def forward(self, x, ctx, cos, sin, residual, gate, ctx_len=None):
        cfg = self.cfg
        B, S, D = x.shape
        H, Dh = cfg.heads, cfg.head_dim
        if self.rope:
            qkv = packed_projection(x, (self.q_proj, self.k_proj, self.v_proj))
            qkv = ops.qk_norm_rope(qkv, H, Dh, self.q_norm.weight, self.k_norm.weight, cos, sin, eps=1e-6, interleaved=False)
            q, k, v = [qkv[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3)]
        else:
            q = self.q_norm(self.q_proj(x).unflatten(-1, (H, Dh)))
            kv = packed_projection(ctx, (self.k_proj, self.v_proj))
            k = self.k_norm(kv[..., :D].unflatten(-1, (H, Dh)))
            v = kv[..., D:].unflatten(-1, (H, Dh))
        o = ops.attention(q, k, v, kv_len=ctx_len).reshape(B, S, D)
        return self.output_proj(o, residual=residual, gate=gate, rows_per_group=S)


class _AdaLNLoRA(nn.Module):
    def __init__(self, D, r, n, dtype, device):
        super().__init__()
        self.add_module("1", Linear(D, r, False, dtype, device))
        self.add_module("2", Linear(r, n * D, False, dtype, device))

    def forward(self, t_silu, base=None):
        m = getattr(self, "2")(getattr(self, "1")(t_silu))
        return m if base is None else m + base


class AnimaBlock(nn.Module):
    def __init__(self, cfg, dtype, device):
        super().__init__()
        D, r = cfg.hidden, cfg.adaln_lora_dim
        self.self_attn = _Attn(cfg, D, True, dtype, device)
        self.cross_attn = _Attn(cfg, cfg.context_dim, False, dtype, device)
        mlp = nn.Module()
        mlp.layer1, mlp.layer2 = Linear(D, cfg.mlp_hidden, False, dtype, device), Linear(cfg.mlp_hidden, D, False, dtype, device)
        self.mlp = mlp
        self.adaln_modulation_self_attn = _AdaLNLoRA(D, r, 3, dtype, device)
        self.adaln_modulation_cross_attn = _AdaLNLoRA(D, r, 3, dtype, device)
        self.adaln_modulation_mlp = _AdaLNLoRA(D, r, 3, dtype, device)

    def forward(self, x, ctx, t_silu, base, cos, sin, ctx_len=None):
        D, S = x.shape[-1], x.shape[1]
        m = self.adaln_modulation_self_attn(t_silu, base)
        h = ops.norm_modulate(x, scale=m[:, D:2 * D], shift=m[:, :D], eps=1e-6)
        x = self.self_attn(h, None, cos, sin, x, m[:, 2 * D:])
        m = self.adaln_modulation_cross_attn(t_silu, base)
        h = ops.norm_modulate(x, scale=m[:, D:2 * D], shift=m[:, :D], eps=1e-6)
        x = self.cross_attn(h, ctx, None, None, x, m[:, 2 * D:], ctx_len)
        m = self.adaln_modulation_mlp(t_silu, base)
        h = ops.norm_modulate(x, scale=m[:, D:2 * D], shift=m[:, :D], eps=1e-6)
        return self.mlp.layer2(self.mlp.layer1(h, act="gelu_erf"), residual=x, gate=m[:, 2 * D:], rows_per_group=S)


class _Net(nn.Module):
    pass


class Anima(nn.Module):
    """forward(latent [B, C, T, H, W], context [B, L, context_dim], sigma [B]) -> velocity in the latent's shape."""

    def __init__(self, cfg: AnimaConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert cfg.heads * cfg.head_dim == D and sum(cfg.axes_dim) == cfg.head_dim
        net = _Net()
        xe = nn.Module()
        xe.proj = _seq((1, Linear(cfg.patch_in, D, False, dtype, device)))
        net.x_embedder = xe
        te = nn.Module()
        te.linear_1, te.linear_2 = Linear(D, D, False, dtype, device), Linear(D, 3 * D, False, dtype, device)
        net.t_embedder = _seq((1, te))
        net.t_embedding_norm = RMSNorm(D, 1e-6, dtype, device)
        net.blocks = nn.ModuleList([AnimaBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        fl = nn.Module()
        fl.adaln_modulation = _AdaLNLoRA(D, cfg.adaln_lora_dim, 2, dtype, device)
        fl.linear = Linear(D, cfg.patch_out, False, dtype, device)
        net.final_layer = fl
        self.net = net
        self.gradient_checkpointing = False

    def patchify(self, z):
        B, C, T, H, W = z.shape
        p = self.cfg.patch
        z = torch.cat((z, torch.zeros(B, 1, T, H, W, dtype=z.dtype, device=z.device)), dim=1)          # padding-mask channel
        z = z.reshape(B, C + 1, T, H // p, p, W // p, p).permute(0, 2, 3, 5, 1, 4, 6)
        return z.reshape(B, T * (H // p) * (W // p), (C + 1) * p * p), (T, H // p, W // p)

    def unpatchify(self, y, grid):
        B = y.shape[0]
        T, h, w = grid
        p, C = self.cfg.patch, self.cfg.latent_channels
        y = y.reshape(B, T, h, w, p, p, C).permute(0, 6, 1, 2, 4, 3, 5)
        return y.reshape(B, C, T, h * p, w * p)

    def forward(self, latent, context, sigma, ctx_len: Optional[torch.Tensor] = None):
        cfg, net = self.cfg, self.net
        D = cfg.hidden
        image = latent.dim() == 4
        if image:
            latent = latent.unsqueeze(2)
        dt = net.final_layer.linear.weight.dtype
        tokens, grid = self.patchify(latent.to(dt))
        T, h, w = grid
        ids = torch.stack(torch.meshgrid(torch.arange(T), torch.arange(h), torch.arange(w), indexing="ij"), dim=-1).reshape(-1, 3).float().to(latent.device)
        cos, sin = ops.rope_table(ids, cfg.axes_dim, cfg.theta)
        e = timestep_embedding(sigma, D, time_factor=1.0).to(dt)
        te = getattr(net.t_embedder, "1")
        base = te.linear_2(te.linear_1(e, act="silu"))
        t_silu = ops.activation(net.t_embedding_norm(e), "silu")
        x = getattr(net.x_embedder.proj, "1")(tokens)
        ctx = context.to(dt)
        for blk in net.blocks:
            if self.gradient_checkpointing and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(blk, x, ctx, t_silu, base, cos, sin, ctx_len, use_reentrant=False, preserve_rng_state=False)
            else:
                x = blk(x, ctx, t_silu, base, cos, sin, ctx_len)
        m = net.final_layer.adaln_modulation(t_silu) + base[:, :2 * D]
        y = net.final_layer.linear(ops.norm_modulate(x, scale=m[:, D:], shift=m[:, :D], eps=1e-6))
        out = self.unpatchify(y, grid)
        return out.squeeze(2) if image else out

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)


def anima_sigmas(steps: int = 30, shift: float = 3.0):
    from ..sampling.flow_match import shifted_sigmas
    return shifted_sigmas(steps, shift)


def anima_lora_targets(depth: int):
    out = []
    for i in range(depth):
        b = f"net.blocks.{i}."
        for att in ("self_attn", "cross_attn"):
            out += [b + att + "." + n for n in ("q_proj", "k_proj", "v_proj", "output_proj")]
        out += [b + "mlp.layer1", b + "mlp.layer2"]
    return out
