"""SDXL-shaped UNet (DDPM-family, epsilon prediction): ResBlocks (GroupNorm32 -> SiLU -> conv3x3 + timestep embedding)
and SpatialTransformers (self-attention, cross-attention to a [77, 2048] context, GEGLU feed-forward), NHWC inside.

Shape facts: serenitymojo/models/dit/sdxl_unet.mojo:6-45 (in/out 4, ch 320, mult (1,2,4), 2 res blocks, ctx 2048,
adm 2816, head 64, transformer depth in [0,0,2,2,10,10] mid 10 out [10,10,10,2,2,2,0,0,0]) and :196-552 (block order);
parameter names are the LDM keys (`input_blocks.4.1.transformer_blocks.0.attn2.to_k.weight`, `time_embed.0.weight`,
`label_emb.0.0.weight`, `out.2.weight`). LoRA targets are the Linear layers of the 11 SpatialTransformers
(serenitymojo/models/sdxl/sdxl_real_train.mojo:289,462).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import conv as C
from .layers import LayerNorm, Linear, init_module_weights, packed_projection, timestep_embedding
from .vae import Conv2d, GroupNorm


@dataclass
class UNetConfig:
    in_channels: int = 4
    out_channels: int = 4
    model_channels: int = 320
    channel_mult: Tuple[int, ...] = (1, 2, 4)
    num_res_blocks: int = 2
    transformer_depth: Tuple[int, ...] = (0, 2, 10)     # per resolution level
    context_dim: int = 2048
    adm_in_channels: int = 2816
    head_dim: int = 64
    num_heads: int = 0                       # > 0: fixed head COUNT per attention (SD1.5: 8), head_dim = channels / num_heads
    mid_transformer_depth: int = -1          # -1: that of the deepest level
    name: str = "sdxl-unet"


def sdxl_config() -> UNetConfig:
    return UNetConfig()


def sd15_config() -> UNetConfig:
    """Stable Diffusion 1.5: four levels (1, 2, 4, 4), one transformer block at the first three levels and in the middle,
    eight heads per attention (head sizes 40 / 80 / 160), CLIP-L context, no class / size embedding
    (serenitymojo/sampling/sd15_euler.mojo, the SD1.5 contract of serenitymojo/models/dit/sdxl_unet.mojo)."""
    return UNetConfig(channel_mult=(1, 2, 4, 4), transformer_depth=(1, 1, 1, 0), context_dim=768, adm_in_channels=0, head_dim=0, num_heads=8,
                      mid_transformer_depth=1, name="sd15-unet")


def tiny_sd15_config() -> UNetConfig:
    return UNetConfig(model_channels=64, channel_mult=(1, 2, 2), num_res_blocks=1, transformer_depth=(1, 1, 0), context_dim=48,
                      adm_in_channels=0, head_dim=0, num_heads=4, mid_transformer_depth=1, name="tiny-sd15-unet")


def tiny_unet_config() -> UNetConfig:
    return UNetConfig(model_channels=64, channel_mult=(1, 2), num_res_blocks=1, transformer_depth=(0, 1),
                      context_dim=64, adm_in_channels=96, head_dim=64, name="tiny-unet")


class ResBlock(nn.Module):
    def __init__(self, cin, cout, emb_ch, dtype, device):
        super().__init__()
        self.in_layers = nn.ModuleDict({"0": GroupNorm(cin, 32, 1e-5, dtype, device), "2": Conv2d(cin, cout, 3, dtype=dtype, device=device)})
        self.emb_layers = nn.ModuleDict({"1": Linear(emb_ch, cout, True, dtype, device)})
        self.out_layers = nn.ModuleDict({"0": GroupNorm(cout, 32, 1e-5, dtype, device), "3": Conv2d(cout, cout, 3, dtype=dtype, device=device)})
        if cin != cout:
            self.skip_connection = Conv2d(cin, cout, 1, dtype=dtype, device=device)

    def forward(self, x, emb_silu):
        h = self.in_layers["2"](self.in_layers["0"](x, act="silu"))
        e = self.emb_layers["1"](emb_silu)                                    # [B, cout]
        h = h + e[:, None, None, :]
        skip = self.skip_connection(x) if hasattr(self, "skip_connection") else x
        return self.out_layers["3"](self.out_layers["0"](h, act="silu"), residual=skip)


class CrossAttention(nn.Module):
    def __init__(self, dim, ctx_dim, head_dim, dtype, device):
        super().__init__()
        self.heads, self.head_dim = dim // head_dim, head_dim
        self.to_q = Linear(dim, dim, False, dtype, device)
        self.to_k = Linear(ctx_dim, dim, False, dtype, device)
        self.to_v = Linear(ctx_dim, dim, False, dtype, device)
        self.to_out = nn.ModuleList([Linear(dim, dim, True, dtype, device)])

    def forward(self, x, context, residual):
        B, S, D = x.shape
        q = self.to_q(x).unflatten(-1, (self.heads, self.head_dim))
        kv = packed_projection(context, (self.to_k, self.to_v))
        k = kv[..., :D].unflatten(-1, (self.heads, self.head_dim))
        v = kv[..., D:].unflatten(-1, (self.heads, self.head_dim))
        # head sizes the tcgen05 kernel has no tile shape for (SD1.5: 40 / 80 / 160) go through the library attention
        att = ops.attention if self.head_dim in (64, 128, 256) else ops.reference.attention
        return self.to_out[0](att(q, k, v).reshape(B, S, D), residual=residual)


class GEGLUFF(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        proj = nn.Module()
        proj.proj = Linear(dim, 8 * dim, True, dtype, device)       # (value | gate) halves
        self.net = nn.ModuleDict({"0": proj, "2": Linear(4 * dim, dim, True, dtype, device)})

    def forward(self, x, residual):
        p = self.net["0"].proj
        if len(p.slots) == 0:
            h = ops.linear_glu(x, p.weight, p.bias, "gelu", act_on_second=True)
        else:
            h = ops.glu(p(x), "gelu", True)
        return self.net["2"](h, residual=residual)


class BasicTransformerBlock(nn.Module):
    def __init__(self, dim, ctx_dim, head_dim, dtype, device):
        super().__init__()
        self.norm1 = LayerNorm(dim, 1e-5, True, dtype, device)
        self.attn1 = CrossAttention(dim, dim, head_dim, dtype, device)
        self.norm2 = LayerNorm(dim, 1e-5, True, dtype, device)
        self.attn2 = CrossAttention(dim, ctx_dim, head_dim, dtype, device)
        self.norm3 = LayerNorm(dim, 1e-5, True, dtype, device)
        self.ff = GEGLUFF(dim, dtype, device)

    def forward(self, x, context):
        h = self.norm1(x)
        x = self.attn1(h, h, x)
        x = self.attn2(self.norm2(x), context, x)
        return self.ff(self.norm3(x), x)


class SpatialTransformer(nn.Module):
    def __init__(self, ch, depth, ctx_dim, head_dim, dtype, device):
        super().__init__()
        if head_dim < 0:                         # a negative value is a head count
            head_dim = ch // (-head_dim)
        self.norm = GroupNorm(ch, 32, 1e-6, dtype, device)
        self.proj_in = Linear(ch, ch, True, dtype, device)
        self.transformer_blocks = nn.ModuleList([BasicTransformerBlock(ch, ctx_dim, head_dim, dtype, device) for _ in range(depth)])
        self.proj_out = Linear(ch, ch, True, dtype, device)

    def forward(self, x, context):
        N, H, W, Cc = x.shape
        h = self.proj_in(self.norm(x).reshape(N, H * W, Cc))
        for blk in self.transformer_blocks:
            h = blk(h, context)
        return self.proj_out(h, residual=x.reshape(N, H * W, Cc)).reshape(N, H, W, Cc)


class Downsample(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.op = Conv2d(ch, ch, 3, stride=2, padding=1, dtype=dtype, device=device)

    def forward(self, x, *a):
        return self.op(x)


class Upsample(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.conv = Conv2d(ch, ch, 3, dtype=dtype, device=device)

    def forward(self, x, *a):
        return self.conv(C.upsample_nearest2x_nhwc(x))


def _run(block: nn.ModuleList, x, emb_silu, context):
    for m in block:
        if isinstance(m, ResBlock):
            x = m(x, emb_silu)
        elif isinstance(m, SpatialTransformer):
            x = m(x, context)
        else:
            x = m(x)
    return x


class UNet(nn.Module):
    """forward(x [B,4,h,w], timesteps [B] (0..999), context [B,77,2048], y [B,2816]) -> eps [B,4,h,w]."""

    def __init__(self, cfg: UNetConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        mc = cfg.model_channels
        ted = 4 * mc
        hd = -cfg.num_heads if cfg.num_heads > 0 else cfg.head_dim
        mid_depth = cfg.transformer_depth[-1] if cfg.mid_transformer_depth < 0 else cfg.mid_transformer_depth
        self.time_embed = nn.ModuleDict({"0": Linear(mc, ted, True, dtype, device), "2": Linear(ted, ted, True, dtype, device)})
        if cfg.adm_in_channels > 0:
            le = nn.ModuleDict({"0": Linear(cfg.adm_in_channels, ted, True, dtype, device), "2": Linear(ted, ted, True, dtype, device)})
            self.label_emb = nn.ModuleList([le])
        self.input_blocks = nn.ModuleList([nn.ModuleList([Conv2d(cfg.in_channels, mc, 3, dtype=dtype, device=device)])])
        chans = [mc]
        ch = mc
        nl = len(cfg.channel_mult)
        for lvl, mult in enumerate(cfg.channel_mult):
            for _ in range(cfg.num_res_blocks):
                layers = [ResBlock(ch, mult * mc, ted, dtype, device)]
                ch = mult * mc
                if cfg.transformer_depth[lvl] > 0:
                    layers.append(SpatialTransformer(ch, cfg.transformer_depth[lvl], cfg.context_dim, hd, dtype, device))
                self.input_blocks.append(nn.ModuleList(layers))
                chans.append(ch)
            if lvl != nl - 1:
                self.input_blocks.append(nn.ModuleList([Downsample(ch, dtype, device)]))
                chans.append(ch)
        self.middle_block = nn.ModuleList([ResBlock(ch, ch, ted, dtype, device),
                                           SpatialTransformer(ch, mid_depth, cfg.context_dim, hd, dtype, device),
                                           ResBlock(ch, ch, ted, dtype, device)])
        self.output_blocks = nn.ModuleList()
        for lvl in reversed(range(nl)):
            mult = cfg.channel_mult[lvl]
            for i in range(cfg.num_res_blocks + 1):
                ich = chans.pop()
                layers = [ResBlock(ch + ich, mult * mc, ted, dtype, device)]
                ch = mult * mc
                if cfg.transformer_depth[lvl] > 0:
                    layers.append(SpatialTransformer(ch, cfg.transformer_depth[lvl], cfg.context_dim, hd, dtype, device))
                if lvl and i == cfg.num_res_blocks:
                    layers.append(Upsample(ch, dtype, device))
                self.output_blocks.append(nn.ModuleList(layers))
        self.out = nn.ModuleDict({"0": GroupNorm(ch, 32, 1e-5, dtype, device), "2": Conv2d(ch, cfg.out_channels, 3, dtype=dtype, device=device)})

    def forward(self, x, timesteps, context, y=None):
        cfg = self.cfg
        dt = self.time_embed["0"].weight.dtype
        t_emb = timestep_embedding(timesteps, cfg.model_channels, time_factor=1.0).to(dt)
        emb = self.time_embed["2"](self.time_embed["0"](t_emb, act="silu"))
        if cfg.adm_in_channels > 0:
            le = self.label_emb[0]
            emb = emb + le["2"](le["0"](y.to(dt), act="silu"))
        emb_silu = ops.activation(emb, "silu")
        h = x.permute(0, 2, 3, 1).to(dt).contiguous()
        context = context.to(dt)
        hs = []
        for blk in self.input_blocks:
            h = _run(blk, h, emb_silu, context)
            hs.append(h)
        h = _run(self.middle_block, h, emb_silu, context)
        for blk in self.output_blocks:
            h = _run(blk, torch.cat((h, hs.pop()), dim=-1), emb_silu, context)
        h = self.out["2"](self.out["0"](h, act="silu"))
        return h.permute(0, 3, 1, 2)

    def init_weights(self, seed: int = 0, std: float = 0.03):
        return init_module_weights(self, seed, std)

    def lora_target_names(self) -> List[str]:
        """Module paths of every Linear inside the SpatialTransformers (the reference's SDXL LoRA surface)."""
        return [n for n, m in self.named_modules() if isinstance(m, Linear) and "transformer_blocks" in n]
