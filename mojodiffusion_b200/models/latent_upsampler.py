"""LTX-2 latent upsampler (second-stage refinement works on a 2x larger latent): a small 3-D convolutional network on the
128-channel video latent.

    initial_conv 128 -> mid, GroupNorm(32) + SiLU, 4 residual blocks, the up-sampling stage, 4 residual blocks,
    final_conv mid -> 128

A residual block is conv -> GroupNorm -> SiLU -> conv -> GroupNorm -> SiLU(x + skip). The spatial variant (mid 1024)
up-samples every frame with a 2-D convolution to 4 * mid channels and a (2, 2) pixel shuffle; the temporal variant (mid 512)
uses a 3-D convolution to 2 * mid channels, interleaves the two halves along time and drops the first frame. All
convolutions are 3x3x3 with zero padding; GroupNorm (eps 1e-5) normalises each group over all frames and pixels. Work
tensors are channel-last [B, T, H, W, C]. Parameter names follow the checkpoint: ``initial_conv``, ``initial_norm``,
``res_blocks.{i}.{conv1,norm1,conv2,norm2}``, ``upsampler.conv`` (spatial) / ``upsampler.0`` (temporal),
``post_upsample_res_blocks.{i}.*``, ``final_conv``; weights in torch's [O, I, kT, kH, kW] / [O, I, kH, kW] layouts.

Facts: serenitymojo/models/upsampler/ltx2_upsampler.mojo:10-45."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn

from ..ops import conv as C
from .layers import init_module_weights


@dataclass
class UpsamplerConfig:
    channels: int = 128
    mid: int = 1024
    temporal: bool = False
    blocks: int = 4
    groups: int = 32
    name: str = "ltx2-spatial-upsampler-x2"


def ltx2_spatial_upsampler_config() -> UpsamplerConfig:
    return UpsamplerConfig()


def ltx2_temporal_upsampler_config() -> UpsamplerConfig:
    return UpsamplerConfig(mid=512, temporal=True, name="ltx2-temporal-upsampler-x2")


def tiny_upsampler_config(temporal: bool = False) -> UpsamplerConfig:
    return UpsamplerConfig(channels=8, mid=32, temporal=temporal, blocks=1, groups=4, name="tiny-upsampler")


class _Conv3(nn.Module):
    def __init__(self, cin, cout, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cout, cin, 3, 3, 3, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device))

    def forward(self, x):
        return C.conv3d_ndhwc(x, self.weight.permute(0, 2, 3, 4, 1).contiguous(), self.bias, None, "zeros")


class _Conv2(nn.Module):
    def __init__(self, cin, cout, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cout, cin, 3, 3, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device))

    def forward(self, x):                                     # x: [N, H, W, C]
        return C.conv2d_nhwc(x, self.weight.permute(0, 2, 3, 1).contiguous(), self.bias, 1, 1)


class _GN(nn.Module):
    def __init__(self, ch, groups, dtype, device):
        super().__init__()
        self.groups = groups
        self.weight = nn.Parameter(torch.ones(ch, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device))

    def forward(self, x, act=None):
        B, T, H, W, Ch = x.shape                              # statistics over all frames and pixels of a group
        return C.group_norm_nhwc(x.reshape(B, T * H * W, 1, Ch), self.weight, self.bias, self.groups, 1e-5, act).reshape(x.shape)


class _Res(nn.Module):
    def __init__(self, ch, groups, dtype, device):
        super().__init__()
        self.conv1, self.conv2 = _Conv3(ch, ch, dtype, device), _Conv3(ch, ch, dtype, device)
        self.norm1, self.norm2 = _GN(ch, groups, dtype, device), _GN(ch, groups, dtype, device)

    def forward(self, x):
        h = self.norm1(self.conv1(x), "silu")
        h = self.norm2(self.conv2(h))
        return torch.nn.functional.silu((h.float() + x.float())).to(x.dtype)


class _SpatialUp(nn.Module):
    def __init__(self, mid, dtype, device):
        super().__init__()
        self.conv = _Conv2(mid, 4 * mid, dtype, device)

    def forward(self, x):
        B, T, H, W, Ch = x.shape
        y = self.conv(x.reshape(B * T, H, W, Ch))                                 # [BT, H, W, 4C], channel = (c, p1, p2)
        y = y.reshape(B, T, H, W, Ch, 2, 2).permute(0, 1, 2, 5, 3, 6, 4)
        return y.reshape(B, T, 2 * H, 2 * W, Ch)


class LatentUpsampler(nn.Module):
    """forward(latent [B, 128, F, H, W]) -> [B, 128, F, 2H, 2W] (spatial) or [B, 128, 2F - 1, H, W] (temporal)."""

    def __init__(self, cfg: UpsamplerConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        m, g = cfg.mid, cfg.groups
        self.initial_conv = _Conv3(cfg.channels, m, dtype, device)
        self.initial_norm = _GN(m, g, dtype, device)
        self.res_blocks = nn.ModuleList([_Res(m, g, dtype, device) for _ in range(cfg.blocks)])
        if cfg.temporal:
            self.upsampler = nn.ModuleList([_Conv3(m, 2 * m, dtype, device)])
        else:
            self.upsampler = _SpatialUp(m, dtype, device)
        self.post_upsample_res_blocks = nn.ModuleList([_Res(m, g, dtype, device) for _ in range(cfg.blocks)])
        self.final_conv = _Conv3(m, cfg.channels, dtype, device)

    @torch.no_grad()
    def forward(self, latent):
        dt = self.initial_conv.weight.dtype
        x = latent.permute(0, 2, 3, 4, 1).to(dt)
        x = self.initial_norm(self.initial_conv(x), "silu")
        for r in self.res_blocks:
            x = r(x)
        if self.cfg.temporal:
            y = self.upsampler[0](x)                                              # [B, T, H, W, 2C], channel = (c, p1)
            B, T, H, W, C2 = y.shape
            y = y.reshape(B, T, H, W, C2 // 2, 2).permute(0, 1, 5, 2, 3, 4).reshape(B, 2 * T, H, W, C2 // 2)
            x = y[:, 1:]
        else:
            x = self.upsampler(x)
        for r in self.post_upsample_res_blocks:
            x = r(x)
        return self.final_conv(x).permute(0, 4, 1, 2, 3)

    def init_weights(self, seed: int = 0, std: float = 0.05):
        return init_module_weights(self, seed, std)
