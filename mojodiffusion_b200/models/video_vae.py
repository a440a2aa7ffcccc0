"""LTX-2-shaped video VAE (decoder and the mirrored causal encoder): 128 latent channels, 32x spatial and 8x temporal.

    latent [B,128,F,H,W] -> x*std + mean (per channel) -> conv_in 128->1024
      -> Mid(1024, 2 res) -> D2S(2,2,2; /2) -> Mid(512, 2) -> D2S(2,2,2) -> Mid(512, 4) -> D2S(2,1,1; /2)
      -> Mid(256, 6) -> D2S(1,2,2; /2) -> Mid(128, 4) -> PixelNorm -> SiLU -> conv_out 128->48 -> unpatchify(4)
      -> video [B, 3, 1 + (F-1)*8, 32H, 32W]

Every convolution is 3x3x3 with zero spatial padding and the first / last frame repeated in time (non-causal decoder);
a residual block is PixelNorm -> SiLU -> conv -> PixelNorm -> SiLU -> conv + skip, PixelNorm being the RMS over channels
with eps 1e-6 and no weights; a depth-to-space stage is a convolution to ``C_out * ft*fh*fw`` channels followed by the
c-major rearrangement, and a temporal factor of 2 drops the first output frame. Work tensors are channel-last
[B, T, H, W, C]. Parameter names follow the checkpoint (``decoder.conv_in.conv.weight``,
``decoder.up_blocks.{i}.res_blocks.{r}.conv{1,2}.conv.weight``, ``decoder.up_blocks.{i}.conv.conv.weight``,
``per_channel_statistics.{std-of-means,mean-of-means}``), weights in torch's [O, I, kT, kH, kW] layout.

Facts: serenitymojo/models/vae/ltx2_vae_decoder.mojo:11-66 (schedule), :272-283 (residual block), :296-313
(depth-to-space, frame drop), :316-375 (unpatchify order)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import conv as C
from .layers import init_module_weights


@dataclass
class VideoVAEConfig:
    latent_channels: int = 128
    base_channels: int = 1024
    # (kind, arg...) : ("mid", channels, n_res) | ("d2s", in_ch, ft, fh, fw, reduction)
    blocks: Tuple[Tuple, ...] = (("mid", 1024, 2), ("d2s", 1024, 2, 2, 2, 2), ("mid", 512, 2), ("d2s", 512, 2, 2, 2, 1),
                                 ("mid", 512, 4), ("d2s", 512, 2, 1, 1, 2), ("mid", 256, 6), ("d2s", 256, 1, 2, 2, 2),
                                 ("mid", 128, 4))
    out_channels: int = 3
    patch: int = 4
    enc_base: int = 128
    # ("mid", channels, n_res) | ("s2d", in_ch, out_ch, ft, fh, fw)
    enc_blocks: Tuple[Tuple, ...] = (("mid", 128, 4), ("s2d", 128, 256, 1, 2, 2), ("mid", 256, 6), ("s2d", 256, 512, 2, 1, 1),
                                     ("mid", 512, 4), ("s2d", 512, 1024, 2, 2, 2), ("mid", 1024, 2), ("s2d", 1024, 1024, 2, 2, 2),
                                     ("mid", 1024, 2))
    name: str = "ltx2-video-vae"


def ltx2_vae_config() -> VideoVAEConfig:
    return VideoVAEConfig()


def tiny_video_vae_config() -> VideoVAEConfig:
    return VideoVAEConfig(latent_channels=8, base_channels=64, blocks=(("mid", 64, 1), ("d2s", 64, 2, 2, 2, 2), ("mid", 32, 1),
                                                                       ("d2s", 32, 1, 2, 2, 2), ("mid", 16, 1)),
                          patch=2, enc_base=16, enc_blocks=(("mid", 16, 1), ("s2d", 16, 32, 1, 2, 2), ("mid", 32, 1),
                                                            ("s2d", 32, 64, 2, 2, 2), ("mid", 64, 1)),
                          name="tiny-video-vae")


class _Conv(nn.Module):
    """Holds ``conv.weight`` / ``conv.bias`` under the checkpoint's nesting (``<name>.conv.weight``)."""

    def __init__(self, cin, cout, dtype, device, pad: str = "replicate"):
        super().__init__()
        inner = nn.Module()
        inner.weight = nn.Parameter(torch.empty(cout, cin, 3, 3, 3, dtype=dtype, device=device))
        inner.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device))
        self.conv = inner
        self._taps = None
        self.pad = pad

    def forward(self, x, act=None):
        w = self._taps
        if w is None or w.device != self.conv.weight.device or torch.is_grad_enabled():
            w = self.conv.weight.permute(0, 2, 3, 4, 1).contiguous()          # [O, kT, kH, kW, I]
            if not torch.is_grad_enabled():
                self._taps = w
        return C.conv3d_ndhwc(x, w, self.conv.bias, act, self.pad)


def pixel_norm(x, act=None, eps: float = 1e-6):
    y = ops.norm_modulate(x, eps=eps, rms=True)
    return ops.activation(y, act) if act else y


class _Res(nn.Module):
    def __init__(self, ch, dtype, device, pad: str = "replicate"):
        super().__init__()
        self.conv1, self.conv2 = _Conv(ch, ch, dtype, device, pad), _Conv(ch, ch, dtype, device, pad)

    def forward(self, x):
        h = self.conv1(pixel_norm(x, "silu"))
        return x + self.conv2(pixel_norm(h, "silu"))


class _Mid(nn.Module):
    def __init__(self, ch, n, dtype, device, pad: str = "replicate"):
        super().__init__()
        self.res_blocks = nn.ModuleList([_Res(ch, dtype, device, pad) for _ in range(n)])

    def forward(self, x):
        for r in self.res_blocks:
            x = r(x)
        return x


class _D2S(nn.Module):
    def __init__(self, cin, ft, fh, fw, red, dtype, device):
        super().__init__()
        self.f = (ft, fh, fw)
        self.conv = _Conv(cin, ft * fh * fw * cin // red, dtype, device)

    def forward(self, x):
        y = C.depth_to_space_3d(self.conv(x), *self.f)
        return y[:, 1:] if self.f[0] == 2 else y


class _S2D(nn.Module):
    """Space-to-depth down-sampling with a parameter-free skip: the input (first frame repeated once when time is
    halved) goes through a causal convolution to ``out / prod(stride)`` channels and the c-major space-to-depth
    rearrangement; the skip is the rearranged input itself with every ``in * prod / out`` consecutive channels averaged."""

    def __init__(self, cin, cout, ft, fh, fw, dtype, device):
        super().__init__()
        self.f = (ft, fh, fw)
        prod = ft * fh * fw
        self.group = cin * prod // cout
        self.conv = _Conv(cin, cout // prod, dtype, device, "causal")

    def forward(self, x):
        if self.f[0] == 2:
            x = torch.cat((x[:, :1], x), dim=1)
        skip = C.space_to_depth_3d(x, *self.f)
        if self.group > 1:
            skip = skip.float().unflatten(-1, (-1, self.group)).mean(-1).to(x.dtype)
        return C.space_to_depth_3d(self.conv(x), *self.f) + skip


class _Encoder(nn.Module):
    def __init__(self, cfg: "VideoVAEConfig", dtype, device):
        super().__init__()
        p = cfg.patch
        ch = cfg.enc_base
        self.conv_in = _Conv(cfg.out_channels * p * p, ch, dtype, device, "causal")
        downs = []
        for b in cfg.enc_blocks:
            if b[0] == "mid":
                assert b[1] == ch, (b, ch)
                downs.append(_Mid(ch, b[2], dtype, device, "causal"))
            else:
                assert b[1] == ch, (b, ch)
                downs.append(_S2D(ch, b[2], b[3], b[4], b[5], dtype, device))
                ch = b[2]
        self.down_blocks = nn.ModuleList(downs)
        self.conv_out = _Conv(ch, cfg.latent_channels + 1, dtype, device, "causal")


class _Decoder(nn.Module):
    def __init__(self, cfg: VideoVAEConfig, dtype, device):
        super().__init__()
        self.conv_in = _Conv(cfg.latent_channels, cfg.base_channels, dtype, device)
        ups, ch = [], cfg.base_channels
        for b in cfg.blocks:
            if b[0] == "mid":
                assert b[1] == ch, (b, ch)
                ups.append(_Mid(ch, b[2], dtype, device))
            else:
                assert b[1] == ch, (b, ch)
                ups.append(_D2S(ch, b[2], b[3], b[4], b[5], dtype, device))
                ch = ch // b[5]
        self.up_blocks = nn.ModuleList(ups)
        self.conv_out = _Conv(ch, cfg.out_channels * cfg.patch * cfg.patch, dtype, device)


class VideoVAE(nn.Module):
    def __init__(self, cfg: VideoVAEConfig, dtype=torch.bfloat16, device=None, with_encoder: bool = False):
        super().__init__()
        self.cfg = cfg
        self.decoder = _Decoder(cfg, dtype, device)
        if with_encoder:
            self.encoder = _Encoder(cfg, dtype, device)
        stats = nn.Module()
        stats.register_buffer("std-of-means", torch.ones(cfg.latent_channels, dtype=torch.float32, device=device))
        stats.register_buffer("mean-of-means", torch.zeros(cfg.latent_channels, dtype=torch.float32, device=device))
        self.per_channel_statistics = stats

    def expansion(self) -> Tuple[int, int]:
        t = s = 1
        for b in self.cfg.blocks:
            if b[0] == "d2s":
                t, s = t * b[2], s * b[3]
        return t, s * self.cfg.patch

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        """latent [B, C, F, H, W] (normalised) -> video [B, 3, 1 + (F-1)*ft, H*fs, W*fs], roughly in [-1, 1]."""
        cfg, d = self.cfg, self.decoder
        dt = d.conv_in.conv.weight.dtype
        st = self.per_channel_statistics
        z = latent.permute(0, 2, 3, 4, 1).float() * getattr(st, "std-of-means") + getattr(st, "mean-of-means")
        h = d.conv_in(z.to(dt))
        for blk in d.up_blocks:
            h = blk(h)
        h = d.conv_out(pixel_norm(h, "silu"))                                   # [B, T, H, W, 3*p*p]
        B, T, H, W, _ = h.shape
        p = cfg.patch
        # channel = (c, a, b) c-major; b indexes the row offset and a the column offset inside a patch
        h = h.reshape(B, T, H, W, cfg.out_channels, p, p).permute(0, 4, 1, 2, 6, 3, 5)
        return h.reshape(B, cfg.out_channels, T, H * p, W * p)

    @torch.no_grad()
    def encode(self, video: torch.Tensor) -> torch.Tensor:
        """video [B, 3, T, H, W] in [-1, 1] (T = 1 + 8k) -> normalised latent mean [B, C, T', H / 32, W / 32]: pixel-unshuffle
        by the patch size, causal convolutions (the first frame repeated on the left), residual blocks and space-to-depth
        stages, PixelNorm (eps 1e-8) + SiLU, a projection to C + 1 channels of which the first C are the mean
        (serenitymojo/models/vae/ltx2_vae_encoder.mojo:13-34, :47-58)."""
        cfg, e = self.cfg, self.encoder
        dt = e.conv_in.conv.weight.dtype
        B, Cc, T, H, W = video.shape
        p = cfg.patch
        x = video.reshape(B, Cc, T, H // p, p, W // p, p).permute(0, 2, 3, 5, 1, 6, 4)        # channel = (c, col, row)
        h = e.conv_in(x.reshape(B, T, H // p, W // p, Cc * p * p).to(dt))
        for blk in e.down_blocks:
            h = blk(h)
        h = e.conv_out(pixel_norm(h, "silu", 1e-8))
        mu = h[..., :cfg.latent_channels].float()
        st = self.per_channel_statistics
        mu = (mu - getattr(st, "mean-of-means")) / getattr(st, "std-of-means")
        return mu.permute(0, 4, 1, 2, 3)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
