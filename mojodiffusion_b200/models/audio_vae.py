"""LTX-2 audio VAE (decoder and encoder) over [B, 8, T, 16] latents (8 channels x 16 mel bins per time step).

Decoder (serenitymojo/models/vae/ltx2_audio_vae.mojo:1-90): un-normalise with the 128 per-channel statistics (latent
rearranged ``b c t f -> b t (c f)``) -> causal conv_in 8 -> 512 -> mid (two residual blocks, no attention) -> three up
stages visited from the deepest (512 -> 512 with upsample, 512 -> 256 with upsample, 256 -> 128 without), each upsample =
nearest x2 in time and frequency, causal conv, first time frame dropped -> PixelNorm (channel RMS, eps 1e-6) -> SiLU ->
causal conv_out 128 -> 2 (stereo log-mel for the vocoder). Time grows T -> 2T-1 -> 4T-3, frequency 16 -> 64. Causal
convolution: zero padding of ``k - 1`` rows before the first time step, symmetric zero padding in frequency. Computed in
fp32 (the reference keeps the audio VAE and the vocoder in fp32). The encoder mirrors the decoder (causal strided
convolutions down, mean / log-variance head).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn as nn
import torch.nn.functional as TF

from .layers import init_module_weights


@dataclass
class AudioVAEConfig:
    latent_channels: int = 8
    mel_bins_latent: int = 16
    base_channels: int = 128
    ch_mult: Tuple[int, ...] = (1, 2, 4)          # up[0] .. up[2] output widths: 128, 256, 512
    num_res_blocks: int = 3
    out_channels: int = 2
    name: str = "ltx2-audio-vae"


def ltx2_audio_vae_config() -> AudioVAEConfig:
    return AudioVAEConfig()


def tiny_audio_vae_config() -> AudioVAEConfig:
    return AudioVAEConfig(latent_channels=4, mel_bins_latent=4, base_channels=16, ch_mult=(1, 2), num_res_blocks=1, name="tiny-audio-vae")


class CausalConv2d(nn.Module):
    """2-D convolution over [B, C, T, F]: causal (zero pad k-1 before) along T, symmetric zero pad along F."""

    def __init__(self, cin, cout, k=3, stride=1, dtype=torch.float32, device=None):
        super().__init__()
        self.conv = nn.Conv2d(cin, cout, k, stride=stride, padding=0, dtype=dtype, device=device)
        self.k = k

    def forward(self, x):
        k = self.k
        return self.conv(TF.pad(x, ((k - 1) // 2, (k - 1) // 2, k - 1, 0)))


def pixel_norm(x, eps: float = 1e-6):
    return x * torch.rsqrt(x.pow(2).mean(dim=1, keepdim=True) + eps)


class ResnetBlock(nn.Module):
    def __init__(self, cin, cout, dtype, device):
        super().__init__()
        self.conv1 = CausalConv2d(cin, cout, 3, 1, dtype, device)
        self.conv2 = CausalConv2d(cout, cout, 3, 1, dtype, device)
        if cin != cout:
            self.nin_shortcut = CausalConv2d(cin, cout, 1, 1, dtype, device)

    def forward(self, x):
        h = self.conv1(TF.silu(pixel_norm(x)))
        h = self.conv2(TF.silu(pixel_norm(h)))
        return (self.nin_shortcut(x) if hasattr(self, "nin_shortcut") else x) + h


class Upsample(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.conv = CausalConv2d(ch, ch, 3, 1, dtype, device)

    def forward(self, x):
        x = TF.interpolate(x, scale_factor=2.0, mode="nearest")
        return self.conv(x)[:, :, 1:]                      # the first time frame has no causal support: dropped


class Downsample(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.conv = CausalConv2d(ch, ch, 3, 2, dtype, device)

    def forward(self, x):
        return self.conv(x)


class _Stage(nn.Module):
    def __init__(self):
        super().__init__()
        self.block = nn.ModuleList()


class AudioDecoder(nn.Module):
    def __init__(self, cfg: AudioVAEConfig, dtype, device):
        super().__init__()
        top = cfg.base_channels * cfg.ch_mult[-1]
        self.conv_in = CausalConv2d(cfg.latent_channels, top, 3, 1, dtype, device)
        mid = nn.Module()
        mid.block_1, mid.block_2 = ResnetBlock(top, top, dtype, device), ResnetBlock(top, top, dtype, device)
        self.mid = mid
        self.up = nn.ModuleList()
        ch = top
        stages = []
        for lvl in reversed(range(len(cfg.ch_mult))):
            st = _Stage()
            out = cfg.base_channels * cfg.ch_mult[lvl]
            for _ in range(cfg.num_res_blocks):
                st.block.append(ResnetBlock(ch, out, dtype, device))
                ch = out
            if lvl != 0:
                st.upsample = Upsample(ch, dtype, device)
            stages.append(st)
        for st in reversed(stages):                        # stored up[0] (shallowest) .. up[n-1]; visited in reverse
            self.up.append(st)
        self.conv_out = CausalConv2d(ch, cfg.out_channels, 3, 1, dtype, device)

    def forward(self, z):
        h = self.conv_in(z)
        h = self.mid.block_2(self.mid.block_1(h))
        for st in reversed(self.up):
            for b in st.block:
                h = b(h)
            if hasattr(st, "upsample"):
                h = st.upsample(h)
        return self.conv_out(TF.silu(pixel_norm(h)))


class AudioEncoder(nn.Module):
    def __init__(self, cfg: AudioVAEConfig, dtype, device):
        super().__init__()
        ch = cfg.base_channels
        self.conv_in = CausalConv2d(cfg.out_channels, ch, 3, 1, dtype, device)
        self.down = nn.ModuleList()
        for lvl, mult in enumerate(cfg.ch_mult):
            st = _Stage()
            out = cfg.base_channels * mult
            for _ in range(cfg.num_res_blocks):
                st.block.append(ResnetBlock(ch, out, dtype, device))
                ch = out
            if lvl != len(cfg.ch_mult) - 1:
                st.downsample = Downsample(ch, dtype, device)
            self.down.append(st)
        mid = nn.Module()
        mid.block_1, mid.block_2 = ResnetBlock(ch, ch, dtype, device), ResnetBlock(ch, ch, dtype, device)
        self.mid = mid
        self.conv_out = CausalConv2d(ch, 2 * cfg.latent_channels, 3, 1, dtype, device)

    def forward(self, mel):
        h = self.conv_in(mel)
        for st in self.down:
            for b in st.block:
                h = b(h)
            if hasattr(st, "downsample"):
                h = st.downsample(h)
        h = self.mid.block_2(self.mid.block_1(h))
        return self.conv_out(TF.silu(pixel_norm(h)))


class AudioVAE(nn.Module):
    def __init__(self, cfg: AudioVAEConfig, dtype=torch.float32, device=None, with_encoder: bool = True):
        super().__init__()
        self.cfg = cfg
        self.decoder = AudioDecoder(cfg, dtype, device)
        if with_encoder:
            self.encoder = AudioEncoder(cfg, dtype, device)
        st = nn.Module()
        n = cfg.latent_channels * cfg.mel_bins_latent
        st.register_buffer("mean-of-means", torch.zeros(n, dtype=dtype, device=device))
        st.register_buffer("std-of-means", torch.ones(n, dtype=dtype, device=device))
        self.per_channel_statistics = st

    def _stats(self):
        st = self.per_channel_statistics
        return getattr(st, "mean-of-means"), getattr(st, "std-of-means")

    def un_normalize(self, z):
        """[B, C, T, F] latent -> physical scale, statistics indexed by (channel, mel bin)."""
        B, Cc, T, Fq = z.shape
        mean, std = self._stats()
        x = z.permute(0, 2, 1, 3).reshape(B, T, Cc * Fq).float() * std.float() + mean.float()
        return x.reshape(B, T, Cc, Fq).permute(0, 2, 1, 3)

    def normalize(self, z):
        B, Cc, T, Fq = z.shape
        mean, std = self._stats()
        x = (z.permute(0, 2, 1, 3).reshape(B, T, Cc * Fq).float() - mean.float()) / std.float()
        return x.reshape(B, T, Cc, Fq).permute(0, 2, 1, 3)

    @torch.no_grad()
    def decode(self, z):
        """latent [B, 8, T, 16] -> stereo log-mel [B, 2, 4T-3, 64]."""
        return self.decoder(self.un_normalize(z).to(self.decoder.conv_in.conv.weight.dtype))

    @torch.no_grad()
    def encode(self, mel, sample: bool = False, generator=None):
        moments = self.encoder(mel.to(self.decoder.conv_in.conv.weight.dtype))
        mean, logvar = moments.chunk(2, dim=1)
        z = mean
        if sample:
            z = mean + torch.exp(0.5 * logvar.clamp(-30, 20)) * torch.randn(mean.shape, generator=generator, dtype=mean.dtype).to(mean.device)
        return self.normalize(z)

    def init_weights(self, seed: int = 0, std: float = 0.05):
        return init_module_weights(self, seed, std)
