"""BigVGAN-style neural vocoder (mel -> waveform) and an iSTFT head variant: conv_pre, a ladder of transposed-conv
upsamplers each followed by multi-receptive-field residual blocks with Snake activations, conv_post. Key names follow the
usual checkpoint layout (``conv_pre``, ``ups.{i}``, ``resblocks.{j}.convs1.{k}`` / ``convs2.{k}`` / ``activations``,
``conv_post``) (serenitymojo/models/vocoder/ltx2_vocoder.mojo, ltx2_stft.mojo)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
from torch import nn

from ..ops import audio as A


@dataclass
class VocoderConfig:
    n_mels: int = 64
    upsample_initial_channel: int = 512
    upsample_rates: Tuple[int, ...] = (5, 4, 2, 2)
    upsample_kernel_sizes: Tuple[int, ...] = (11, 8, 4, 4)
    resblock_kernel_sizes: Tuple[int, ...] = (3, 7, 11)
    resblock_dilations: Tuple[Tuple[int, ...], ...] = ((1, 3, 5), (1, 3, 5), (1, 3, 5))
    istft_head: bool = False          # predict magnitude + phase for a final inverse STFT instead of raw samples
    istft_n_fft: int = 16
    istft_hop: int = 4


def tiny_vocoder_config():
    return VocoderConfig(n_mels=16, upsample_initial_channel=32, upsample_rates=(2, 2), upsample_kernel_sizes=(4, 4),
                         resblock_kernel_sizes=(3,), resblock_dilations=((1, 3),))


class _Conv1d(nn.Module):
    def __init__(self, cin, cout, k, dilation=1, dtype=torch.float32, device=None):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(cout, cin, k, dtype=dtype, device=device) * (1.0 / (cin * k) ** 0.5))
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device))
        self.dilation, self.k = dilation, k

    def forward(self, x):
        return A.conv1d(x, self.weight, self.bias, padding=self.dilation * (self.k - 1) // 2, dilation=self.dilation)


class _Snake(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.alpha = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device))
        self.beta = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device))

    def forward(self, x):
        return A.snake(x, self.alpha, self.beta)


class ResBlock(nn.Module):
    def __init__(self, ch, k, dilations, dtype, device):
        super().__init__()
        self.convs1 = nn.ModuleList([_Conv1d(ch, ch, k, d, dtype, device) for d in dilations])
        self.convs2 = nn.ModuleList([_Conv1d(ch, ch, k, 1, dtype, device) for _ in dilations])
        self.activations = nn.ModuleList([_Snake(ch, dtype, device) for _ in range(2 * len(dilations))])

    def forward(self, x):
        for i, (c1, c2) in enumerate(zip(self.convs1, self.convs2)):
            x = x + c2(self.activations[2 * i + 1](c1(self.activations[2 * i](x))))
        return x


class Vocoder(nn.Module):
    def __init__(self, cfg: VocoderConfig, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        ch = cfg.upsample_initial_channel
        self.conv_pre = _Conv1d(cfg.n_mels, ch, 7, 1, dtype, device)
        self.ups = nn.ParameterList()
        self.up_bias = nn.ParameterList()
        self.resblocks = nn.ModuleList()
        for r, k in zip(cfg.upsample_rates, cfg.upsample_kernel_sizes):
            self.ups.append(nn.Parameter(torch.randn(ch, ch // 2, k, dtype=dtype, device=device) * (1.0 / (ch * k) ** 0.5)))
            self.up_bias.append(nn.Parameter(torch.zeros(ch // 2, dtype=dtype, device=device)))
            ch //= 2
            for rk, rd in zip(cfg.resblock_kernel_sizes, cfg.resblock_dilations):
                self.resblocks.append(ResBlock(ch, rk, rd, dtype, device))
        self.act_post = _Snake(ch, dtype, device)
        out_ch = (cfg.istft_n_fft + 2) if cfg.istft_head else 1
        self.conv_post = _Conv1d(ch, out_ch, 7, 1, dtype, device)

    @property
    def hop(self) -> int:
        h = 1
        for r in self.cfg.upsample_rates:
            h *= r
        return h * (self.cfg.istft_hop if self.cfg.istft_head else 1)

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        """mel [B, n_mels, T] -> waveform [B, T * hop] in [-1, 1]."""
        cfg = self.cfg
        x = self.conv_pre(mel)
        nk = len(cfg.resblock_kernel_sizes)
        for i, (r, k) in enumerate(zip(cfg.upsample_rates, cfg.upsample_kernel_sizes)):
            x = A.conv_transpose1d(x, self.ups[i], self.up_bias[i], stride=r, padding=(k - r) // 2)
            x = sum(self.resblocks[i * nk + j](x) for j in range(nk)) / nk
        x = self.conv_post(self.act_post(x))
        if cfg.istft_head:
            F_ = cfg.istft_n_fft // 2 + 1
            mag, phase = torch.exp(x[:, :F_].float().clamp(max=10.0)), torch.sin(x[:, F_:].float()) * 3.141592653589793
            return A.istft(mag, phase, cfg.istft_n_fft, cfg.istft_hop).clamp(-1, 1)
        return torch.tanh(x.float()).squeeze(1)
