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


# ---- BigVGAN-v2 generator with anti-aliased activations, and the bandwidth-extension wrapper --------------------------
@dataclass
class BigVGAN2Config:
    """Stereo generator of the LTX-2 audio stack: ``in_channels`` = 2 x 64 mel bins, six transposed-conv stages
    (5, 2, 2, 2, 2, 2) from 1536 channels, three AMP blocks (kernel 3 / 7 / 11, dilations 1 / 3 / 5) per stage whose
    outputs are averaged, an anti-aliased SnakeBeta before conv_post, two output channels, no final tanh. The
    bandwidth-extension generator has five stages (6, 5, 2, 2, 2)
    (serenitymojo/models/vocoder/ltx2_vocoder.mojo:9-22,80-115)."""
    in_channels: int = 128
    upsample_initial_channel: int = 1536
    upsample_rates: Tuple[int, ...] = (5, 2, 2, 2, 2, 2)
    upsample_kernel_sizes: Tuple[int, ...] = (11, 4, 4, 4, 4, 4)
    resblock_kernel_sizes: Tuple[int, ...] = (3, 7, 11)
    resblock_dilations: Tuple[int, ...] = (1, 3, 5)
    out_channels: int = 2
    use_tanh_at_final: bool = False
    conv_post_bias: bool = True


def ltx2_vocoder_config() -> BigVGAN2Config:
    return BigVGAN2Config()


def ltx2_bwe_config() -> BigVGAN2Config:
    return BigVGAN2Config(upsample_initial_channel=512, upsample_rates=(6, 5, 2, 2, 2), upsample_kernel_sizes=(12, 11, 4, 4, 4))


def tiny_bigvgan2_config(in_channels: int = 16, rates=(2, 2)) -> BigVGAN2Config:
    return BigVGAN2Config(in_channels=in_channels, upsample_initial_channel=16, upsample_rates=tuple(rates),
                          upsample_kernel_sizes=tuple(2 * r for r in rates), resblock_kernel_sizes=(3, 7), resblock_dilations=(1, 3))


class _Filter(nn.Module):
    def __init__(self, filt):
        super().__init__()
        self.register_buffer("filter", filt.view(1, 1, -1).clone())


class Activation1d(nn.Module):
    """SnakeBeta evaluated at twice the rate between a kaiser-sinc interpolator and decimator. Keys ``act.alpha``,
    ``act.beta``, ``upsample.filter``, ``downsample.lowpass.filter`` (ltx2_vocoder.mojo:150-215)."""

    def __init__(self, ch, dtype, device):
        super().__init__()
        act = nn.Module()
        act.alpha = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device))
        act.beta = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device))
        self.act = act
        f = A.kaiser_sinc_filter1d(0.25, 0.3, 12).to(device=device, dtype=dtype)
        self.upsample = _Filter(f)
        down = nn.Module()
        down.lowpass = _Filter(f)
        self.downsample = down

    def forward(self, x):
        return A.activation1d(x, self.act.alpha, self.act.beta, self.upsample.filter.flatten(), self.downsample.lowpass.filter.flatten())


class AMPBlock1(nn.Module):
    def __init__(self, ch, k, dilations, dtype, device):
        super().__init__()
        self.convs1 = nn.ModuleList([_Conv1d(ch, ch, k, d, dtype, device) for d in dilations])
        self.convs2 = nn.ModuleList([_Conv1d(ch, ch, k, 1, dtype, device) for _ in dilations])
        self.acts1 = nn.ModuleList([Activation1d(ch, dtype, device) for _ in dilations])
        self.acts2 = nn.ModuleList([Activation1d(ch, dtype, device) for _ in dilations])

    def forward(self, x):
        for a1, c1, a2, c2 in zip(self.acts1, self.convs1, self.acts2, self.convs2):
            x = x + c2(a2(c1(a1(x))))
        return x


class _Up(nn.Module):
    def __init__(self, cin, cout, k, stride, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(cin, cout, k, dtype=dtype, device=device) * (1.0 / (cin * k) ** 0.5))
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device))
        self.stride, self.k = stride, k

    def forward(self, x):
        return A.conv_transpose1d(x, self.weight, self.bias, stride=self.stride, padding=(self.k - self.stride) // 2)


class BigVGAN2(nn.Module):
    """mel [B, 2, T, F] (or [B, C, T]) -> waveform [B, out_channels, T * prod(rates)] in fp32."""

    def __init__(self, cfg: BigVGAN2Config, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        ch = cfg.upsample_initial_channel
        self.conv_pre = _Conv1d(cfg.in_channels, ch, 7, 1, dtype, device)
        self.ups = nn.ModuleList()
        self.resblocks = nn.ModuleList()
        for r, k in zip(cfg.upsample_rates, cfg.upsample_kernel_sizes):
            self.ups.append(_Up(ch, ch // 2, k, r, dtype, device))
            ch //= 2
            for rk in cfg.resblock_kernel_sizes:
                self.resblocks.append(AMPBlock1(ch, rk, cfg.resblock_dilations, dtype, device))
        self.act_post = Activation1d(ch, dtype, device)
        self.conv_post = _Conv1d(ch, cfg.out_channels, 7, 1, dtype, device)
        if not cfg.conv_post_bias:
            self.conv_post.bias.requires_grad_(False)

    @property
    def hop(self) -> int:
        h = 1
        for r in self.cfg.upsample_rates:
            h *= r
        return h

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        if mel.dim() == 4:                                   # [B, 2, T, F] -> [B, 2F, T]
            B, Cc, T, Fq = mel.shape
            mel = mel.permute(0, 1, 3, 2).reshape(B, Cc * Fq, T)
        x = self.conv_pre(mel.float())
        nk = len(self.cfg.resblock_kernel_sizes)
        for i, up in enumerate(self.ups):
            x = up(x)
            acc = self.resblocks[i * nk](x)
            for j in range(1, nk):
                acc = acc + self.resblocks[i * nk + j](x)
            x = acc / nk
        x = self.conv_post(self.act_post(x))
        return torch.tanh(x) if self.cfg.use_tanh_at_final else x


class _STFTBasis(nn.Module):
    def __init__(self, n_fft, dtype, device):
        super().__init__()
        n = torch.arange(n_fft, dtype=torch.float64)
        k = torch.arange(n_fft // 2 + 1, dtype=torch.float64)[:, None]
        win = torch.hann_window(n_fft, periodic=True, dtype=torch.float64)
        ang = 2 * torch.pi * k * n / n_fft
        basis = torch.cat([torch.cos(ang) * win, -torch.sin(ang) * win], 0)[:, None]          # real rows first
        self.register_buffer("forward_basis", basis.to(dtype=dtype, device=device))


class MelSTFT(nn.Module):
    """Log-mel of a waveform by a strided convolution with a windowed Fourier basis (no FFT): zero padding of
    ``win - hop`` samples on the left only, magnitude from the real-first / imaginary-second halves, mel projection,
    clamp(1e-5) and log (serenitymojo/models/vocoder/ltx2_stft.mojo:9-22)."""

    def __init__(self, n_fft=512, hop=80, n_mels=64, sample_rate=16000, dtype=torch.float32, device=None):
        super().__init__()
        self.hop = hop
        self.stft_fn = _STFTBasis(n_fft, dtype, device)
        self.register_buffer("mel_basis", A.mel_filterbank(n_mels, n_fft, sample_rate).to(dtype=dtype, device=device))

    def forward(self, audio):
        B, Cc, T = audio.shape
        basis = self.stft_fn.forward_basis
        win = basis.shape[-1]
        flat = torch.nn.functional.pad(audio.float().reshape(B * Cc, 1, T), (win - self.hop, 0))
        spec = torch.nn.functional.conv1d(flat, basis.float(), stride=self.hop)
        nf = basis.shape[0] // 2
        mag = torch.sqrt(spec[:, :nf] ** 2 + spec[:, nf:] ** 2)
        mel = torch.einsum("mf,bft->bmt", self.mel_basis.float(), mag)
        return torch.log(mel.clamp(1e-5, 1e10)).reshape(B, Cc, -1, mel.shape[-1])


class VocoderWithBWE(nn.Module):
    """16 kHz generator, then bandwidth extension to 48 kHz: log-mel of the (hop-padded) low-rate waveform -> second
    generator -> residual added to a Hann-sinc x3 upsampling of the low-rate waveform, clamped to [-1, 1] and trimmed to
    ``len16 * 3``. Keys ``vocoder.*``, ``bwe_generator.*``, ``mel_stft.*`` (ltx2_vocoder.mojo:24-33,575-625)."""

    def __init__(self, voc_cfg: BigVGAN2Config, bwe_cfg: BigVGAN2Config, input_sr: int = 16000, output_sr: int = 48000,
                 n_fft: int = 512, hop: int = 80, n_mels: int = 64, dtype=torch.float32, device=None):
        super().__init__()
        self.vocoder = BigVGAN2(voc_cfg, dtype, device)
        self.bwe_generator = BigVGAN2(bwe_cfg, dtype, device)
        self.mel_stft = MelSTFT(n_fft, hop, n_mels, input_sr, dtype, device)
        self.input_sr, self.output_sr, self.hop_length = input_sr, output_sr, hop

    @torch.no_grad()
    def forward(self, mel):
        x = self.vocoder(mel)
        L16 = x.shape[-1]
        out_len = L16 * self.output_sr // self.input_sr
        rem = L16 % self.hop_length
        if rem:
            x = torch.nn.functional.pad(x, (0, self.hop_length - rem))
        mel_bwe = self.mel_stft(x)                                        # [B, 2, 64, Tf]
        residual = self.bwe_generator(mel_bwe.permute(0, 1, 3, 2))
        skip = A.sinc_upsample(x, self.output_sr // self.input_sr)
        n = min(residual.shape[-1], skip.shape[-1])
        return (residual[..., :n] + skip[..., :n]).clamp(-1, 1)[..., :out_len]
