"""1-D convolution family, STFT / inverse STFT and the small ops of a neural vocoder.

conv1d runs as the NHWC implicit-GEMM convolution with a height of 1 when shapes allow (channels a multiple of 8, stride
and dilation 1); other cases and transposed convolutions go through torch (library path) until they matter for a
benchmark. Transposed convolution is also available in its zero-insert form (insert stride-1 zeros, pad, convolve with
the flipped kernel), which is how a vocoder upsampler maps onto the plain conv kernel
(serenitymojo/ops/conv1d.mojo:177-330,390-450,516-700; serenitymojo/models/vocoder/ltx2_stft.mojo; audio/wav.mojo)."""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as TF

from . import conv as C
from . import native


def conv1d(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, stride: int = 1, padding: int = 0,
           dilation: int = 1, groups: int = 1) -> torch.Tensor:
    """x [B, Cin, T], w [Cout, Cin/groups, K] -> [B, Cout, T']."""
    Cout, Cin_g, K = w.shape
    fast = (native.use_native(x) and x.dtype == torch.bfloat16 and stride == 1 and dilation == 1 and groups == 1
            and Cin_g % 8 == 0 and Cout % 8 == 0 and not torch.is_grad_enabled())
    if fast:
        xn = x.permute(0, 2, 1).unsqueeze(1).contiguous()                 # [B, 1, T, Cin] NHWC with H = 1
        wn = w.permute(0, 2, 1).unsqueeze(1).contiguous()                 # [Cout, 1, K, Cin]
        y = C.conv2d_nhwc(xn, wn, b, padding=(0, padding))
        return y.squeeze(1).permute(0, 2, 1)
    return TF.conv1d(x, w, b, stride, padding, dilation, groups)


def zero_insert1d(x: torch.Tensor, stride: int) -> torch.Tensor:
    """[B, C, T] -> [B, C, (T-1)*stride + 1] with stride-1 zeros between samples."""
    if stride == 1:
        return x
    B, Cc, T = x.shape
    out = x.new_zeros(B, Cc, (T - 1) * stride + 1)
    out[..., ::stride] = x
    return out


def replicate_pad1d(x: torch.Tensor, left: int, right: int) -> torch.Tensor:
    return TF.pad(x, (left, right), mode="replicate")


def conv_transpose1d(x, w, b=None, stride: int = 1, padding: int = 0, output_padding: int = 0, zero_insert: bool = False):
    """x [B, Cin, T], w [Cin, Cout, K]. ``zero_insert=True`` evaluates it as zero-insert + pad + plain conv with the
    flipped, transposed kernel (identical result)."""
    if not zero_insert:
        return TF.conv_transpose1d(x, w, b, stride, padding, output_padding)
    K = w.shape[-1]
    xz = zero_insert1d(x, stride)
    xz = TF.pad(xz, (K - 1 - padding, K - 1 - padding + output_padding))
    wf = w.flip(-1).permute(1, 0, 2).contiguous()                        # [Cout, Cin, K]
    return conv1d(xz, wf, b)


def snake(x: torch.Tensor, alpha: torch.Tensor, beta: Optional[torch.Tensor] = None, log_scale: bool = True) -> torch.Tensor:
    """Snake / SnakeBeta activation of BigVGAN-style vocoders: x + sin(alpha x)^2 / beta, per channel."""
    a = alpha.float().exp() if log_scale else alpha.float()
    bt = a if beta is None else (beta.float().exp() if log_scale else beta.float())
    a, bt = a.view(1, -1, 1), bt.view(1, -1, 1)
    xf = x.float()
    return (xf + torch.sin(a * xf) ** 2 / (bt + 1e-9)).to(x.dtype)


def stft(x: torch.Tensor, n_fft: int, hop: int, win_length: Optional[int] = None, center: bool = True):
    """x [B, T] -> (magnitude [B, F, N], phase [B, F, N]) with a Hann window."""
    win_length = win_length or n_fft
    window = torch.hann_window(win_length, device=x.device, dtype=torch.float32)
    spec = torch.stft(x.float(), n_fft, hop, win_length, window, center=center, return_complex=True)
    return spec.abs(), torch.angle(spec)


def istft(mag: torch.Tensor, phase: torch.Tensor, n_fft: int, hop: int, win_length: Optional[int] = None, center: bool = True,
          length: Optional[int] = None):
    win_length = win_length or n_fft
    window = torch.hann_window(win_length, device=mag.device, dtype=torch.float32)
    spec = torch.polar(mag.float(), phase.float())
    return torch.istft(spec, n_fft, hop, win_length, window, center=center, length=length)


def mel_filterbank(n_mels: int, n_fft: int, sample_rate: int, f_min: float = 0.0, f_max: Optional[float] = None) -> torch.Tensor:
    """Slaney-style triangular mel filters [n_mels, n_fft/2 + 1]."""
    f_max = f_max or sample_rate / 2
    hz2mel = lambda f: 2595.0 * math.log10(1.0 + f / 700.0)
    mel2hz = lambda m: 700.0 * (10.0 ** (m / 2595.0) - 1.0)
    mels = torch.linspace(hz2mel(f_min), hz2mel(f_max), n_mels + 2)
    hz = torch.tensor([mel2hz(float(m)) for m in mels])
    bins = torch.linspace(0, sample_rate / 2, n_fft // 2 + 1)
    fb = torch.zeros(n_mels, n_fft // 2 + 1)
    for i in range(n_mels):
        lo, ce, hi = hz[i], hz[i + 1], hz[i + 2]
        up = (bins - lo) / (ce - lo)
        down = (hi - bins) / (hi - ce)
        fb[i] = torch.clamp(torch.minimum(up, down), min=0.0)
    return fb


def log_mel(x: torch.Tensor, n_fft: int, hop: int, n_mels: int, sample_rate: int, eps: float = 1e-5) -> torch.Tensor:
    mag, _ = stft(x, n_fft, hop)
    fb = mel_filterbank(n_mels, n_fft, sample_rate).to(x.device)
    return torch.log(torch.clamp(fb @ mag, min=eps))
