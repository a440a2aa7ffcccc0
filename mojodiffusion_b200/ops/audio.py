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


# ---- anti-aliased activation and resampling (BigVGAN-v2 / torchaudio semantics) ---------------------------------------
def kaiser_sinc_filter1d(cutoff: float, half_width: float, kernel_size: int) -> torch.Tensor:
    """Kaiser-windowed sinc low-pass FIR [kernel_size], normalised to unit DC gain (the ratio-2 filters of the
    anti-aliased activation use cutoff 0.5 / ratio, half width 0.6 / ratio, 12 taps)."""
    even = kernel_size % 2 == 0
    half = kernel_size // 2
    delta_f = 4 * half_width
    A_ = 2.285 * (half - 1) * math.pi * delta_f + 7.95
    beta = 0.1102 * (A_ - 8.7) if A_ > 50.0 else (0.5842 * (A_ - 21) ** 0.4 + 0.07886 * (A_ - 21.0) if A_ >= 21.0 else 0.0)
    window = torch.kaiser_window(kernel_size, beta=beta, periodic=False, dtype=torch.float64)
    t = (torch.arange(-half, half, dtype=torch.float64) + 0.5) if even else (torch.arange(kernel_size, dtype=torch.float64) - half)
    if cutoff == 0:
        return torch.zeros(kernel_size)
    f = 2 * cutoff * window * torch.sinc(2 * cutoff * t)
    return (f / f.sum()).float()


def activation1d(x: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor, up_filter: Optional[torch.Tensor] = None,
                 down_filter: Optional[torch.Tensor] = None, ratio: int = 2, log_scale: bool = True) -> torch.Tensor:
    """Anti-aliased SnakeBeta: upsample by ``ratio`` with a kaiser-sinc FIR (replicate pad 5, zero insert, 12-tap filter,
    gain ``ratio``, trim 15 / 15), apply the activation at the higher rate, low-pass and decimate back (replicate pad
    5 / 6, stride ``ratio``). Length is preserved. x [B, C, L]; alpha / beta [C]
    (serenitymojo/ops/activation1d.mojo:1-70)."""
    B, Cc, Lx = x.shape
    K = 12
    if up_filter is None:
        up_filter = kaiser_sinc_filter1d(0.5 / ratio, 0.6 / ratio, K)
    if down_filter is None:
        down_filter = kaiser_sinc_filter1d(0.5 / ratio, 0.6 / ratio, K)
    uf = up_filter.to(x.device, torch.float32).view(1, 1, K)
    df = down_filter.to(x.device, torch.float32).view(1, 1, K)
    xf = x.float().reshape(B * Cc, 1, Lx)
    pad = K // ratio - 1                                            # 5
    y = zero_insert1d(replicate_pad1d(xf, pad, pad), ratio)
    side = K - 1
    y = TF.conv1d(TF.pad(y, (side, side)), uf) * float(ratio)
    left = pad * ratio + (K - ratio) // 2                           # 15
    right = pad * ratio + (K - ratio + 1) // 2                      # 15
    y = y[..., left:y.shape[-1] - right]
    y = snake(y.reshape(B, Cc, -1), alpha, beta, log_scale).float().reshape(B * Cc, 1, -1)
    pl, pr = K // 2 - ratio // 2, K // 2 - ratio // 2 + (K % 2 == 0)  # 5, 6
    out = TF.conv1d(replicate_pad1d(y, pl, pr), df, stride=ratio)
    return out.reshape(B, Cc, -1).to(x.dtype)


def resample_hann(x: torch.Tensor, orig_freq: int, new_freq: int, rolloff: float = 0.99, lowpass_filter_width: int = 6) -> torch.Tensor:
    """Band-limited resampling as one strided convolution with a Hann-windowed sinc kernel bank (one phase per output sample
    of a period): the rule of torchaudio's ``sinc_interp_hann``. x [B, C, L] -> [B, C, ceil(L * new / orig)]
    (serenitymojo/ops/resample.mojo:1-40)."""
    g = math.gcd(int(orig_freq), int(new_freq))
    orig, new = int(orig_freq) // g, int(new_freq) // g
    if orig == new:
        return x
    base = min(orig, new) * rolloff
    width = int(math.ceil(lowpass_filter_width * orig / base))
    idx = torch.arange(-width, width + orig, dtype=torch.float64)[None, None] / orig
    t = (torch.arange(0, -new, -1, dtype=torch.float64)[:, None, None] / new + idx) * base
    t = t.clamp(-lowpass_filter_width, lowpass_filter_width)
    window = torch.cos(t * math.pi / lowpass_filter_width / 2) ** 2
    t = t * math.pi
    kern = torch.where(t == 0, torch.ones_like(t), torch.sin(t) / t) * window * (base / orig)       # [new, 1, K]
    B, Cc, Lx = x.shape
    xf = TF.pad(x.float().reshape(B * Cc, 1, Lx), (width, width + orig))
    y = TF.conv1d(xf, kern.float().to(x.device), stride=orig)                                      # [B*C, new, L/orig]
    y = y.transpose(1, 2).reshape(B, Cc, -1)
    return y[..., :int(math.ceil(new * Lx / orig))].to(x.dtype)


def sinc_upsample(x: torch.Tensor, ratio: int) -> torch.Tensor:
    """Integer-ratio band-limited upsampling (the skip path of the bandwidth-extension vocoder)."""
    return resample_hann(x, 1, ratio)
