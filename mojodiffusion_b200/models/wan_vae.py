"""Wan-family causal 3-D VAEs: the Wan2.1-style VAE that Qwen-Image uses (z = 16, base 96, x8 spatial / x4 temporal) and the
Wan2.2 high-compression VAE (z = 48, 2 x 2 pixel patches, x16 spatial / x4 temporal, parameter-free duplicate / average
shortcuts around every stage).

All 3-D convolutions are causal in time (``2 * pad`` frames on the left: zeros for Qwen-Image, optionally the repeated
first frame). The reference decodes frame chunks through a feature cache; a whole-sequence causal pass is the same
function, with two rules kept from the cache protocol: the first frame bypasses every temporal up/down-sampling
convolution, and the temporal up-sampling convolution never sees the first frame as history. A single latent frame
(image mode) therefore decodes to a single image, T latent frames to ``1 + 4 (T - 1)`` frames.

Per-channel latent statistics un-normalise (``z * std + mean``) before ``conv2`` and normalise after ``conv1``. Channel
RMS norms carry a ``gamma``; the middle attention is single-head over the pixels of each frame. Key names are the Wan
checkpoint's (``decoder.conv1``, ``decoder.middle.{0,1,2}``, ``decoder.upsamples.*``, ``decoder.head.{0,2}``, ``conv1``,
``conv2``), with ``remap_diffusers_wan_keys`` for the diffusers spelling Qwen-Image ships
(serenitymojo/models/vae/qwenimage_decoder.mojo:1-60, qwenimage_encoder.mojo, wan22_decoder.mojo:1011-1104,274-304,
wan22_vae_encoder.mojo). Convolutions run through torch (library path: one decode per image, not a hot loop).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as TF

from .layers import init_module_weights

QWEN_MEAN = (-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508, 0.4134, -0.0715, 0.5517, -0.3632, -0.1922,
             -0.9497, 0.2503, -0.2921)
QWEN_STD = (2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743, 3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253,
            2.8251, 1.9160)
WAN22_MEAN = (-0.2289, -0.0052, -0.1323, -0.2339, -0.2799, 0.0174, 0.1838, 0.1557, -0.1382, 0.0542, 0.2813, 0.0891, 0.1570,
              -0.0098, 0.0375, -0.1825, -0.2246, -0.1207, -0.0698, 0.5109, 0.2665, -0.2108, -0.2158, 0.2502, -0.2055, -0.0322,
              0.1109, 0.1567, -0.0729, 0.0899, -0.2799, -0.1230, -0.0313, -0.1649, 0.0117, 0.0723, -0.2839, -0.2083, -0.0520,
              0.3748, 0.0152, 0.1957, 0.1433, -0.2944, 0.3573, -0.0548, -0.1681, -0.0667)
WAN22_STD = (0.4765, 1.0364, 0.4514, 1.1677, 0.5313, 0.4990, 0.4818, 0.5013, 0.8158, 1.0344, 0.5894, 1.0901, 0.6885, 0.6165,
             0.8454, 0.4978, 0.5759, 0.3523, 0.7135, 0.6804, 0.5833, 1.4146, 0.8986, 0.5659, 0.7069, 0.5338, 0.4889, 0.4917,
             0.4069, 0.4999, 0.6866, 0.4093, 0.5709, 0.6065, 0.6415, 0.4944, 0.5726, 1.2042, 0.5458, 1.6887, 0.3971, 1.0600,
             0.3943, 0.5537, 0.5444, 0.4089, 0.7468, 0.7744)


@dataclass
class WanVAEConfig:
    variant: str = "wan21"                       # "wan21" (Qwen-Image) or "wan22" (high compression)
    z_dim: int = 16
    enc_dim: int = 96
    dec_dim: int = 96
    dim_mult: Tuple[int, ...] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    temporal_down: Tuple[bool, ...] = (False, True, True)
    pad_mode: str = "zero"                       # left temporal padding: "zero" or "replicate"
    patch: int = 1                               # pixel patch folded into channels (Wan2.2: 2)
    mean: Tuple[float, ...] = QWEN_MEAN
    std: Tuple[float, ...] = QWEN_STD
    name: str = "qwen-image-vae"

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.dim_mult) - 1) * self.patch

    @property
    def temporal_factor(self) -> int:
        return 2 ** sum(self.temporal_down)


def qwen_image_vae_config() -> WanVAEConfig:
    return WanVAEConfig()


def wan22_vae_config() -> WanVAEConfig:
    return WanVAEConfig(variant="wan22", z_dim=48, enc_dim=160, dec_dim=256, patch=2, mean=WAN22_MEAN, std=WAN22_STD, name="wan2.2-vae")


def tiny_wan_vae_config(variant: str = "wan21") -> WanVAEConfig:
    if variant == "wan22":
        return WanVAEConfig(variant="wan22", z_dim=6, enc_dim=8, dec_dim=8, dim_mult=(1, 2, 2), num_res_blocks=1, temporal_down=(True, True),
                            patch=2, mean=WAN22_MEAN[:6], std=WAN22_STD[:6], name="tiny-wan22-vae")
    return WanVAEConfig(z_dim=4, enc_dim=8, dec_dim=8, dim_mult=(1, 2, 2), num_res_blocks=1, temporal_down=(True, True),
                        mean=QWEN_MEAN[:4], std=QWEN_STD[:4], name="tiny-wan21-vae")


class CausalConv3d(nn.Conv3d):
    """Conv3d over [B, C, T, H, W]; symmetric spatial padding, all temporal padding on the left."""

    def __init__(self, cin, cout, k, stride=1, padding=0, pad_mode="zero", dtype=torch.float32, device=None):
        k = (k, k, k) if isinstance(k, int) else tuple(k)
        p = (padding,) * 3 if isinstance(padding, int) else tuple(padding)
        super().__init__(cin, cout, k, stride=stride, padding=0, dtype=dtype, device=device)
        self._pad = (p[2], p[2], p[1], p[1], 2 * p[0], 0)
        self.pad_mode = pad_mode

    def forward(self, x, left=None):
        """``left``: frames to use as temporal history instead of padding (same channel count)."""
        pw = self._pad
        if left is not None:
            x = torch.cat((left[:, :, -pw[4]:], x), dim=2) if pw[4] else x
            pad = (pw[0], pw[1], pw[2], pw[3], max(0, pw[4] - left.shape[2]), 0)
        else:
            pad = pw
        if any(pad):
            if self.pad_mode == "replicate" and pad[4] and left is None:
                x = torch.cat((x[:, :, :1].expand(-1, -1, pad[4], -1, -1), x), dim=2)
                pad = (pad[0], pad[1], pad[2], pad[3], 0, 0)
            x = TF.pad(x, pad)
        return super().forward(x)


class RMSNormC(nn.Module):
    """x / sqrt(mean_c x^2) * gamma over the channel dim of [B, C, ...]."""

    def __init__(self, dim, images: bool, dtype, device):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones((dim, 1, 1) if images else (dim, 1, 1, 1), dtype=dtype, device=device))

    def forward(self, x):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(dim=1, keepdim=True) + 1e-12)
        return (y * self.gamma.float()).to(x.dtype)


class ResidualBlock(nn.Module):
    def __init__(self, cin, cout, pad_mode, dtype, device):
        super().__init__()
        self.residual = nn.ModuleList([RMSNormC(cin, False, dtype, device), nn.SiLU(), CausalConv3d(cin, cout, 3, padding=1, pad_mode=pad_mode, dtype=dtype, device=device),
                                       RMSNormC(cout, False, dtype, device), nn.SiLU(), nn.Dropout(0.0),
                                       CausalConv3d(cout, cout, 3, padding=1, pad_mode=pad_mode, dtype=dtype, device=device)])
        self.shortcut = CausalConv3d(cin, cout, 1, dtype=dtype, device=device) if cin != cout else nn.Identity()

    def forward(self, x):
        h = x
        for layer in self.residual:
            h = layer(h)
        return h + self.shortcut(x)


class AttentionBlock(nn.Module):
    """Single-head attention over the pixels of every frame."""

    def __init__(self, dim, dtype, device):
        super().__init__()
        self.norm = RMSNormC(dim, True, dtype, device)
        self.to_qkv = nn.Conv2d(dim, dim * 3, 1, dtype=dtype, device=device)
        self.proj = nn.Conv2d(dim, dim, 1, dtype=dtype, device=device)

    def forward(self, x):
        B, Cc, T, H, W = x.shape
        y = x.permute(0, 2, 1, 3, 4).reshape(B * T, Cc, H, W)
        q, k, v = self.to_qkv(self.norm(y)).reshape(B * T, 1, 3 * Cc, H * W).permute(0, 1, 3, 2).chunk(3, dim=-1)
        o = TF.scaled_dot_product_attention(q, k, v)
        o = self.proj(o.squeeze(1).permute(0, 2, 1).reshape(B * T, Cc, H, W))
        return x + o.reshape(B, T, Cc, H, W).permute(0, 2, 1, 3, 4)


class Resample(nn.Module):
    """mode: upsample2d / upsample3d / downsample2d / downsample3d. ``halve``: the Wan2.1 up-sampler halves the channels
    in its 2-D convolution, the Wan2.2 one keeps them."""

    def __init__(self, dim, mode, halve: bool, pad_mode, dtype, device):
        super().__init__()
        self.mode = mode
        if mode.startswith("upsample"):
            self.resample = nn.ModuleList([nn.Upsample(scale_factor=(2.0, 2.0), mode="nearest-exact"),
                                           nn.Conv2d(dim, dim // 2 if halve else dim, 3, padding=1, dtype=dtype, device=device)])
            if mode == "upsample3d":
                self.time_conv = CausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0), pad_mode="zero", dtype=dtype, device=device)
        else:
            self.resample = nn.ModuleList([nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=2, dtype=dtype, device=device)])
            if mode == "downsample3d":
                self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0), dtype=dtype, device=device)

    def forward(self, x):
        B, Cc, T, H, W = x.shape
        if self.mode == "upsample3d" and T > 1:
            # the first frame passes through; later frames double, with zero history before frame 1
            rest = self.time_conv(x[:, :, 1:])
            rest = rest.reshape(B, 2, Cc, T - 1, H, W).permute(0, 2, 3, 1, 4, 5).reshape(B, Cc, 2 * (T - 1), H, W)
            x = torch.cat((x[:, :, :1], rest), dim=2)
            T = x.shape[2]
        y = x.permute(0, 2, 1, 3, 4).reshape(B * T, Cc, H, W)
        for layer in self.resample:
            y = layer(y)
        y = y.reshape(B, T, *y.shape[1:]).permute(0, 2, 1, 3, 4)
        if self.mode == "downsample3d" and T > 1:
            # first frame passes through; every later output frame sees (previous, two new) frames
            y = torch.cat((y[:, :, :1], self.time_conv(y)), dim=2)
        return y


def dup_up3d(x, cout, ft, fs, first_chunk=True):
    """Parameter-free up-sampling shortcut: channels repeated, then folded out into (time, height, width) factors."""
    B, Cc, T, H, W = x.shape
    rep = cout * ft * fs * fs // Cc
    y = x.repeat_interleave(rep, dim=1).reshape(B, cout, ft, fs, fs, T, H, W)
    y = y.permute(0, 1, 5, 2, 6, 3, 7, 4).reshape(B, cout, T * ft, H * fs, W * fs)
    return y[:, :, ft - 1:] if first_chunk else y


def avg_down3d(x, cout, ft, fs):
    """Parameter-free down-sampling shortcut: (time, height, width) factors folded into channels, then group means."""
    B, Cc, T, H, W = x.shape
    pad_t = (ft - T % ft) % ft
    if pad_t:
        x = TF.pad(x, (0, 0, 0, 0, pad_t, 0))
        T += pad_t
    y = x.reshape(B, Cc, T // ft, ft, H // fs, fs, W // fs, fs).permute(0, 1, 3, 5, 7, 2, 4, 6)
    y = y.reshape(B, Cc * ft * fs * fs, T // ft, H // fs, W // fs)
    g = Cc * ft * fs * fs // cout
    return y.reshape(B, cout, g, T // ft, H // fs, W // fs).mean(dim=2)


class _Stage22(nn.Module):
    """Wan2.2 stage: residual blocks (+ resample) with a parameter-free shortcut added around the whole stage."""

    def __init__(self, cin, cout, n_blocks, temporal, resample, up: bool, pad_mode, dtype, device):
        super().__init__()
        blocks = []
        ch = cin
        for _ in range(n_blocks):
            blocks.append(ResidualBlock(ch, cout, pad_mode, dtype, device))
            ch = cout
        if resample:
            mode = ("upsample" if up else "downsample") + ("3d" if temporal else "2d")
            blocks.append(Resample(cout, mode, False, pad_mode, dtype, device))
        name = "upsamples" if up else "downsamples"
        setattr(self, name, nn.ModuleList(blocks))
        self._name, self.up, self.resample, self.ft, self.cout = name, up, resample, 2 if temporal else 1, cout

    def forward(self, x):
        h = x
        for b in getattr(self, self._name):
            h = b(h)
        if not self.resample:
            return h if self.up else h + avg_down3d(x, self.cout, 1, 1)
        if self.up:
            return h + dup_up3d(x, self.cout, self.ft, 2, True)
        sc = avg_down3d(x, self.cout, self.ft, 2)
        return h + sc[:, :, -h.shape[2]:]


class Decoder3d(nn.Module):
    def __init__(self, cfg: WanVAEConfig, dtype, device):
        super().__init__()
        pm = cfg.pad_mode
        dims = [cfg.dec_dim * u for u in [cfg.dim_mult[-1]] + list(cfg.dim_mult[::-1])]
        t_up = list(cfg.temporal_down[::-1])
        self.conv1 = CausalConv3d(cfg.z_dim, dims[0], 3, padding=1, pad_mode=pm, dtype=dtype, device=device)
        self.middle = nn.ModuleList([ResidualBlock(dims[0], dims[0], pm, dtype, device), AttentionBlock(dims[0], dtype, device),
                                     ResidualBlock(dims[0], dims[0], pm, dtype, device)])
        ups = []
        n_stage = len(cfg.dim_mult)
        if cfg.variant == "wan22":
            for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
                last = i == n_stage - 1
                ups.append(_Stage22(cin, cout, cfg.num_res_blocks + 1, (not last) and t_up[i], not last, True, pm, dtype, device))
        else:
            for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
                if i in (1, 2, 3):
                    cin = cin // 2                       # the previous up-sampler halved the channels
                for _ in range(cfg.num_res_blocks + 1):
                    ups.append(ResidualBlock(cin, cout, pm, dtype, device))
                    cin = cout
                if i != n_stage - 1:
                    ups.append(Resample(cout, "upsample3d" if t_up[i] else "upsample2d", True, pm, dtype, device))
        self.upsamples = nn.ModuleList(ups)
        out_ch = 3 * cfg.patch * cfg.patch
        self.head = nn.ModuleList([RMSNormC(dims[-1], False, dtype, device), nn.SiLU(),
                                   CausalConv3d(dims[-1], out_ch, 3, padding=1, pad_mode=pm, dtype=dtype, device=device)])

    def forward(self, z):
        x = self.conv1(z)
        for m in self.middle:
            x = m(x)
        for u in self.upsamples:
            x = u(x)
        for h in self.head:
            x = h(x)
        return x


class Encoder3d(nn.Module):
    def __init__(self, cfg: WanVAEConfig, dtype, device):
        super().__init__()
        pm = cfg.pad_mode
        dims = [cfg.enc_dim * u for u in [1] + list(cfg.dim_mult)]
        n_stage = len(cfg.dim_mult)
        self.conv1 = CausalConv3d(3 * cfg.patch * cfg.patch, dims[0], 3, padding=1, pad_mode=pm, dtype=dtype, device=device)
        downs = []
        if cfg.variant == "wan22":
            for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
                last = i == n_stage - 1
                downs.append(_Stage22(cin, cout, cfg.num_res_blocks, (not last) and cfg.temporal_down[i], not last, False, pm, dtype, device))
        else:
            for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
                for _ in range(cfg.num_res_blocks):
                    downs.append(ResidualBlock(cin, cout, pm, dtype, device))
                    cin = cout
                if i != n_stage - 1:
                    downs.append(Resample(cout, "downsample3d" if cfg.temporal_down[i] else "downsample2d", False, pm, dtype, device))
        self.downsamples = nn.ModuleList(downs)
        self.middle = nn.ModuleList([ResidualBlock(dims[-1], dims[-1], pm, dtype, device), AttentionBlock(dims[-1], dtype, device),
                                     ResidualBlock(dims[-1], dims[-1], pm, dtype, device)])
        self.head = nn.ModuleList([RMSNormC(dims[-1], False, dtype, device), nn.SiLU(),
                                   CausalConv3d(dims[-1], 2 * cfg.z_dim, 3, padding=1, pad_mode=pm, dtype=dtype, device=device)])

    def forward(self, x):
        x = self.conv1(x)
        for d in self.downsamples:
            x = d(x)
        for m in self.middle:
            x = m(x)
        for h in self.head:
            x = h(x)
        return x


def patchify(x, p: int):
    if p == 1:
        return x
    B, Cc, T, H, W = x.shape
    return x.reshape(B, Cc, T, H // p, p, W // p, p).permute(0, 1, 6, 4, 2, 3, 5).reshape(B, Cc * p * p, T, H // p, W // p)


def unpatchify(x, p: int):
    if p == 1:
        return x
    B, Cp, T, H, W = x.shape
    Cc = Cp // (p * p)
    return x.reshape(B, Cc, p, p, T, H, W).permute(0, 1, 4, 5, 3, 6, 2).reshape(B, Cc, T, H * p, W * p)


class WanVAE(nn.Module):
    """encode(video [B, 3, T, H, W] in [-1, 1]) -> normalised latent [B, z, 1 + (T-1)/4, H/f, W/f]; decode is the inverse.
    4-D inputs are images (T = 1) and come back 4-D."""

    def __init__(self, cfg: WanVAEConfig, dtype=torch.float32, device=None, with_encoder: bool = True):
        super().__init__()
        self.cfg = cfg
        self.decoder = Decoder3d(cfg, dtype, device)
        self.conv2 = CausalConv3d(cfg.z_dim, cfg.z_dim, 1, dtype=dtype, device=device)
        if with_encoder:
            self.encoder = Encoder3d(cfg, dtype, device)
            self.conv1 = CausalConv3d(2 * cfg.z_dim, 2 * cfg.z_dim, 1, dtype=dtype, device=device)
        self.register_buffer("latent_mean", torch.tensor(cfg.mean, dtype=torch.float32, device=device).view(1, -1, 1, 1, 1), persistent=False)
        self.register_buffer("latent_std", torch.tensor(cfg.std, dtype=torch.float32, device=device).view(1, -1, 1, 1, 1), persistent=False)

    @torch.no_grad()
    def decode(self, z):
        image = z.dim() == 4
        if image:
            z = z.unsqueeze(2)
        dt = self.conv2.weight.dtype
        x = (z.float() * self.latent_std + self.latent_mean).to(dt)
        x = unpatchify(self.decoder(self.conv2(x)), self.cfg.patch).clamp(-1.0, 1.0)
        return x.squeeze(2) if image else x

    @torch.no_grad()
    def encode(self, x, sample: bool = False, generator=None):
        image = x.dim() == 4
        if image:
            x = x.unsqueeze(2)
        dt = self.conv2.weight.dtype
        mom = self.conv1(self.encoder(patchify(x.to(dt), self.cfg.patch))).float()
        mu, logvar = mom.chunk(2, dim=1)
        if sample:
            mu = mu + torch.exp(0.5 * logvar.clamp(-30.0, 20.0)) * torch.randn(mu.shape, generator=generator, dtype=mu.dtype).to(mu.device)
        z = (mu - self.latent_mean) / self.latent_std
        return z.squeeze(2) if image else z

    def init_weights(self, seed: int = 0, std: float = 0.05):
        init_module_weights(self, seed, std)
        with torch.no_grad():
            for n, p in self.named_parameters():
                if n.endswith("gamma"):
                    p.fill_(1.0)
        return self


_RESNET_LEAF = {"norm1": "residual.0", "conv1": "residual.2", "norm2": "residual.3", "conv2": "residual.6", "conv_shortcut": "shortcut"}


def remap_diffusers_wan_keys(sd: Dict[str, torch.Tensor], num_res_blocks: int = 2) -> Dict[str, torch.Tensor]:
    """diffusers AutoencoderKLQwenImage names -> the Wan checkpoint names this module uses: ``conv_in`` -> ``conv1``,
    ``mid_block.resnets.{0,1}`` / ``attentions.0`` -> ``middle.{0,2}`` / ``middle.1``, ``up_blocks.{g}.resnets.{j}`` ->
    ``upsamples.{g * (n + 2) + j}``, ``up_blocks.{g}.upsamplers.0`` -> ``upsamples.{g * (n + 2) + n + 1}``,
    ``down_blocks.{i}`` -> ``downsamples.{i}``, ``norm_out`` / ``conv_out`` -> ``head.0`` / ``head.2``,
    ``quant_conv`` / ``post_quant_conv`` -> ``conv1`` / ``conv2``; inside a resnet ``norm1, conv1, norm2, conv2,
    conv_shortcut`` -> ``residual.{0,2,3,6}, shortcut``."""
    import re
    per = num_res_blocks + 2
    out = {}

    def resnet_leaf(rest: str) -> str:
        head, _, tail = rest.partition(".")
        return _RESNET_LEAF[head] + "." + tail if head in _RESNET_LEAF else rest

    for k, v in sd.items():
        if k.startswith("post_quant_conv."):
            n = "conv2." + k.split(".", 1)[1]
        elif k.startswith("quant_conv."):
            n = "conv1." + k.split(".", 1)[1]
        else:
            side, rest = k.split(".", 1)
            m = re.match(r"mid_block\.resnets\.(\d)\.(.*)", rest)
            if rest.startswith("conv_in."):
                n = f"{side}.conv1." + rest[len("conv_in."):]
            elif rest.startswith("norm_out."):
                n = f"{side}.head.0." + rest[len("norm_out."):]
            elif rest.startswith("conv_out."):
                n = f"{side}.head.2." + rest[len("conv_out."):]
            elif m:
                n = f"{side}.middle.{2 * int(m.group(1))}." + resnet_leaf(m.group(2))
            elif rest.startswith("mid_block.attentions.0."):
                n = f"{side}.middle.1." + rest[len("mid_block.attentions.0."):]
            elif (m := re.match(r"up_blocks\.(\d+)\.resnets\.(\d+)\.(.*)", rest)):
                n = f"{side}.upsamples.{int(m.group(1)) * per + int(m.group(2))}." + resnet_leaf(m.group(3))
            elif (m := re.match(r"up_blocks\.(\d+)\.upsamplers\.0\.(.*)", rest)):
                n = f"{side}.upsamples.{int(m.group(1)) * per + per - 1}." + m.group(2)
            elif (m := re.match(r"down_blocks\.(\d+)\.(.*)", rest)):
                n = f"{side}.downsamples.{m.group(1)}." + resnet_leaf(m.group(2))
            else:
                n = k
        out[n] = v
    return out
