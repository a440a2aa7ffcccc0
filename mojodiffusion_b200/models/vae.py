"""LDM-style AutoencoderKL (decoder + encoder) in NHWC with the implicit-GEMM convolution, fused GroupNorm+SiLU and
tiled decode with overlap + feather. Factories give the SDXL / SD1.5 (4-ch), FLUX.1 / SD3 (16-ch) and FLUX.2 (32-ch)
variants (serenitymojo/models/vae/ldm_decoder.mojo:446-885, ldm_encoder.mojo:156-652; shared block kit
serenitymojo/models/vae/decoder2d.mojo:150-362; tiled decode serenitymojo/pipeline/flux_tiled_decode.mojo).
Parameter names are the LDM checkpoint keys (`decoder.up.3.block.0.conv1.weight`, `decoder.mid.attn_1.q.weight` ...),
weights are kept in checkpoint layout [Cout, Cin, KH, KW] and transposed once to the kernel's [Cout, KH, KW, Cin].
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import conv as C
from .layers import init_module_weights


@dataclass
class VAEConfig:
    in_channels: int = 3
    z_channels: int = 16
    ch: int = 128
    ch_mult: Tuple[int, ...] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    scale_factor: float = 0.3611
    shift_factor: float = 0.1159
    name: str = "flux-ae"


def flux_vae_config():
    return VAEConfig()


def sdxl_vae_config():
    return VAEConfig(z_channels=4, scale_factor=0.13025, shift_factor=0.0, name="sdxl-vae")


def sd3_vae_config():
    return VAEConfig(z_channels=16, scale_factor=1.5305, shift_factor=0.0609, name="sd3-vae")


def flux2_vae_config():
    return VAEConfig(z_channels=32, scale_factor=1.0, shift_factor=0.0, name="flux2-vae")


def tiny_vae_config():
    return VAEConfig(z_channels=4, ch=64, ch_mult=(1, 2), num_res_blocks=1, name="tiny-vae")


class Conv2d(nn.Module):
    def __init__(self, cin, cout, k=3, stride=1, padding=None, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.stride = stride
        self.padding = (k // 2) if padding is None else padding
        self.weight = nn.Parameter(torch.empty(cout, cin, k, k, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device))
        self._ohwi = None

    def ohwi(self):
        if self._ohwi is None or self._ohwi.device != self.weight.device or torch.is_grad_enabled():
            w = self.weight.permute(0, 2, 3, 1).contiguous()
            if torch.is_grad_enabled():
                return w
            self._ohwi = w
        return self._ohwi

    def forward(self, x, act=None, residual=None):
        return C.conv2d_nhwc(x, self.ohwi(), self.bias, self.stride, self.padding, act, residual)


class GroupNorm(nn.Module):
    def __init__(self, ch, groups=32, eps=1e-6, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.groups, self.eps = groups, eps
        self.weight = nn.Parameter(torch.ones(ch, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device))

    def forward(self, x, act=None):
        return C.group_norm_nhwc(x, self.weight, self.bias, self.groups, self.eps, act)


class ResnetBlock(nn.Module):
    def __init__(self, cin, cout, dtype, device, temb_ch: int = 0):
        super().__init__()
        self.norm1 = GroupNorm(cin, dtype=dtype, device=device)
        self.conv1 = Conv2d(cin, cout, 3, dtype=dtype, device=device)
        self.norm2 = GroupNorm(cout, dtype=dtype, device=device)
        self.conv2 = Conv2d(cout, cout, 3, dtype=dtype, device=device)
        if cin != cout:
            self.nin_shortcut = Conv2d(cin, cout, 1, dtype=dtype, device=device)

    def forward(self, x):
        h = self.conv1(self.norm1(x, act="silu"))
        skip = self.nin_shortcut(x) if hasattr(self, "nin_shortcut") else x
        return self.conv2(self.norm2(h, act="silu"), residual=skip)


class AttnBlock(nn.Module):
    """Single-head spatial self-attention (1x1 conv q/k/v/proj)."""

    def __init__(self, ch, dtype, device):
        super().__init__()
        self.norm = GroupNorm(ch, dtype=dtype, device=device)
        self.q, self.k, self.v, self.proj_out = [Conv2d(ch, ch, 1, dtype=dtype, device=device) for _ in range(4)]

    def forward(self, x):
        N, H, W, Cc = x.shape
        h = self.norm(x)
        q, k, v = [m(h).reshape(N, H * W, 1, Cc) for m in (self.q, self.k, self.v)]
        if Cc in (64, 128):
            o = ops.attention(q, k, v)
        else:                                   # head dim 512 of the standard AE: plain attention math (one layer)
            o = ops.reference.attention(q, k, v)
        return self.proj_out(o.reshape(N, H, W, Cc), residual=x)


class Upsample(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.conv = Conv2d(ch, ch, 3, dtype=dtype, device=device)

    def forward(self, x):
        return self.conv(C.upsample_nearest2x_nhwc(x))


class Downsample(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.conv = Conv2d(ch, ch, 3, stride=2, padding=0, dtype=dtype, device=device)

    def forward(self, x):
        from ..ops import native
        if native.use_native(x) and x.dtype == torch.bfloat16 and x.shape[1] % 2 == 0 and x.shape[2] % 2 == 0:
            # far-side padded stride-2 convolution = the "same" convolution sampled at the odd positions (native kernel)
            return C.conv2d_nhwc(x, self.conv.ohwi(), self.conv.bias, 2, 1, offset=1)
        x = torch.nn.functional.pad(x, (0, 0, 0, 1, 0, 1))          # NHWC: pad W and H on the far side
        return self.conv(x)


class _Level(nn.Module):
    pass


class Decoder(nn.Module):
    def __init__(self, cfg: VAEConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        n = len(cfg.ch_mult)
        bi = cfg.ch * cfg.ch_mult[-1]
        self.conv_in = Conv2d(cfg.z_channels, bi, 3, dtype=dtype, device=device)
        self.mid = _Level()
        self.mid.block_1 = ResnetBlock(bi, bi, dtype, device)
        self.mid.attn_1 = AttnBlock(bi, dtype, device)
        self.mid.block_2 = ResnetBlock(bi, bi, dtype, device)
        self.up = nn.ModuleList()
        levels = []
        for i in reversed(range(n)):
            lv = _Level()
            bo = cfg.ch * cfg.ch_mult[i]
            lv.block = nn.ModuleList()
            for _ in range(cfg.num_res_blocks + 1):
                lv.block.append(ResnetBlock(bi, bo, dtype, device))
                bi = bo
            if i != 0:
                lv.upsample = Upsample(bi, dtype, device)
            levels.insert(0, lv)
        self.up.extend(levels)
        self.norm_out = GroupNorm(bi, dtype=dtype, device=device)
        self.conv_out = Conv2d(bi, cfg.in_channels, 3, dtype=dtype, device=device)

    def forward(self, z):            # z: NHWC latent
        h = self.conv_in(z)
        h = self.mid.block_2(self.mid.attn_1(self.mid.block_1(h)))
        for i in reversed(range(len(self.up))):
            for blk in self.up[i].block:
                h = blk(h)
            if hasattr(self.up[i], "upsample"):
                h = self.up[i].upsample(h)
        return self.conv_out(self.norm_out(h, act="silu"))


class Encoder(nn.Module):
    def __init__(self, cfg: VAEConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        n = len(cfg.ch_mult)
        self.conv_in = Conv2d(cfg.in_channels, cfg.ch, 3, dtype=dtype, device=device)
        self.down = nn.ModuleList()
        bi = cfg.ch
        for i in range(n):
            lv = _Level()
            bo = cfg.ch * cfg.ch_mult[i]
            lv.block = nn.ModuleList()
            for _ in range(cfg.num_res_blocks):
                lv.block.append(ResnetBlock(bi, bo, dtype, device))
                bi = bo
            if i != n - 1:
                lv.downsample = Downsample(bi, dtype, device)
            self.down.append(lv)
        self.mid = _Level()
        self.mid.block_1 = ResnetBlock(bi, bi, dtype, device)
        self.mid.attn_1 = AttnBlock(bi, dtype, device)
        self.mid.block_2 = ResnetBlock(bi, bi, dtype, device)
        self.norm_out = GroupNorm(bi, dtype=dtype, device=device)
        self.conv_out = Conv2d(bi, 2 * cfg.z_channels, 3, dtype=dtype, device=device)

    def forward(self, x):
        h = self.conv_in(x)
        for lv in self.down:
            for blk in lv.block:
                h = blk(h)
            if hasattr(lv, "downsample"):
                h = lv.downsample(h)
        h = self.mid.block_2(self.mid.attn_1(self.mid.block_1(h)))
        return self.conv_out(self.norm_out(h, act="silu"))


class AutoencoderKL(nn.Module):
    """encode(image NCHW in [-1,1]) -> latent NCHW (scaled); decode(latent NCHW) -> image NCHW."""

    def __init__(self, cfg: VAEConfig, dtype=torch.bfloat16, device=None, with_encoder: bool = True):
        super().__init__()
        self.cfg = cfg
        self.decoder = Decoder(cfg, dtype, device)
        if with_encoder:
            self.encoder = Encoder(cfg, dtype, device)

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.cfg.ch_mult) - 1)

    def encode(self, img, sample: bool = True, generator=None):
        dt = self.decoder.conv_in.weight.dtype
        moments = self.encoder(img.permute(0, 2, 3, 1).to(dt)).float()
        mean, logvar = moments.chunk(2, dim=-1)
        z = mean
        if sample:
            std = torch.exp(0.5 * logvar.clamp(-30.0, 20.0))
            z = mean + std * torch.randn(mean.shape, generator=generator, device=mean.device)
        z = (z - self.cfg.shift_factor) * self.cfg.scale_factor
        return z.permute(0, 3, 1, 2)

    def decode(self, z):
        dt = self.decoder.conv_in.weight.dtype
        z = z.float() / self.cfg.scale_factor + self.cfg.shift_factor
        return self.decoder(z.permute(0, 2, 3, 1).to(dt)).permute(0, 3, 1, 2)

    @torch.no_grad()
    def tiled_decode(self, z, tile: int = 64, overlap: int = 16):
        """Decode latent tiles of `tile` x `tile` with `overlap` latent pixels of context, blending the seams with a
        linear feather (bounded activation memory for large images)."""
        B, Cz, H, W = z.shape
        f = self.spatial_factor
        if H <= tile and W <= tile:
            return self.decode(z)
        out = torch.zeros(B, self.cfg.in_channels, H * f, W * f, dtype=torch.float32, device=z.device)
        acc = torch.zeros(1, 1, H * f, W * f, dtype=torch.float32, device=z.device)
        step = tile - overlap
        ys = list(range(0, max(H - overlap, 1), step))
        xs = list(range(0, max(W - overlap, 1), step))
        for y0 in ys:
            for x0 in xs:
                y1, x1 = min(y0 + tile, H), min(x0 + tile, W)
                y0c, x0c = max(0, y1 - tile), max(0, x1 - tile)
                piece = self.decode(z[:, :, y0c:y1, x0c:x1]).float()
                ph, pw = piece.shape[-2:]
                ramp = overlap * f
                wy = torch.ones(ph, device=z.device)
                wx = torch.ones(pw, device=z.device)
                if ramp > 0:
                    r = torch.linspace(1.0 / ramp, 1.0, ramp, device=z.device)
                    if y0c > 0:
                        wy[:ramp] = r
                    if y1 < H:
                        wy[-ramp:] = r.flip(0)
                    if x0c > 0:
                        wx[:ramp] = r
                    if x1 < W:
                        wx[-ramp:] = r.flip(0)
                wgt = wy[:, None] * wx[None, :]
                out[:, :, y0c * f:y1 * f, x0c * f:x1 * f] += piece * wgt
                acc[:, :, y0c * f:y1 * f, x0c * f:x1 * f] += wgt
        return (out / acc.clamp_min(1e-6)).to(z.dtype if z.dtype != torch.float32 else torch.float32)

    def init_weights(self, seed: int = 0, std: float = 0.05):
        return init_module_weights(self, seed, std)


# ---- diffusers key layout, Z-Image and FLUX.2 / Klein variants ---------------------------------------------------------
def zimage_vae_config():
    """The Z-Image VAE is the 16-channel FLUX autoencoder (scale 0.3611, shift 0.1159, no post-quant convolution) stored
    under diffusers names (serenitymojo/models/vae/zimage_decoder.mojo:1-27)."""
    return VAEConfig(name="zimage-vae")


def klein_vae_config():
    return VAEConfig(z_channels=32, scale_factor=1.0, shift_factor=0.0, name="flux2-klein-vae")


_ATTN_LEAF = {"group_norm": "norm", "to_q": "q", "to_k": "k", "to_v": "v", "to_out.0": "proj_out", "query": "q", "key": "k", "value": "v",
              "proj_attn": "proj_out"}


def remap_diffusers_vae_keys(sd, n_levels: int = 4):
    """diffusers AutoencoderKL names -> the LDM names of this module. Decoder ``up_blocks.{g}`` run from the deepest level,
    LDM ``up.{n-1-g}`` stores them by resolution; ``resnets.{j}`` -> ``block.{j}``, ``upsamplers.0.conv`` ->
    ``upsample.conv``, ``downsamplers.0.conv`` -> ``downsample.conv``, ``conv_shortcut`` -> ``nin_shortcut``,
    ``mid_block.resnets.{0,1}`` -> ``mid.block_{1,2}``, ``mid_block.attentions.0.{group_norm,to_q,to_k,to_v,to_out.0}`` ->
    ``mid.attn_1.{norm,q,k,v,proj_out}`` with linear weights [C, C] reshaped to 1x1 convolutions, ``conv_norm_out`` ->
    ``norm_out``. Other keys (``quant_conv``, ``post_quant_conv``, ``bn.*``) pass through."""
    import re
    out = {}
    for k, v in sd.items():
        n = k
        m = re.match(r"(encoder|decoder)\.(.*)", k)
        if m:
            side, rest = m.group(1), m.group(2)
            rest = rest.replace("conv_norm_out.", "norm_out.").replace("conv_shortcut.", "nin_shortcut.")
            mm = re.match(r"up_blocks\.(\d+)\.resnets\.(\d+)\.(.*)", rest)
            if mm:
                rest = f"up.{n_levels - 1 - int(mm.group(1))}.block.{mm.group(2)}.{mm.group(3)}"
            elif (mm := re.match(r"up_blocks\.(\d+)\.upsamplers\.0\.(.*)", rest)):
                rest = f"up.{n_levels - 1 - int(mm.group(1))}.upsample.{mm.group(2)}"
            elif (mm := re.match(r"down_blocks\.(\d+)\.resnets\.(\d+)\.(.*)", rest)):
                rest = f"down.{mm.group(1)}.block.{mm.group(2)}.{mm.group(3)}"
            elif (mm := re.match(r"down_blocks\.(\d+)\.downsamplers\.0\.(.*)", rest)):
                rest = f"down.{mm.group(1)}.downsample.{mm.group(2)}"
            elif (mm := re.match(r"mid_block\.resnets\.(\d)\.(.*)", rest)):
                rest = f"mid.block_{int(mm.group(1)) + 1}.{mm.group(2)}"
            elif (mm := re.match(r"mid_block\.attentions\.0\.(.*)\.(weight|bias)", rest)):
                leaf = _ATTN_LEAF.get(mm.group(1), mm.group(1))
                rest = f"mid.attn_1.{leaf}.{mm.group(2)}"
                if mm.group(2) == "weight" and v.dim() == 2:
                    v = v[:, :, None, None]
            n = f"{side}.{rest}"
        out[n] = v
    return out


class KleinVAE(AutoencoderKL):
    """FLUX.2 / Klein autoencoder: 32 latent channels at 1/8 resolution, exchanged with the transformer as 128 packed
    channels at 1/16 (2 x 2 pixel-unshuffle, packed channel = (c * 2 + dy) * 2 + dx) normalised by a BatchNorm's running
    statistics (eps 1e-4, no affine part). decode: inverse BatchNorm -> unpack -> post_quant_conv -> decoder; encode:
    encoder -> quant_conv -> posterior mean -> pack -> BatchNorm
    (serenitymojo/models/vae/klein_decoder.mojo:36-96,207-256, klein_encoder.mojo:13-27)."""

    BN_EPS = 1e-4

    def __init__(self, cfg: Optional[VAEConfig] = None, dtype=torch.float32, device=None, with_encoder: bool = True):
        cfg = cfg or klein_vae_config()
        super().__init__(cfg, dtype, device, with_encoder)
        z = cfg.z_channels
        self.post_quant_conv = Conv2d(z, z, 1, dtype=dtype, device=device)
        if with_encoder:
            self.quant_conv = Conv2d(2 * z, 2 * z, 1, dtype=dtype, device=device)
        bn = nn.Module()
        bn.register_buffer("running_mean", torch.zeros(4 * z, dtype=torch.float32, device=device))
        bn.register_buffer("running_var", torch.ones(4 * z, dtype=torch.float32, device=device))
        self.bn = bn

    @property
    def spatial_factor(self) -> int:
        return 2 ** (len(self.cfg.ch_mult) - 1) * 2

    @staticmethod
    def pack(z):
        B, Cc, H, W = z.shape
        return z.reshape(B, Cc, H // 2, 2, W // 2, 2).permute(0, 1, 3, 5, 2, 4).reshape(B, Cc * 4, H // 2, W // 2)

    @staticmethod
    def unpack(zp):
        B, Cp, H, W = zp.shape
        return zp.reshape(B, Cp // 4, 2, 2, H, W).permute(0, 1, 4, 2, 5, 3).reshape(B, Cp // 4, H * 2, W * 2)

    def decode(self, zp):
        dt = self.decoder.conv_in.weight.dtype
        std = torch.sqrt(self.bn.running_var.float() + self.BN_EPS).view(1, -1, 1, 1)
        z = self.unpack(zp.float() * std + self.bn.running_mean.float().view(1, -1, 1, 1))
        h = self.post_quant_conv(z.permute(0, 2, 3, 1).to(dt))
        return self.decoder(h).permute(0, 3, 1, 2)

    def encode(self, img, sample: bool = False, generator=None):
        dt = self.decoder.conv_in.weight.dtype
        mom = self.quant_conv(self.encoder(img.permute(0, 2, 3, 1).to(dt))).float()
        mean, logvar = mom.chunk(2, dim=-1)
        z = mean
        if sample:
            z = mean + torch.exp(0.5 * logvar.clamp(-30.0, 20.0)) * torch.randn(mean.shape, generator=generator, device=mean.device)
        zp = self.pack(z.permute(0, 3, 1, 2))
        inv = torch.rsqrt(self.bn.running_var.float() + self.BN_EPS).view(1, -1, 1, 1)
        return (zp - self.bn.running_mean.float().view(1, -1, 1, 1)) * inv
