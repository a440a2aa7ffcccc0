"""Z-Image L2P: the Z-Image single-stream trunk run directly on RGB pixels (no VAE) with a small U-Net pixel head.

* 16 x 16 pixel patches (768 values in (row, column, channel) order) enter through ``all_x_embedder.16-1``; captions,
  timestep embedding, the two refiner stacks and the 30 main blocks are the Z-Image ones (width 3840, 30 heads of 128,
  tanh gates, sandwich RMSNorms) except that rotary pairs are interleaved; the model timestep is ``(1 - sigma) * 1000``;
* there is no final layer: the hidden image tokens become a feature map [B, 3840, H / 16, W / 16];
* ``local_decoder``: a four-level U-Net over the NOISY image (3 -> 64 -> 128 -> 256 -> 512 channels, 3 x 3 convolutions with
  SiLU and 2 x 2 max pooling); at the bottom the feature map is concatenated and mixed by a 1 x 1 convolution; the way up is
  nearest-neighbour 2 x upsampling + 3 x 3 convolution, concatenation with the skip and a 3 x 3 convolution with SiLU;
  a 1 x 1 convolution gives 3 channels. The model's prediction is the NEGATED head output.

Sampling: sigma_i = shift * t / (1 + (shift - 1) * t) with t = 1 - i / steps (shift 3, 30 steps), guidance
``uncond + s * (cond - uncond)`` (s = 2), Euler ``x += (sigma_next - sigma) * prediction``.

Behaviour: serenitymojo/models/dit/zimage_l2p_contract.mojo:17-45,69-107 (sizes, schedule),
serenitymojo/models/dit/zimage_l2p_dit.mojo:137-180 (patch order), :427-570 (block),
serenitymojo/models/dit/zimage_l2p_local_decoder.mojo:246-531 (pixel head),
serenitymojo/pipeline/zimage_l2p_pipeline_512_multistep.mojo:385-463 (forward order, sign, guidance, Euler step).
Checkpoint names are the reference's (``all_x_embedder.16-1``, ``layers.N...``, ``local_decoder.enc1.0``, ``local_decoder.up4.1``,
``local_decoder.out_conv``); convolution weights are stored [out, kh, kw, in] here (``remap_l2p_keys`` permutes).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import conv as C
from .single_dit import SingleDiTConfig, SingleStreamDiT


def zimage_l2p_config() -> SingleDiTConfig:
    return SingleDiTConfig(in_channels=768, patch_key="16-1", rope_interleaved=True, final_layer=False, name="zimage-l2p")


def tiny_zimage_l2p_config() -> SingleDiTConfig:
    return SingleDiTConfig(in_channels=768, hidden=256, heads=4, head_dim=64, depth=2, depth_noise_refiner=1,
                           depth_context_refiner=1, cap_dim=128, mlp_hidden=512, axes_dim=(16, 24, 24), adaln_dim=64,
                           patch_key="16-1", rope_interleaved=True, final_layer=False, name="tiny-zimage-l2p")


def l2p_sigmas(steps: int, shift: float = 3.0) -> List[float]:
    if steps <= 0:
        raise ValueError("l2p_sigmas: steps must be positive")
    out = []
    for i in range(steps):
        t = 1.0 - i / steps
        out.append(shift * t / (1.0 + (shift - 1.0) * t))
    return out + [0.0]


def patchify_pixels(x: torch.Tensor, p: int) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H / p)(W / p), p * p * C] with (row in patch, column in patch, channel) order."""
    B, Cn, H, W = x.shape
    return x.reshape(B, Cn, H // p, p, W // p, p).permute(0, 2, 4, 3, 5, 1).reshape(B, (H // p) * (W // p), p * p * Cn)


class _Conv(nn.Module):
    """NHWC convolution parameters, weight [out, k, k, in]."""

    def __init__(self, cin, cout, k, dtype, device):
        super().__init__()
        self.k = k
        self.weight = nn.Parameter(torch.empty(cout, k, k, cin, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device))

    def forward(self, x, act=None):
        return C.conv2d_nhwc(x, self.weight, self.bias, 1, self.k // 2, act)


def _stage(conv: _Conv, index: str) -> nn.ModuleDict:
    return nn.ModuleDict({index: conv})


class LocalDecoder(nn.Module):
    def __init__(self, feat_dim: int, channels: Tuple[int, int, int, int] = (64, 128, 256, 512), pixel_channels: int = 3,
                 dtype=torch.bfloat16, device=None):
        super().__init__()
        c1, c2, c3, c4 = channels
        mk = lambda a, b, k=3: _Conv(a, b, k, dtype, device)
        self.enc1, self.enc2 = _stage(mk(pixel_channels, c1), "0"), _stage(mk(c1, c2), "0")
        self.enc3, self.enc4 = _stage(mk(c2, c3), "0"), _stage(mk(c3, c4), "0")
        self.bottleneck = _stage(mk(c4 + feat_dim, c4, 1), "0")
        self.up4, self.dec4 = _stage(mk(c4, c4), "1"), _stage(mk(2 * c4, c3), "0")
        self.up3, self.dec3 = _stage(mk(c3, c3), "1"), _stage(mk(2 * c3, c2), "0")
        self.up2, self.dec2 = _stage(mk(c2, c2), "1"), _stage(mk(2 * c2, c1), "0")
        self.up1, self.dec1 = _stage(mk(c1, c1), "1"), _stage(mk(2 * c1, c1), "0")
        self.out_conv = mk(c1, pixel_channels, 1)

    def forward(self, noisy_nhwc: torch.Tensor, feat_nhwc: torch.Tensor) -> torch.Tensor:
        """noisy [B, H, W, 3], feature map [B, H / 16, W / 16, feat_dim] -> [B, H, W, 3]."""
        pool = lambda v: torch.nn.functional.max_pool2d(v.permute(0, 3, 1, 2), 2).permute(0, 2, 3, 1).contiguous()
        up = lambda v: v.repeat_interleave(2, 1).repeat_interleave(2, 2)
        e1 = self.enc1["0"](noisy_nhwc, "silu")
        e2 = self.enc2["0"](pool(e1), "silu")
        e3 = self.enc3["0"](pool(e2), "silu")
        e4 = self.enc4["0"](pool(e3), "silu")
        h = self.bottleneck["0"](torch.cat((pool(e4), feat_nhwc), -1), "silu")
        for upc, dec, skip in ((self.up4, self.dec4, e4), (self.up3, self.dec3, e3), (self.up2, self.dec2, e2), (self.up1, self.dec1, e1)):
            h = dec["0"](torch.cat((upc["1"](up(h)), skip), -1), "silu")
        return self.out_conv(h)


class ZImageL2P(SingleStreamDiT):
    """forward(pixels [B, 3, H, W], cap [B, S_cap, cap_dim], sigma [B] in [0, 1]) -> prediction [B, 3, H, W] with
    ``x_next = x + (sigma_next - sigma) * prediction``."""

    def __init__(self, cfg: SingleDiTConfig, dtype=torch.bfloat16, device=None, decoder_channels=(64, 128, 256, 512)):
        super().__init__(cfg, dtype, device)
        self.patch = 16                      # the pixel head pools four times: the feature map is 1 / 16 of the image
        assert not cfg.final_layer and cfg.in_channels == 3 * self.patch * self.patch
        self.local_decoder = LocalDecoder(cfg.hidden, tuple(decoder_channels), 3, dtype, device)

    def forward(self, pixels, cap, sigma, cap_len: Optional[torch.Tensor] = None):
        B, _, H, W = pixels.shape
        p = self.patch
        gh, gw = H // p, W // p
        dt = self.all_x_embedder[self.cfg.patch_key].weight.dtype
        st = self.embed(patchify_pixels(pixels.to(dt), p), cap, 1.0 - sigma.float(), (gh, gw), cap_len)
        feat = self.run_layers(st).reshape(B, gh, gw, self.cfg.hidden)
        out = self.local_decoder(pixels.to(dt).permute(0, 2, 3, 1).contiguous(), feat)
        return -out.permute(0, 3, 1, 2)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        super().init_weights(seed, std)
        g = torch.Generator().manual_seed(seed + 1)
        with torch.no_grad():
            for m in self.local_decoder.modules():
                if isinstance(m, _Conv):
                    fan = m.weight.shape[1] * m.weight.shape[2] * m.weight.shape[3]
                    m.weight.copy_((torch.randn(m.weight.shape, generator=g) / fan ** 0.5).to(m.weight.dtype))
        return self


def remap_l2p_keys(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint convolution weights [out, in, kh, kw] -> [out, kh, kw, in]."""
    return {k: (v.permute(0, 2, 3, 1).contiguous() if k.startswith("local_decoder.") and v.dim() == 4 else v) for k, v in sd.items()}


@torch.no_grad()
def l2p_sample(model: ZImageL2P, cap: torch.Tensor, uncond_cap: Optional[torch.Tensor], height: int, width: int, steps: int = 30,
               cfg_scale: float = 2.0, shift: float = 3.0, seed: int = 0, x: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Pixel-space Euler sampling -> [1, 3, height, width] in the model's dtype."""
    dev = model.x_pad_token.device
    dt = model.x_pad_token.dtype
    if x is None:
        x = ops.randn((1, 3, height, width), seed, 0, torch.float32, dev)
    x = x.to(dt)
    sig = l2p_sigmas(steps, shift)
    for i in range(steps):
        s = torch.tensor([sig[i]], dtype=torch.float32, device=dev)
        pred = model(x, cap, s)
        if uncond_cap is not None:
            pu = model(x, uncond_cap, s)
            pred = pu + cfg_scale * (pred - pu)
        x = x + (sig[i + 1] - sig[i]) * pred
    return x
