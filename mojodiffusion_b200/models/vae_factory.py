"""One place that knows which autoencoder a backbone family decodes with, and how its checkpoint is spelled.

    flux / chroma / zimage -> 16-channel LDM autoencoder (Z-Image ships it under diffusers names)
    sd3 / sdxl             -> their LDM autoencoders
    klein                  -> FLUX.2 autoencoder with packed latents and BatchNorm statistics
    qwenimage              -> Wan2.1-style causal 3-D VAE in image mode
    wan22                  -> Wan2.2 high-compression VAE
    ltx2                   -> LTX-2 video VAE

``decode_latent`` takes the latent in the layout the family adapter produces ([B, C, h, w], video [B, C, F, h, w]).
"""
from __future__ import annotations

import os
from typing import Optional

import torch


def build_family_vae(family: str, dtype=torch.bfloat16, device=None, with_encoder: bool = False, vae_config_fn: str = ""):
    from . import vae as V
    if family == "klein":
        return V.KleinVAE(V.klein_vae_config(), dtype, device, with_encoder)
    if family == "qwenimage":
        from .wan_vae import WanVAE, qwen_image_vae_config
        return WanVAE(qwen_image_vae_config(), dtype, device, with_encoder)
    if family in ("wan22", "wan"):
        from .wan_vae import WanVAE, wan22_vae_config
        return WanVAE(wan22_vae_config(), dtype, device, with_encoder)
    if family == "ltx2":
        from .video_vae import VideoVAE, ltx2_vae_config
        return VideoVAE(ltx2_vae_config(), dtype, device)
    name = vae_config_fn or {"sd3": "sd3_vae_config", "sdxl": "sdxl_vae_config", "zimage": "zimage_vae_config"}.get(family, "flux_vae_config")
    return V.AutoencoderKL(getattr(V, name)(), dtype, device, with_encoder)


def load_vae_weights(vae, path: str, device=None, dtype=None) -> str:
    """Load a checkpoint in either spelling (LDM / Wan names, or the diffusers names of the same tensors). Returns
    "checkpoint", or raises when nothing matched."""
    from ..io.safetensors_io import load_safetensors
    sd = load_safetensors(path, device=str(device) if device is not None else "cpu", dtype=dtype)
    if any(k.startswith(("decoder.up_blocks.", "encoder.down_blocks.", "decoder.mid_block.")) for k in sd):
        from .wan_vae import WanVAE, remap_diffusers_wan_keys
        if isinstance(vae, WanVAE):
            sd = remap_diffusers_wan_keys(sd, vae.cfg.num_res_blocks)
        else:
            from .vae import remap_diffusers_vae_keys
            sd = remap_diffusers_vae_keys(sd, len(vae.cfg.ch_mult))
    own = vae.state_dict()
    hit = {k: v for k, v in sd.items() if k in own and tuple(v.shape) == tuple(own[k].shape)}
    if not hit:
        raise ValueError(f"{os.path.basename(path)}: no tensor matches this autoencoder's parameters")
    vae.load_state_dict(hit, strict=False)
    return "checkpoint"


def decode_latent(vae, z: torch.Tensor, tile_above: int = 96) -> torch.Tensor:
    """latent -> image [B, 3, H, W] (or video [B, 3, T, H, W]) in [-1, 1]."""
    from .vae import KleinVAE
    if isinstance(vae, KleinVAE):
        return vae.decode(KleinVAE.pack(z))
    if z.dim() == 4 and hasattr(vae, "tiled_decode") and max(z.shape[-2:]) > tile_above:
        return vae.tiled_decode(z)
    return vae.decode(z)


def latent_geometry(vae):
    """(channels, pixels per latent cell) of the latent layout ``decode_latent`` takes."""
    from .vae import KleinVAE
    from .wan_vae import WanVAE
    if isinstance(vae, KleinVAE):
        return vae.cfg.z_channels, vae.spatial_factor // 2          # unpacked 32-channel latent at 1/8 resolution
    if isinstance(vae, WanVAE):
        return vae.cfg.z_dim, vae.cfg.spatial_factor
    return vae.cfg.z_channels, vae.spatial_factor
