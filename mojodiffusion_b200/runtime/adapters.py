"""Family adapters: the few lines that differ between backbones when the same trainer, validation sampler and CLIs drive
them. An adapter turns a cache batch (VAE latents [B,C,h,w] + text embeddings) into model-space tensors, evaluates the
model as a velocity field in the rectified-flow convention ``v = eps - x0`` (or as ``eps`` for the DDPM family), attaches
adapters under the family's checkpoint key scheme and names the layout its LoRA files use.

Reference call sites per family: FLUX serenitymojo/models/flux/flux_stack_lora.mojo:786-1170, Klein
serenitymojo/models/klein/klein_stack_lora.mojo:2468-2511, Qwen-Image serenitymojo/models/qwenimage/qwenimage_stack_lora.mojo:205-234,
Z-Image serenitymojo/models/zimage/zimage_stack_lora.mojo:1655-1700 (model clock ``1 - sigma``, negated output), SD3.5
serenitymojo/models/sd35/sd35_stack_lora.mojo, SDXL serenitymojo/models/sdxl/sdxl_real_train.mojo:289,462 (eps target over the
scaled-linear DDPM grid), LTX-2 serenitymojo/training/ltx2/lora_surface.mojo:25-90.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..models.mmdit import pack_latents, unpack_latents
from .manifest import ModelManifest


@dataclass
class Cond:
    """Conditioning of one batch in model space."""
    txt: torch.Tensor                       # [B, T, D]
    pooled: Optional[torch.Tensor] = None   # [B, P]
    txt_len: Optional[torch.Tensor] = None  # [B] int32 valid text tokens (key mask), families that use one
    hw: Optional[Tuple[int, int]] = None    # token grid (rows, cols) of packed image latents
    grid: Optional[Tuple[int, int, int]] = None   # (frames, rows, cols) of video latents
    guidance: float = 1.0
    control: Optional[torch.Tensor] = None  # packed, normalised control latent (ControlNet training / sampling)


class FamilyAdapter:
    def __init__(self, manifest: ModelManifest):
        self.m = manifest
        self.family = manifest.family

    # ---- layout ------------------------------------------------------------------------------------------------
    def to_model_space(self, latent: torch.Tensor) -> Tuple[torch.Tensor, Cond]:
        """latent [B,C,h,w] (or [B,C,F,h,w] for video) -> (x0 in the layout the model consumes, a Cond with the grid)."""
        L = self.m.latent
        if latent.dim() == 5:                                   # video: tokens in (frame, row, col) order
            B, C, Fr, h, w = latent.shape
            x = latent.permute(0, 2, 3, 4, 1).reshape(B, Fr * h * w, C)
            return x, Cond(txt=None, grid=(Fr, h, w))
        if L.packed:
            h, w = latent.shape[-2] // L.patch, latent.shape[-1] // L.patch
            return pack_latents(latent, L.patch), Cond(txt=None, hw=(h, w))
        if self.family == "ernie":                              # one token per latent cell, channels as features
            return latent.flatten(2).transpose(1, 2), Cond(txt=None, hw=(latent.shape[-2], latent.shape[-1]))
        return latent, Cond(txt=None)

    def to_latent(self, x: torch.Tensor, cond: Cond) -> torch.Tensor:
        if cond.grid is not None:
            Fr, h, w = cond.grid
            return x.reshape(x.shape[0], Fr, h, w, -1).permute(0, 4, 1, 2, 3)
        if self.m.latent.packed:
            return unpack_latents(x, cond.hw[0], cond.hw[1], self.m.latent.patch)
        if self.family == "ernie":
            return x.transpose(1, 2).reshape(x.shape[0], -1, cond.hw[0], cond.hw[1])
        return x

    def conditioning(self, cond: Cond, text: torch.Tensor, mask: Optional[torch.Tensor], pooled: Optional[torch.Tensor],
                     model_cfg, guidance: float = 1.0) -> Cond:
        cond.txt = text
        cond.guidance = guidance
        T = self.m.text
        if T.key_mask or self.family in ("zimage", "anima"):
            if mask is not None:
                cond.txt_len = mask.to(torch.float32).sum(-1).round().to(torch.int32).clamp(min=1).to(text.device)
        P = self.pooled_dim(model_cfg)
        if P:
            if pooled is None or pooled.shape[-1] != P:
                pooled = torch.zeros(text.shape[0], P, dtype=text.dtype, device=text.device)
            cond.pooled = pooled.to(text.device, text.dtype)
        return cond

    def text_dim(self, model_cfg) -> int:
        """Width of the text features one token carries in a cache file or a hash embedding."""
        if self.family == "lens":
            return model_cfg.text_layers * model_cfg.text_hidden
        if self.family == "krea2":
            return model_cfg.txtlayers * model_cfg.txtdim
        return getattr(model_cfg, "context_dim", None) or getattr(model_cfg, "cap_dim", None) or self.m.text.dim

    def pooled_dim(self, model_cfg) -> int:
        if self.family == "flux":
            return model_cfg.vec_dim
        if self.family == "sd3":
            return model_cfg.pooled_dim
        if self.family == "sdxl":
            return model_cfg.adm_in_channels
        return 0

    # ---- the model as a velocity (or eps) field ----------------------------------------------------------------
    def predict(self, model, x: torch.Tensor, sigma: torch.Tensor, c: Cond) -> torch.Tensor:
        """x: noisy input in model space (model dtype); sigma: [B] fp32 in (0, 1] (DDPM family: integer timesteps as
        floats). Returns the prediction in the same layout as x."""
        f = self.family
        if f == "flux":
            g = None
            if model.cfg.guidance_embed:
                g = torch.full((x.shape[0],), float(c.guidance), device=x.device)
            return model(x, c.txt, sigma, c.pooled, g, hw=c.hw)
        if f in ("klein", "chroma"):
            return model(x, c.txt, sigma, c.hw)
        if f == "qwenimage":
            return model(x, c.txt, sigma, c.hw, c.txt_len)
        if f == "zimage":
            if c.control is not None:
                return -model(x, c.txt, 1.0 - sigma, c.hw, c.txt_len, control=c.control.to(x.dtype))
            return -model(x, c.txt, 1.0 - sigma, c.hw, c.txt_len)     # the model's clock runs from noise (0) to image (1)
        if f == "sd3":
            return model(x, c.txt, sigma, c.pooled)
        if f == "sdxl":
            return model(x, sigma, c.txt, c.pooled)
        if f == "ltx2":
            return model(x, c.txt, sigma, c.grid)
        if f == "ernie":
            return model(x, c.txt, sigma, c.hw, c.txt_len)
        if f == "anima":
            return model(x, c.txt, sigma, c.txt_len)
        if f == "lens":           # text features arrive as the concatenation of the captured encoder layers
            mc = model.cfg
            return model(x, c.txt.unflatten(-1, (mc.text_layers, mc.text_hidden)), sigma, c.hw, c.txt_len)
        if f == "krea2":          # twelve stacked encoder layers per token; text rows sit at position 0, image rows at (0, r, c)
            from ..models.krea2 import krea2_positions
            mc = model.cfg
            ctx = c.txt.unflatten(-1, (mc.txtlayers, mc.txtdim))
            return model(x, ctx, sigma, krea2_positions(ctx.shape[1], c.hw[0], c.hw[1], x.device))
        raise NotImplementedError(f"no adapter for family '{f}'")

    # ---- adapters --------------------------------------------------------------------------------------------------
    def inject_lora(self, model, rank: int, alpha: float):
        from ..training import lora as L
        spec = self.m.lora
        if spec is None:
            raise NotImplementedError(f"{self.m.model_id}: no LoRA surface is defined for this family")
        return getattr(L, spec.injector)(model, rank=rank, alpha=alpha)

    @property
    def lora_layout(self) -> str:
        return self.m.lora.layout if self.m.lora else "peft"


def adapter_for(manifest: ModelManifest) -> FamilyAdapter:
    return FamilyAdapter(manifest)


def schedule_for(m: ModelManifest, steps: int, image_tokens: int, shift: float = 0.0) -> List[float]:
    """Sigma table (steps + 1 values, 1 -> 0) of the family's default sampler."""
    from ..sampling import flow_match as fm
    k = m.schedule.kind
    if k == "flux1":
        return fm.flux1_sigmas(steps, image_tokens)
    if k == "flux2_klein":
        return fm.flux2_klein_sigmas(steps, image_tokens)
    if k == "qwen_image":
        return fm.qwen_image_sigmas(steps, image_tokens)
    if k == "sd3":
        return fm.sd3_sigmas(steps, shift or m.schedule.shift)
    if k == "ltx2_linear_quadratic":
        return fm.ltx2_linear_quadratic_sigmas(steps)
    if k == "shifted":
        return fm.shifted_sigmas(steps, shift or m.schedule.shift)
    if k == "lens_exp_shift":
        from ..sampling.family_schedules import lens_sigmas
        return list(lens_sigmas(steps, image_tokens)) + [0.0]
    if k == "krea2_exp_shift":
        from ..sampling.family_schedules import krea2_timesteps
        return krea2_timesteps(image_tokens, steps)
    raise ValueError(f"{m.model_id}: schedule kind '{k}' has no sigma table (DDPM families use sampling.ddpm)")
