"""One train step for any backbone family, driven by its manifest adapter.

Flow-matching families: sample sigma (config's timestep distribution and shift) -> ``x_t = (1 - sigma) x0 + sigma eps``,
``target = eps - x0`` (fused kernel with the seeded on-device noise) -> model as a velocity field -> loss levers -> backward
-> [data-parallel sync] -> clip + AdamW in one launch. The DDPM family (SDXL) draws an integer timestep, noises with the
scaled-linear alpha-bar table and regresses ``eps``. Step anatomy: serenitymojo/training/train_step.mojo:297-392,
serenitymojo/training/train_anima_ot.mojo:1027-1165; SDXL recipe: TRAINING_PLAN_sdxl.md:297-315.
"""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import torch

from .. import ops
from ..io.config import TrainConfig
from ..runtime.adapters import Cond, FamilyAdapter
from . import features as F
from .losses import diffusion_loss
from .schedule import sample_discrete_timesteps, sample_sigmas
from .trainer import StepConfig


class FamilyTrainer:
    def __init__(self, adapter: FamilyAdapter, model, params: Sequence[torch.nn.Parameter], optimizer, cfg: TrainConfig,
                 dp=None, step_cfg: Optional[StepConfig] = None):
        self.a, self.model, self.params, self.opt, self.cfg, self.dp = adapter, model, list(params), optimizer, cfg, dp
        self.sc = step_cfg or StepConfig(seed=cfg.seed)
        self._seed = self.sc.stream_seed()
        self._gen = torch.Generator().manual_seed(self._seed)
        self.step_index = 0
        self.eps_prediction = adapter.m.schedule.prediction == "epsilon"
        if self.eps_prediction:
            from ..sampling.ddpm import alphas_cumprod
            self._ac = alphas_cumprod(cfg.num_train_timesteps, cfg.beta_start, cfg.beta_end)
        self._accum = 0

    def zero_grad(self):
        if self.dp is not None:
            self.dp.zero_grad()
        else:
            self.opt.zero_grad(set_to_none=True)

    def _sigmas(self, B: int, dev):
        c = self.cfg
        kind = {"LOGIT_NORMAL": "logit_normal", "UNIFORM": "uniform", "SIGMOID": "sigmoid"}.get(c.timestep_distribution.upper(), "")
        if kind:
            return sample_sigmas(B, self._gen, kind, c.timestep_shift or 1.0).to(dev), None
        if c.timestep_distribution.upper() in ("DISCRETE", "ONETRAINER_DISCRETE"):
            s, t = sample_discrete_timesteps(B, self._gen, c.timestep_shift or 1.0)
            return s.to(dev), t.to(dev)
        raise ValueError(f"unknown timestep_distribution {c.timestep_distribution}")

    def loss_and_backward(self, batch: Dict[str, torch.Tensor], loss_scale: float = 1.0) -> torch.Tensor:
        """batch: ``latent`` [B,C,h,w] (VAE space, unscaled), ``text_embedding`` [B,T,D], ``text_mask`` [B,T], optional
        ``pooled`` [B,P], ``latent_mask``, ``control_latent`` [B,C,h,w] (ControlNet). Returns the detached loss."""
        m, c = self.a.m, self.cfg
        dev = next(self.model.parameters()).device
        dt = next(self.model.parameters()).dtype
        lat = batch["latent"].to(dev, torch.float32)
        lat = (lat - m.latent.shift) * m.latent.scale
        x0, cond = self.a.to_model_space(lat)
        text = batch["text_embedding"].to(dev, dt)
        if c.caption_dropout_prob > 0:
            text = F.drop_caption(text, None, c.caption_dropout_prob, self._gen)
        pooled = batch.get("pooled")
        cond = self.a.conditioning(cond, text, batch.get("text_mask"), pooled.to(dev, dt) if pooled is not None else None,
                                   self.model.cfg, guidance=self.sc.guidance)
        ctrl = batch.get("control_latent")
        if ctrl is not None:                          # the control image enters as a VAE latent with the training normalisation
            cl = (ctrl.to(dev, torch.float32) - m.latent.shift) * m.latent.scale
            cond.control, _ = self.a.to_model_space(cl)
        B = x0.shape[0]
        noise = ops.randn(tuple(x0.shape), seed=self._seed * 7919 + self.step_index, device=dev).float()
        mask = batch.get("latent_mask")
        if self.eps_prediction:
            t_idx = torch.randint(0, c.num_train_timesteps, (B,), generator=self._gen)
            ab = self._ac[t_idx].to(dev).float().view(B, *([1] * (x0.dim() - 1)))
            xt = ab.sqrt() * x0.float() + (1.0 - ab).sqrt() * noise
            pred = self.a.predict(self.model, xt.to(dt), t_idx.float().to(dev), cond)
            loss = diffusion_loss(pred, noise, None, c.loss_fn, mask.to(dev) if mask is not None else None,
                                  huber_delta=c.huber_delta, smooth_l1_beta=c.smooth_l1_beta)
        else:
            sigma, _ = self._sigmas(B, dev)
            xt, target = ops.flow_match(x0.float(), noise, sigma.float())
            pred = self.a.predict(self.model, xt.to(dt), sigma.float(), cond)
            lm = None
            if mask is not None:
                lm, _ = self.a.to_model_space(mask.to(dev, torch.float32).expand_as(lat))
            loss = diffusion_loss(pred, target, sigma, c.loss_fn, lm, min_snr_gamma=c.min_snr_gamma_flow,
                                  huber_delta=c.huber_delta, smooth_l1_beta=c.smooth_l1_beta)
        (loss * loss_scale).backward()
        return loss.detach()

    def step(self, batch: Dict[str, torch.Tensor], lr: Optional[float] = None, accumulate: int = 1) -> torch.Tensor:
        """One optimizer step (``accumulate`` > 1: call it that many times, the update happens on the last call)."""
        if self._accum == 0:
            self.zero_grad()
        loss = self.loss_and_backward(batch, 1.0 / accumulate)
        self._accum += 1
        self.step_index += 1
        if self._accum < accumulate:
            return loss
        self._accum = 0
        scale = self.dp.sync() if self.dp is not None else 1.0
        self.opt.step(grad_scale=scale, lr=lr)
        return loss

    def grad_norm(self):
        g = getattr(self.opt, "grad_norm", None)
        return g() if callable(g) else 0.0
