"""LoRA / finetune train step for flow-matching backbones.

One step = sample sigma -> x_t, target (fused kernel) -> model forward -> MSE (fp32 accumulate) -> backward ->
[data-parallel gradient sync] -> clip + AdamW in one launch. Mirrors the step anatomy of the reference trainers
(serenitymojo/training/train_step.mojo:297-392, serenitymojo/training/train_anima_ot.mojo:1027-1165) with every
tensor resident on the device and no host round trip inside the step except the optional loss read-back.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from .. import ops
from ..parallel.dp import DataParallelGrads
from .optim import FusedAdamW
from .schedule import sample_sigmas


@dataclass
class StepConfig:
    timestep_kind: str = "logit_normal"
    timestep_shift: float = 1.0
    guidance: float = 1.0
    seed: int = 0
    rank: int = 0                 # data-parallel rank and world size: every rank draws its own sigmas and noise
    world: int = 1                # (seed * world + rank); set rank_identical_draws for the DP-N == batch-N parity tests
    rank_identical_draws: bool = False

    def stream_seed(self) -> int:
        if self.rank_identical_draws or self.world <= 1:
            return self.seed
        return self.seed * self.world + self.rank


class FlowMatchTrainer:
    """Drives ``model(img, txt, t, y, guidance)`` towards the rectified-flow velocity ``eps - x0``."""

    def __init__(self, model, params: Sequence[torch.nn.Parameter], optimizer: FusedAdamW,
                 dp: Optional[DataParallelGrads] = None, cfg: Optional[StepConfig] = None, use_cuda_graph: bool = False):
        """``use_cuda_graph``: forward + backward of the step are captured once (fixed shapes) and replayed; sigma and
        noise are drawn outside the graph into its static inputs, the optimizer runs after the replay."""
        self.use_cuda_graph = use_cuda_graph
        self._graphed = None
        self._graph_key = None
        self.model = model
        self.params = list(params)
        self.opt = optimizer
        self.dp = dp
        self.cfg = cfg or StepConfig()
        self.step_index = 0
        self._seed = self.cfg.stream_seed()
        self._gen = torch.Generator().manual_seed(self._seed)

    def zero_grad(self):
        if self.dp is not None:
            self.dp.zero_grad()
        else:
            self.opt.zero_grad(set_to_none=True)

    def loss_and_backward(self, x0: torch.Tensor, txt: torch.Tensor, y: torch.Tensor,
                          sigma: Optional[torch.Tensor] = None, noise: Optional[torch.Tensor] = None,
                          hw=None, loss_scale: float = 1.0) -> torch.Tensor:
        """x0: packed clean latents [B, S, C] (fp32). Returns the detached loss (device scalar)."""
        B = x0.shape[0]
        dev = x0.device
        if sigma is None:
            sigma = sample_sigmas(B, self._gen, self.cfg.timestep_kind, self.cfg.timestep_shift).to(dev)
        if noise is None:
            noise = ops.randn(tuple(x0.shape), seed=self._seed * 7919 + self.step_index, device=dev)
        xt, target = ops.flow_match(x0.float(), noise.float(), sigma.float())
        dt = next(self.model.parameters()).dtype
        guidance = torch.full((B,), self.cfg.guidance, device=dev) if self.model.cfg.guidance_embed else None
        pred = self.model(xt.to(dt), txt.to(dt), sigma.float(), y.to(dt), guidance, hw=hw)
        loss = ops.mse_loss(pred, target)
        (loss * loss_scale).backward()
        return loss.detach()

    def _graphed_loss_and_backward(self, x0, txt, y, sigma, noise, hw) -> torch.Tensor:
        from ..utils.cuda_graph import GraphedTrainStep
        B, dev = x0.shape[0], x0.device
        if sigma is None:
            sigma = sample_sigmas(B, self._gen, self.cfg.timestep_kind, self.cfg.timestep_shift).to(dev)
        if noise is None:
            noise = ops.randn(tuple(x0.shape), seed=self._seed * 7919 + self.step_index, device=dev)
        inputs = [x0.float(), txt, y, sigma.float(), noise.float()]
        key = (tuple(x0.shape), tuple(txt.shape), tuple(y.shape), hw)
        if self._graphed is None or self._graph_key != key:
            dt = next(self.model.parameters()).dtype
            guidance = torch.full((B,), self.cfg.guidance, device=dev) if self.model.cfg.guidance_embed else None

            def loss_fn(x0_, txt_, y_, sigma_, noise_):
                xt, target = ops.flow_match(x0_, noise_, sigma_)
                pred = self.model(xt.to(dt), txt_.to(dt), sigma_, y_.to(dt), guidance, hw=hw)
                return ops.mse_loss(pred, target)

            flat = getattr(self.opt, "flat_grads", None) is not None      # gradients are views of one buffer: clear it in the graph
            self._graphed = GraphedTrainStep(loss_fn, self.params, inputs, zero_grad=self.opt.zero_grad if flat else None).capture()
            self._graph_key = key
        return self._graphed(*inputs).detach()

    def step(self, x0, txt, y, sigma=None, noise=None, hw=None, lr: Optional[float] = None) -> torch.Tensor:
        if self.use_cuda_graph and x0.is_cuda and self.dp is None and (type(self.opt) is FusedAdamW or hasattr(self.opt, "flat_grads")):
            loss = self._graphed_loss_and_backward(x0, txt, y, sigma, noise, hw)
            self.opt.step(grad_scale=1.0, lr=lr)
            self.step_index += 1
            return loss
        self.zero_grad()
        loss = self.loss_and_backward(x0, txt, y, sigma, noise, hw)
        scale = self.dp.sync() if self.dp is not None else 1.0
        self.opt.step(grad_scale=scale, lr=lr)
        self.step_index += 1
        return loss
