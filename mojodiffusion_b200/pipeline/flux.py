"""FLUX-style text-to-image denoise pipeline (the public sampler entry of this package).

``FluxPipeline.denoise`` runs the guidance-distilled loop of the reference CLI
(serenitymojo/pipeline/flux_sample_cli.mojo:247-307): packed latents, BFL time-shifted sigmas with
mu(image_seq_len), one forward per step with ``t`` and ``guidance`` fed as values in [0, 1] (scaled by 1000 inside
the embedders), Euler update on an fp32 latent state. ``step_from_host`` is the serving-worker form of one denoise
step: inputs arrive in pinned host memory, the updated latent goes back to pinned host memory (the preview /
progress payload of serenitymojo/serve/flux_backend.mojo:482-512).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .. import ops
from ..models.mmdit import MMDiT, pack_latents
from ..sampling import flow_match as fm


class FluxPipeline:
    def __init__(self, model: MMDiT, device=None, sp=None, use_cuda_graph: bool = False):
        """``sp``: optional :class:`~mojodiffusion_b200.parallel.ulysses.UlyssesContext`; tensors handed to the
        pipeline are then this rank's token shards. ``use_cuda_graph`` replays the captured forward each step."""
        self.model = model
        self.device = torch.device(device) if device is not None else next(model.parameters()).device
        self.dtype = next(model.parameters()).dtype
        self.sp = sp
        self.use_cuda_graph = use_cuda_graph and self.device.type == "cuda"
        self._dev_buf = {}
        self._graph = None

    # ---- one velocity evaluation (eager or replayed graph) --------------------------------------------------
    def _forward(self, xb, txt, t, y, g, ids):
        if not self.use_cuda_graph:
            return self.model(xb, txt, t, y, g, ids=ids, sp=self.sp)
        if self._graph is None:
            from ..utils.cuda_graph import GraphedCallable
            fn = lambda xb_, txt_, t_, y_, g_: self.model(xb_, txt_, t_, y_, g_, ids=ids, sp=self.sp)
            self._graph = GraphedCallable(fn, [xb, txt, t, y, g]).capture()
        return self._graph(xb, txt, t, y, g)

    def global_ids(self, S_img_local: int, S_txt_local: int, hw=None):
        n = self.sp.world if self.sp is not None else 1
        S_img, S_txt = S_img_local * n, S_txt_local * n
        key = ("ids", S_img, S_txt)
        ids = self._dev_buf.get(key)
        if ids is None:
            ids = MMDiT.make_ids(*(hw or self._square(S_img)), S_txt, self.device)
            self._dev_buf[key] = ids
        return ids

    @torch.no_grad()
    def denoise(self, latents: torch.Tensor, txt: torch.Tensor, y: torch.Tensor, steps: int = 28,
                guidance: float = 3.5, hw: Optional[tuple] = None,
                callback: Optional[Callable[[int, torch.Tensor], None]] = None) -> torch.Tensor:
        """latents: packed noise [B, S_img, C] fp32; txt: [B, S_txt, ctx]; y: [B, vec]. Returns packed x0 (fp32)."""
        B, S_img, _ = latents.shape
        sigmas = fm.flux1_sigmas(steps, S_img)
        txt = txt.to(self.device, self.dtype)
        y = y.to(self.device, self.dtype)
        g = torch.full((B,), float(guidance), device=self.device)
        n = self.sp.world if self.sp is not None else 1
        sigmas = fm.flux1_sigmas(steps, S_img * n)
        ids = self.global_ids(S_img, txt.shape[1], hw)
        t = torch.empty((B,), device=self.device)

        def model_fn(xb, s):
            t.fill_(float(s))
            return self._forward(xb.to(self.dtype), txt, t, y, g, ids)

        return fm.euler_flow_sample(model_fn, latents.to(self.device), sigmas, callback=callback)

    @staticmethod
    def _square(n):
        side = int(round(n ** 0.5))
        return side, n // side

    @torch.no_grad()
    def step_from_host(self, x_host: torch.Tensor, txt_host: torch.Tensor, y_host: torch.Tensor, sigma: float,
                       sigma_next: float, guidance: float, out_host: torch.Tensor, hw: Optional[tuple] = None):
        """One denoise step with host I/O: pinned host inputs -> device, forward, Euler update, result -> pinned host.
        Returns (bytes_h2d, bytes_d2h)."""
        dev = self.device
        x = self._stage("x", x_host)
        txt = self._stage("txt", txt_host)
        y = self._stage("y", y_host)
        B, S_img, _ = x.shape
        g = self._const("g", B, float(guidance))
        t = self._const("t", B, float(sigma))
        ids = self.global_ids(S_img, txt.shape[1], hw)
        xb = self._cast("xb", x)
        v = self._forward(xb, self._cast("txtb", txt), t, self._cast("yb", y), g, ids)
        ops.cfg_euler(x, v, None, dt=float(sigma_next - sigma), mode=0)
        out_host.copy_(x, non_blocking=True)
        h2d = sum(t_.numel() * t_.element_size() for t_ in (x_host, txt_host, y_host))
        return h2d, out_host.numel() * out_host.element_size()

    def _const(self, name: str, n: int, value: float) -> torch.Tensor:
        buf = self._dev_buf.get(name)
        if buf is None or buf.numel() != n:
            buf = torch.empty((n,), device=self.device)
            self._dev_buf[name] = buf
        buf.fill_(value)
        return buf

    def _cast(self, name: str, src: torch.Tensor) -> torch.Tensor:
        if src.dtype == self.dtype:
            return src
        buf = self._dev_buf.get(name)
        if buf is None or buf.shape != src.shape:
            buf = torch.empty(src.shape, dtype=self.dtype, device=self.device)
            self._dev_buf[name] = buf
        buf.copy_(src)
        return buf

    def _stage(self, name: str, host: torch.Tensor) -> torch.Tensor:
        buf = self._dev_buf.get(name)
        if buf is None or buf.shape != host.shape or buf.dtype != host.dtype:
            buf = torch.empty(host.shape, dtype=host.dtype, device=self.device)
            self._dev_buf[name] = buf
        buf.copy_(host, non_blocking=True)
        return buf
