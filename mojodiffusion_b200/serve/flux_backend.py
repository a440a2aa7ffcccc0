"""FLUX-family serving backend: ENCODE -> LOAD -> DENOISE x N -> DECODE, one ``step()`` per unit, the phase announced
before the tick that performs it. Weights come from ``MDB_MODEL_DIR`` (BFL-keyed safetensors: ``<model>.safetensors``,
``ae.safetensors``); with no weights on disk the backend runs the same code path on deterministic random weights of the
requested architecture and records ``"weights": "random-init"`` in its result sidecar, so the control plane, the kernels
and the file contracts can be exercised without a checkpoint. Text conditioning is read from pre-encoded caption files
(``sample_caps_pos`` / ``sample_caps_neg``: safetensors with ``text_embedding`` [1,T,4096] and ``pooled`` [1,768]); a
request without one gets a deterministic embedding derived from the prompt hash, marked ``"text": "hash-embedding"``.
The resident model stays loaded between jobs; LoRA stacks are merged into the resident copy at load and unmerged when
the next job asks for a different stack (serenitymojo/serve/flux_backend.mojo:40-46,325-512; result sidecar fields
serve/product_manifest.mojo:54)."""
from __future__ import annotations

import hashlib
import json
import os
import time
from typing import List, Optional

import numpy as np
import torch

from ..io.png import encode_png, load_png, tensor_to_uint8
from ..io.safetensors_io import load_safetensors
from ..sampling import flow_match as fm
from ..utils.tracing import nvtx_range
from .backend import GenBackend, JobParams, StepResult, reject_unsupported_common

_CONFIGS = {"flux": "flux1_dev_config", "tiny": "tiny_mmdit_config"}


def prompt_embedding(prompt: str, tokens: int, dim: int, pooled_dim: int):
    """Deterministic stand-in conditioning: unit-variance Gaussian seeded by the prompt's SHA-256."""
    seed = int.from_bytes(hashlib.sha256(prompt.encode("utf-8")).digest()[:8], "little") & 0x7FFFFFFFFFFFFFFF
    g = torch.Generator().manual_seed(seed)
    return torch.randn(1, tokens, dim, generator=g), torch.randn(1, pooled_dim, generator=g)


class FluxBackend(GenBackend):
    name = "flux"

    def __init__(self, kind: str = "flux", device: Optional[str] = None, arch: Optional[str] = None):
        self.kind = kind
        self.arch = arch or os.environ.get("MDB_FLUX_ARCH", kind)
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.model = self.vae = self.pipe = None
        self.loaded_name = ""
        self.weights_kind = ""
        self.merged_loras: List = []
        self.p: Optional[JobParams] = None
        self._cancel = False
        self.phase = "idle"
        self.stage_s = {}

    def resident_model(self) -> str:
        return self.loaded_name

    # ---- job -----------------------------------------------------------------------------------------------
    def start(self, params: JobParams) -> None:
        reject_unsupported_common(params, inpaint=True, img2img=True)
        if params.sampler and params.sampler.lower() not in ("euler", "flowmatch_euler", "flow_match_euler"):
            raise ValueError(f"flux backend supports the euler flow-matching sampler, not '{params.sampler}'")
        self.p, self._cancel, self.phase, self.i = params, False, "encode", 0
        self.stage_s = {}
        self.text_kind = ""

    def step(self) -> StepResult:
        p = self.p
        assert p is not None
        if self._cancel:
            self.p = None
            self.phase = "idle"
            return StepResult("cancelled")
        t0 = time.perf_counter()
        if self.phase == "encode":
            with nvtx_range("stage/encode"):
                self._encode(p)
            self.stage_s["encode"] = time.perf_counter() - t0
            self.phase = "load"
            return StepResult("progress", 0, p.steps, "load")         # announce what the NEXT tick does
        if self.phase == "load":
            with nvtx_range("stage/load"):
                self._load(p)
                self._prepare_latents(p)
            self.stage_s["load"] = time.perf_counter() - t0
            self.phase = "denoise"
            return StepResult("progress", 0, p.steps, "denoise")
        if self.phase == "denoise":
            with nvtx_range(f"stage/denoise/{self.i}"):
                self._denoise_step()
            self.stage_s["denoise"] = self.stage_s.get("denoise", 0.0) + time.perf_counter() - t0
            self.i += 1
            if self.i >= self.n_steps:
                self.phase = "decode"
                return StepResult("progress", p.steps, p.steps, "decode")
            return StepResult("progress", self.i + (p.steps - self.n_steps), p.steps, "denoise")
        with nvtx_range("stage/decode"):
            path = self._decode_and_save(p)
        self.stage_s["decode"] = time.perf_counter() - t0
        self._write_sidecar(p, path)
        self.p = None
        self.phase = "idle"
        return StepResult("done", output_path=path)

    def trim(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    # ---- phases -------------------------------------------------------------------------------------------------
    def _encode(self, p: JobParams) -> None:
        from ..models import mmdit
        cfg = getattr(mmdit, _CONFIGS.get(self.arch, "flux1_dev_config"))()
        self.cfg = cfg
        if p.sample_caps_pos and os.path.isfile(p.sample_caps_pos):
            d = load_safetensors(p.sample_caps_pos)
            self.txt, self.pooled = d["text_embedding"].float(), d["pooled"].float()
            self.text_kind = "pre-encoded"
        else:
            self.txt, self.pooled = prompt_embedding(p.prompt, 512 if cfg.context_dim >= 1024 else 32, cfg.context_dim, cfg.vec_dim)
            self.text_kind = "hash-embedding"

    def _load(self, p: JobParams) -> None:
        from ..models import mmdit
        from ..models.vae import AutoencoderKL, flux_vae_config, tiny_vae_config
        from ..pipeline.flux import FluxPipeline
        if self.model is None or self.loaded_name != p.model:
            self.model = self.vae = self.pipe = None
            self.trim()
            model = mmdit.MMDiT(self.cfg, self.dtype, self.device)
            root = os.environ.get("MDB_MODEL_DIR", "")
            path = os.path.join(root, p.model if p.model.endswith(".safetensors") else p.model + ".safetensors")
            if root and os.path.isfile(path):
                sd = load_safetensors(path, device=str(self.device), dtype=self.dtype)
                missing = [k for k in model.state_dict() if k not in sd]
                if missing:
                    raise KeyError(f"checkpoint lacks {len(missing)} tensors, e.g. {missing[:3]}")
                model.load_state_dict(sd, strict=False)
                self.weights_kind = "checkpoint"
            else:
                model.init_weights(seed=0)
                self.weights_kind = "random-init"
            tiny = self.arch == "tiny"
            import dataclasses
            vcfg = dataclasses.replace(tiny_vae_config(), z_channels=self.cfg.in_channels // 4) if tiny else flux_vae_config()
            vae = AutoencoderKL(vcfg, self.dtype, self.device, with_encoder=True)
            if self.weights_kind == "random-init":
                torch.manual_seed(0)
                for prm in vae.parameters():
                    if prm.dim() > 1:
                        torch.nn.init.normal_(prm, std=0.05)
            vpath = os.path.join(root, p.vae or "ae.safetensors")
            if root and os.path.isfile(vpath):
                vae.load_state_dict(load_safetensors(vpath, device=str(self.device), dtype=self.dtype), strict=False)
            self.model, self.vae = model.eval(), vae.eval()
            self.pipe = FluxPipeline(self.model, self.device)
            self.loaded_name = p.model
            self.merged_loras = []
        want = [(l.name, l.weight) for l in p.loras]
        if want != self.merged_loras:
            if self.merged_loras or want:
                self._apply_loras(want)
            self.merged_loras = want

    def _apply_loras(self, want) -> None:
        from ..training.lora import inject_flux_lora, load_lora, merge_lora_into_weights
        root = os.environ.get("MDB_LORA_DIR", os.environ.get("MDB_MODEL_DIR", ""))
        # undo the previous stack by merging it with the opposite sign, then merge the new one
        for sign, stack in ((-1.0, self.merged_loras), (1.0, want)):
            for name, weight in stack:
                path = os.path.join(root, name)
                if not os.path.isfile(path):
                    raise FileNotFoundError(f"LoRA file not found: {name}")
                sd = load_safetensors(path)
                rank = next(v.shape[0] for k, v in sd.items() if k.endswith("lora_down.weight") or k.endswith("lora_A.weight"))
                slots = inject_flux_lora(self.model, rank=rank, alpha=float(rank))
                load_lora(path, slots, strict=False)
                merge_lora_into_weights(self.model, sign * weight)

    def _prepare_latents(self, p: JobParams) -> None:
        from ..models.mmdit import pack_latents
        f = self.vae.spatial_factor
        C = self.vae.cfg.z_channels
        h, w = p.height // f, p.width // f
        g = torch.Generator().manual_seed(int(p.seed) & 0x7FFFFFFFFFFFFFFF)
        noise = torch.randn(1, C, h, w, generator=g)
        if p.variation_strength > 0:
            g2 = torch.Generator().manual_seed(int(p.variation_seed) & 0x7FFFFFFFFFFFFFFF)
            from ..sampling.inpaint import slerp
            noise = slerp(noise, torch.randn(1, C, h, w, generator=g2), p.variation_strength)
        self.hw = (h // 2, w // 2)
        S_img = self.hw[0] * self.hw[1]
        sigmas = fm.flux1_sigmas(p.steps, S_img)
        start = 0
        x = noise
        self.init_latent = self.mask = None
        if p.init_image:
            from .image_io import load_image_rgb, load_mask, resize_lanczos
            t = resize_lanczos(load_image_rgb(p.init_image), p.height, p.width).clamp(-1.0, 1.0)
            with torch.no_grad():
                z0 = self.vae.encode(t.to(self.device), sample=False).float().cpu()
            start = min(p.steps - 1, int(round(p.steps * (1.0 - max(0.0, min(1.0, p.creativity))))))
            s0 = float(sigmas[start])
            x = (1.0 - s0) * z0 + s0 * noise
            self.init_latent = z0
            if p.mask_image:
                self.mask = resize_lanczos(load_mask(p.mask_image), h, w).clamp(0.0, 1.0)
        self.noise = noise
        self.sigmas = sigmas
        self.start, self.n_steps = start, p.steps - start
        self.x = pack_latents(x).float().to(self.device)
        self.txt_d = self.txt.to(self.device, self.dtype)
        self.y_d = self.pooled.to(self.device, self.dtype)
        self.ids = self.pipe.global_ids(self.x.shape[1], self.txt_d.shape[1], self.hw)
        self.t = torch.empty(1, device=self.device)
        self.g = torch.full((1,), float(p.cfg if p.cfg > 1.0 else 3.5), device=self.device)

    @torch.no_grad()
    def _denoise_step(self) -> None:
        from .. import ops
        from ..models.mmdit import pack_latents
        k = self.start + self.i
        s, s_next = float(self.sigmas[k]), float(self.sigmas[k + 1])
        self.t.fill_(s)
        v = self.pipe._forward(self.x.to(self.dtype), self.txt_d, self.t, self.y_d, self.g if self.cfg.guidance_embed else None, self.ids)
        self.x = ops.cfg_euler(self.x, v, None, dt=s_next - s, mode=0)
        if self.mask is not None:                 # inpaint: keep the unmasked region on the noised original
            known = pack_latents((1.0 - s_next) * self.init_latent + s_next * self.noise).to(self.device)
            m = pack_latents(self.mask.expand_as(self.init_latent)).to(self.device)
            self.x = m * self.x + (1.0 - m) * known

    @torch.no_grad()
    def _decode_and_save(self, p: JobParams) -> str:
        from ..models.mmdit import unpack_latents
        z = unpack_latents(self.x, self.hw[0], self.hw[1])
        img = self.vae.tiled_decode(z) if max(z.shape[-2:]) > 96 else self.vae.decode(z)
        arr = tensor_to_uint8(img[0].float().permute(1, 2, 0).cpu()).numpy()
        os.makedirs(p.out_dir or ".", exist_ok=True)
        path = p.output_path()
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(encode_png(arr, {"serenity.genparams.v1": p.genparams_text()}))
        os.replace(tmp, path)
        return path

    def _write_sidecar(self, p: JobParams, path: str) -> None:
        peak = torch.cuda.max_memory_allocated() if self.device.type == "cuda" else 0
        side = {"schema": "serenity.flux.daemon_result.v1", "job_id": p.job_id, "model": p.model, "weights": self.weights_kind,
                "text": self.text_kind, "stage_seconds": {k: round(v, 4) for k, v in self.stage_s.items()},
                "peak_device_bytes": int(peak), "steps_run": self.n_steps, "sampler": "euler",
                "lora": [{"name": n, "weight": w} for n, w in self.merged_loras], "device": str(self.device)}
        with open(path + ".worker_result.json", "w") as f:
            json.dump(side, f)
