"""Validation sampling inside or beside training: staged load -> denoise -> VAE decode -> PNG with embedded parameters.

``ValidationSampler`` runs the family's default sampler on a model that is already resident (the training model with its
adapters active, switched to eval / no-grad for the duration) or on one it builds itself; the VAE is built for the decode
stage and dropped afterwards unless ``keep_vae``. Text conditioning comes from a pre-encoded caption file named by the
prompt (``caps.positive`` / ``caps.negative``), else from ``encode_fn(prompt)``, else from the deterministic prompt-hash
embedding the serving workers use for smoke runs (the result sidecar says which).

Reference behaviour: serenitymojo/training/validation_sampler.mojo:169-225 (stage order, one PNG per prompt,
``<prefix>-training-sample-<step>-<epoch>-<epoch_step>-<i>.png``), serenitymojo/sampling/base_sampler.mojo:34-93 (resolution
quantisation, staged load / free discipline), serenitymojo/pipeline/flux_sample_cli.mojo:247-307 (denoise loop).
"""
from __future__ import annotations

import dataclasses
import json
import os
import time
import zlib
from typing import Callable, List, Optional

import torch

from ..io.config import SamplePrompt
from ..io.png import encode_png, tensor_to_uint8
from ..io.safetensors_io import load_safetensors
from ..runtime.adapters import Cond, adapter_for, schedule_for
from ..runtime.manifest import ModelManifest, ProductionGuard, ShapeProfile
from ..sampling.guidance import cfg_cond_anchored, cfg_textbook, cfg_true_with_norm_rescale


def _hash_text(prompt: str, tokens: int, dim: int, pooled: int):
    from ..serve.flux_backend import prompt_embedding
    return prompt_embedding(prompt, tokens, dim, max(pooled, 1))


class ValidationSampler:
    def __init__(self, manifest: ModelManifest, model, device=None, dtype=None, tiny: bool = False, vae=None,
                 vae_path: str = "", encode_fn: Optional[Callable] = None, keep_vae: bool = False):
        self.m, self.model, self.tiny = manifest, model, tiny
        p0 = next(model.parameters())
        self.device = torch.device(device) if device is not None else p0.device
        self.dtype = dtype if dtype is not None else p0.dtype
        self.a = adapter_for(manifest)
        self.vae, self.vae_path, self.keep_vae = vae, vae_path, keep_vae
        self.encode_fn = encode_fn
        self.last_report = {}

    # ---- stages ----------------------------------------------------------------------------------------------
    def _text(self, sp: SamplePrompt, negative: bool):
        cfg = self.model.cfg
        T = 32 if self.tiny else self.m.text.tokens
        D = self.a.text_dim(cfg)
        P = self.a.pooled_dim(cfg)
        path = sp.caps_negative if negative else sp.caps_positive
        prompt = sp.negative if negative else sp.prompt
        if path and os.path.isfile(path):
            d = load_safetensors(path)
            return d["text_embedding"].float(), (d["pooled"].float() if "pooled" in d else None), "pre-encoded"
        if self.encode_fn is not None:
            txt, pooled = self.encode_fn(prompt)
            return txt.float(), (pooled.float() if pooled is not None else None), "encoder"
        txt, pooled = _hash_text(prompt, T, D, P)
        return txt, (pooled if P else None), "hash-embedding"

    def _build_vae(self):
        if self.vae is not None:
            return self.vae
        if self.m.family == "ltx2":
            from ..models.video_vae import VideoVAE, ltx2_vae_config, tiny_video_vae_config
            vcfg = dataclasses.replace(tiny_video_vae_config(), latent_channels=self.model.cfg.in_channels) if self.tiny else ltx2_vae_config()
            vae = VideoVAE(vcfg, self.dtype, self.device)
        else:
            from ..models import vae as V
            if self.tiny:
                zc = self.model.cfg.in_channels // (self.m.latent.patch ** 2) if self.m.latent.packed else self.model.cfg.in_channels
                vcfg = dataclasses.replace(V.tiny_vae_config(), z_channels=zc)
                vae = V.AutoencoderKL(vcfg, self.dtype, self.device, with_encoder=False)
            else:                                  # the family's own autoencoder (Klein: packed + BatchNorm; Qwen-Image: 3-D)
                from ..models.vae_factory import build_family_vae
                vae = build_family_vae(self.m.family, self.dtype, self.device, False, self.m.vae_config_fn)
        if self.vae_path and os.path.isfile(self.vae_path):
            from ..models.vae_factory import load_vae_weights
            self.vae_weights = load_vae_weights(vae, self.vae_path, self.device, self.dtype)
        else:
            vae.init_weights(seed=1)
            self.vae_weights = "random-init"
        vae.eval()
        if self.keep_vae:
            self.vae = vae
        return vae

    @torch.no_grad()
    def denoise(self, sp: SamplePrompt) -> tuple:
        """Returns (latent in VAE space [1,C,h,w] or [1,C,F,h,w], text kind)."""
        m, L, dev, dt = self.m, self.m.latent, self.device, self.dtype
        shape = ShapeProfile.of(m, sp.width, sp.height, max(sp.frames, 1))
        ProductionGuard.check(m, shape)
        g = torch.Generator().manual_seed(int(sp.seed) & 0x7FFFFFFFFFFFFFFF)
        f, ft = L.vae_factor, L.temporal_factor
        if self.tiny:                      # the tiny VAEs expand by less than the real ones: ask the VAE itself
            if self.vae is None:
                keep, self.keep_vae = self.keep_vae, True
                self._build_vae()
                self.keep_vae = keep
            if m.family == "ltx2":
                ft, f = self.vae.expansion()
            else:
                f = self.vae.spatial_factor
        h, w = sp.height // f, sp.width // f
        C = self.model.cfg.in_channels // (L.patch ** 2) if L.packed and m.family != "ltx2" else self.model.cfg.in_channels
        if m.family == "ltx2":
            Fr = 1 + max(sp.frames - 1, 0) // ft
            noise = torch.randn(1, C, Fr, h, w, generator=g)
        else:
            noise = torch.randn(1, C, h, w, generator=g)
        txt, pooled, kind = self._text(sp, False)
        use_cfg = sp.cfg > 1.0 and m.schedule.cfg_rule != "distilled"
        x, cond = self.a.to_model_space(noise.float().to(dev))
        guidance = sp.cfg if m.schedule.cfg_rule == "distilled" else 1.0
        cond = self.a.conditioning(cond, txt.to(dev, dt), None, pooled.to(dev, dt) if pooled is not None else None,
                                   self.model.cfg, guidance=guidance if guidance > 0 else m.schedule.cfg)
        if m.family == "sdxl" and cond.pooled is not None and pooled is not None and pooled.shape[-1] != cond.pooled.shape[-1]:
            pass
        cond_u = None
        if use_cfg:
            tn, pn, _ = self._text(sp, True)
            if tn.shape[1] != txt.shape[1]:
                tn = torch.nn.functional.pad(tn, (0, 0, 0, txt.shape[1] - tn.shape[1]))[:, :txt.shape[1]]
            cond_u = self.a.conditioning(Cond(None, hw=cond.hw, grid=cond.grid), tn.to(dev, dt), None,
                                         pn.to(dev, dt) if pn is not None else None, self.model.cfg)
        was_training = self.model.training
        self.model.eval()
        try:
            if m.schedule.prediction == "epsilon":
                from ..sampling.ddpm import SDXLEulerScheduler
                sched = SDXLEulerScheduler(sp.steps)
                x = x * sched.init_noise_sigma
                t = torch.empty(1, device=dev)
                for i, ts in enumerate(sched.timesteps):
                    t.fill_(float(ts))
                    xin = sched.scale_model_input(x, i).to(dt)
                    e = self.a.predict(self.model, xin, t, cond).float()
                    if cond_u is not None:
                        e = cfg_textbook(e, self.a.predict(self.model, xin, t, cond_u).float(), sp.cfg)
                    x = sched.step(x, e, i)
            else:
                sig = schedule_for(m, sp.steps, shape.image_tokens)
                t = torch.empty(1, device=dev)
                for i in range(sp.steps):
                    s, s_next = float(sig[i]), float(sig[i + 1])
                    t.fill_(s)
                    xb = x.to(dt)
                    v = self.a.predict(self.model, xb, t, cond).float()
                    if cond_u is not None:
                        vu = self.a.predict(self.model, xb, t, cond_u).float()
                        rule = m.schedule.cfg_rule
                        v = (cfg_true_with_norm_rescale(v, vu, sp.cfg) if rule == "true_norm_rescale" else
                             cfg_cond_anchored(v, vu, sp.cfg) if rule == "cond_anchored" else cfg_textbook(v, vu, sp.cfg))
                    last = m.family == "ltx2" and i == sp.steps - 1
                    x = x + ((0.0 - s) if last else (s_next - s)) * v
        finally:
            self.model.train(was_training)
        z = self.a.to_latent(x, cond).float()
        return z / L.scale + L.shift, kind

    @torch.no_grad()
    def decode_to_png(self, z: torch.Tensor, out_png: str, genparams: dict) -> str:
        vae = self._build_vae()
        os.makedirs(os.path.dirname(out_png) or ".", exist_ok=True)
        if z.dim() == 5:
            vid = vae.decode(z.to(self.dtype))[0].float().permute(1, 2, 3, 0).cpu()
            fdir = out_png[:-4] + ".frames"
            os.makedirs(fdir, exist_ok=True)
            for k in range(vid.shape[0]):
                with open(os.path.join(fdir, f"{k:04d}.png"), "wb") as fh:
                    fh.write(encode_png(tensor_to_uint8(vid[k]).numpy(), {}))
            arr = tensor_to_uint8(vid[0]).numpy()
        else:
            zz = z.to(self.device, self.dtype)
            from ..models.vae_factory import decode_latent
            img = decode_latent(vae, zz)
            arr = tensor_to_uint8(img[0].float().permute(1, 2, 0).cpu()).numpy()
        tmp = out_png + ".tmp"
        with open(tmp, "wb") as fh:
            fh.write(encode_png(arr, {"serenity.genparams.v1": json.dumps(genparams, separators=(",", ":"))}))
        os.replace(tmp, out_png)
        if not self.keep_vae and not self.tiny:
            del vae
            if self.device.type == "cuda":
                torch.cuda.empty_cache()
        return out_png

    # ---- pixel-space families (no VAE): the model's own sampling loop gives the image ------------------------------------
    PIXEL_FAMILIES = ("zimage_l2p", "sensenova_u1")

    @torch.no_grad()
    def _pixel_image(self, sp: SamplePrompt) -> tuple:
        """-> (image [1, 3, H, W] in [-1, 1], text kind)."""
        dev, dt, fam = self.device, self.dtype, self.m.family
        seed = int(sp.seed) & 0x7FFFFFFFFFFFFFFF
        noise = torch.randn(1, 3, sp.height, sp.width, generator=torch.Generator().manual_seed(seed)).to(dev)
        if fam == "zimage_l2p":
            from ..models.zimage_l2p import l2p_sample
            txt, _, kind = self._text(sp, False)
            un = self._text(sp, True)[0].to(dev, dt) if sp.cfg > 1.0 else None
            img = l2p_sample(self.model, txt.to(dev, dt), un, sp.height, sp.width, steps=sp.steps, cfg_scale=sp.cfg,
                             shift=self.m.schedule.shift, x=noise)
            return img.float().clamp(-1, 1), kind
        # SenseNova-U1: the prompt is token ids (the model embeds them itself); without a tokenizer the ids are a hash of the words
        vocab = self.model.cfg.vocab_size
        ids = lambda s: [1 + (zlib.crc32(w.encode()) % (vocab - 1)) for w in (s.split() or ["<empty>"])][:self.m.text.tokens]
        img = self.model.sample(ids(sp.prompt), ids(sp.negative or ""), sp.height, sp.width, steps=sp.steps, cfg_scale=max(sp.cfg, 1.0),
                                shift=self.m.schedule.shift, noise=noise)
        return (img.float() * 2.0 - 1.0).clamp(-1, 1), "hash-token-ids"

    def _sample_pixels(self, sp: SamplePrompt, out_png: str, gen: dict) -> str:
        t0 = time.perf_counter()
        was_training = self.model.training
        self.model.eval()
        try:
            img, kind = self._pixel_image(sp)
        finally:
            self.model.train(was_training)
        os.makedirs(os.path.dirname(out_png) or ".", exist_ok=True)
        arr = tensor_to_uint8(img[0].permute(1, 2, 0).cpu()).numpy()
        tmp = out_png + ".tmp"
        with open(tmp, "wb") as fh:
            fh.write(encode_png(arr, {"serenity.genparams.v1": json.dumps(gen, separators=(",", ":"))}))
        os.replace(tmp, out_png)
        self.last_report = {"text": kind, "denoise_s": round(time.perf_counter() - t0, 4), "decode_s": 0.0, "vae_weights": "none (pixel space)"}
        return out_png

    def sample(self, sp: SamplePrompt, out_png: str, extra: Optional[dict] = None) -> str:
        if self.m.family in self.PIXEL_FAMILIES:
            gen = {"schema": "serenity.genparams.v1", "model": self.m.model_id, "prompt": sp.prompt, "negative": sp.negative,
                   "width": sp.width, "height": sp.height, "frames": sp.frames, "steps": sp.steps, "cfg": sp.cfg, "seed": sp.seed,
                   "sampler": "euler", "prompt_id": sp.id}
            gen.update(extra or {})
            return self._sample_pixels(sp, out_png, gen)
        t0 = time.perf_counter()
        z, kind = self.denoise(sp)
        t1 = time.perf_counter()
        gen = {"schema": "serenity.genparams.v1", "model": self.m.model_id, "prompt": sp.prompt, "negative": sp.negative,
               "width": sp.width, "height": sp.height, "frames": sp.frames, "steps": sp.steps, "cfg": sp.cfg, "seed": sp.seed,
               "sampler": "euler", "prompt_id": sp.id}
        gen.update(extra or {})
        path = self.decode_to_png(z, out_png, gen)
        self.last_report = {"text": kind, "denoise_s": round(t1 - t0, 4), "decode_s": round(time.perf_counter() - t1, 4),
                            "vae_weights": getattr(self, "vae_weights", "resident")}
        return path

    def sample_all(self, prompts: List[SamplePrompt], out_dir: str, leaf: str, extra: Optional[dict] = None) -> List[str]:
        return [self.sample(sp, os.path.join(out_dir, f"{leaf}-{i}.png"), extra) for i, sp in enumerate(prompts)]
