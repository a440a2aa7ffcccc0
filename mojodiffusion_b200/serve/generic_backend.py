"""Serving backends for the Z-Image, Qwen-Image, SDXL and LTX-2 families: the same cooperative state machine as the FLUX
backend (ENCODE -> LOAD -> DENOISE x N -> DECODE, one ``step()`` per unit, phase announced before the tick that performs
it), each with its own model class, latent layout, schedule and guidance rule:

* ``zimage``   single-stream DiT, 16-channel VAE, 2x2 patch tokens, shifted flow-matching Euler, textbook CFG with a
  negative prompt (two forwards per step), model timestep ``1 - sigma`` (serenitymojo/serve/zimage_backend.mojo,
  pipeline/zimage_sample_cli.mojo).
* ``qwenimage`` 60-layer MMDiT, dynamic-shift schedule with terminal 0.02, true CFG with norm rescale
  (serenitymojo/serve/qwenimage_backend.mojo).
* ``sdxl``     UNet, eps-prediction Euler over the scaled-linear DDPM grid, CFG, ``y`` = pooled text + six sinusoidal
  size / crop ids (serenitymojo/serve/sdxl_backend.mojo).
* ``sd3``      SD3.5 joint-block MMDiT on [1,16,h,w] latents (patch embedding inside the model), shift-3 flow-matching
  Euler, textbook CFG, context = CLIP (77) + T5 (256) tokens with a 2048-wide pooled vector
  (serenitymojo/serve/sd3_backend.mojo).
* ``klein``    FLUX.2 Klein MMDiT (shared modulation, SwiGLU), 32-channel VAE packed 2x2 into 128-wide tokens, the
  empirical-mu schedule of FLUX.2, textbook CFG for the non-distilled checkpoints (serenitymojo/serve/klein_backend.mojo).
* ``chroma``   Chroma MMDiT (one distilled guidance layer instead of per-block modulation), 16-channel VAE, T5 text,
  shift-1.15 schedule, textbook CFG (serenitymojo/pipeline/chroma_sample_cli.mojo).
* ``ltx2``     48-layer video DiT over [frames x h x w] latent tokens, linear-quadratic (distilled) sigmas, Euler with
  the last step landing on ``x - v * sigma``, textbook CFG; the 128-channel video VAE expands 8x in time and 32x in space;
  frames are written as ``<job>.frames/NNNN.png`` and the first frame as the job's output image; the frame count comes
  from ``"frames"`` in the request's parameter JSON (default 9) (serenitymojo/pipeline/ltx2_sample_cli.mojo,
  sampling/ltx2_sampling.mojo).

Weights are read from ``MDB_MODEL_DIR`` (``<model>.safetensors`` with the key names of the model classes, VAE from the
request's ``vae`` or the family default). Without a checkpoint the backend runs the same path on deterministic random
weights and says so in its result sidecar (``"weights": "random-init"``); ``MDB_ARCH=tiny`` selects the tiny
architectures (CPU tests). Text conditioning comes from pre-encoded caption files (``sample_caps_pos`` / ``_neg``:
``text_embedding`` [1,T,D], optional ``pooled``) or, failing that, from a deterministic embedding of the prompt hash."""
from __future__ import annotations

import dataclasses
import json
import math
import os
import time
from typing import Optional

import torch

from ..io.png import encode_png, tensor_to_uint8
from ..io.safetensors_io import load_safetensors
from ..sampling import flow_match as fm
from ..sampling.guidance import cfg_textbook, cfg_true_with_norm_rescale
from ..utils.tracing import nvtx_range
from .backend import GenBackend, JobParams, StepResult, UnsupportedParam, reject_unsupported_common
from .flux_backend import prompt_embedding

KINDS = ("zimage", "qwenimage", "sdxl", "sd15", "ltx2", "sd3", "klein", "chroma")
_REFUSED: dict = {}


def _size_ids(values, dim: int = 256) -> torch.Tensor:
    """SDXL micro-conditioning: each scalar -> sinusoidal(dim), concatenated."""
    half = dim // 2
    freqs = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32) / half)
    out = []
    for v in values:
        a = float(v) * freqs
        out.append(torch.cat((torch.cos(a), torch.sin(a))))
    return torch.cat(out)[None]


class GenericBackend(GenBackend):
    def __init__(self, kind: str, device: Optional[str] = None):
        if kind in _REFUSED:
            self._refusal = f"{kind}: {_REFUSED[kind]}"
        elif kind not in KINDS:
            raise ValueError(f"no backend for kind '{kind}'")
        else:
            self._refusal = ""
        self.kind = self.name = kind
        self.variant = kind
        if kind == "sd15":                    # the SDXL loop (eps prediction over the DDPM grid) around the SD1.5 UNet shape
            self.kind = "sdxl"
        self.tiny = os.environ.get("MDB_ARCH", "") == "tiny"
        self.device = torch.device(device or ("cuda" if torch.cuda.is_available() else "cpu"))
        self.dtype = torch.bfloat16 if self.device.type == "cuda" else torch.float32
        self.model = self.vae = None
        self.loaded_name = ""
        self.weights_kind = ""
        self.p: Optional[JobParams] = None
        self._cancel = False
        self.phase = "idle"
        self.stage_s = {}

    def resident_model(self) -> str:
        return self.loaded_name

    # ---- job -----------------------------------------------------------------------------------------------
    def start(self, params: JobParams) -> None:
        if self._refusal:
            raise NotImplementedError(self._refusal)
        reject_unsupported_common(params, img2img=False, inpaint=False, lora=False, variation=False)
        s = (params.sampler or "euler").lower()
        if s not in ("euler", "flowmatch_euler", "flow_match_euler"):
            raise UnsupportedParam(f"{self.kind}: the serving loop implements the euler sampler, not '{params.sampler}'")
        self.p, self._cancel, self.phase, self.i = params, False, "encode", 0
        self.stage_s = {}

    def cancel(self) -> None:
        self._cancel = True

    def step(self) -> StepResult:
        p = self.p
        if p is None:
            return StepResult("failed", error=f"{self.kind}: no active job")
        if self._cancel:
            self.p, self.phase = None, "idle"
            return StepResult("cancelled")
        t0 = time.perf_counter()
        if self.phase == "encode":
            with nvtx_range("stage/encode"):
                self._encode(p)
            self.stage_s["encode"] = time.perf_counter() - t0
            self.phase = "load"
            return StepResult("progress", 0, p.steps, "load")
        if self.phase == "load":
            with nvtx_range("stage/load"):
                self._load(p)
                self._prepare(p)
            self.stage_s["load"] = time.perf_counter() - t0
            self.phase = "denoise"
            return StepResult("progress", 0, p.steps, "denoise")
        if self.phase == "denoise":
            with nvtx_range(f"stage/denoise/{self.i}"):
                self._denoise_step(p)
            self.stage_s["denoise"] = self.stage_s.get("denoise", 0.0) + time.perf_counter() - t0
            self.i += 1
            if self.i >= p.steps:
                self.phase = "decode"
                return StepResult("progress", p.steps, p.steps, "decode")
            return StepResult("progress", self.i, p.steps, "denoise")
        with nvtx_range("stage/decode"):
            path = self._decode_and_save(p)
        self.stage_s["decode"] = time.perf_counter() - t0
        self._write_sidecar(p, path)
        self.p, self.phase = None, "idle"
        return StepResult("done", output_path=path)

    def trim(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.empty_cache()

    # ---- family tables ---------------------------------------------------------------------------------------
    def _model_config(self):
        if self.kind == "zimage":
            from ..models import single_dit as M
            return M.tiny_single_dit_config() if self.tiny else M.zimage_config()
        if self.kind == "qwenimage":
            from ..models import qwen_image as M
            return M.tiny_qwen_image_config() if self.tiny else M.qwen_image_config()
        if self.kind == "ltx2":
            from ..models import video_dit as M
            return M.tiny_video_dit_config() if self.tiny else M.ltx2_config()
        if self.kind == "sd3":
            from ..models import sd3 as M
            return M.tiny_sd3_config() if self.tiny else M.sd35_large_config()
        if self.kind == "klein":
            from ..models import flux2 as M
            return M.tiny_flux2_config() if self.tiny else M.klein_9b_config()
        if self.kind == "chroma":
            from ..models import chroma as M
            return M.tiny_chroma_config() if self.tiny else M.chroma_config()
        from ..models import unet as M
        if self.variant == "sd15":
            return M.tiny_sd15_config() if self.tiny else M.sd15_config()
        return M.tiny_unet_config() if self.tiny else M.sdxl_config()

    def _vae_config(self):
        from ..models import vae as V
        zc = 4 if self.kind == "sdxl" else 16
        if self.tiny:
            if self.kind in ("klein", "chroma"):
                zc = self.cfg.in_channels // 4
            return dataclasses.replace(V.tiny_vae_config(), z_channels=self.cfg.in_channels if self.kind == "sd3" else zc)
        if self.kind == "sd3":
            return V.sd3_vae_config()
        if self.kind == "klein":
            return V.flux2_vae_config()
        return V.sdxl_vae_config() if self.kind == "sdxl" else V.flux_vae_config()

    def _text_shape(self, cfg):
        if self.kind == "zimage":
            return (32 if self.tiny else 128), cfg.cap_dim, 0
        if self.kind in ("qwenimage", "ltx2"):
            return (32 if self.tiny else 256), cfg.context_dim, 0
        if self.kind in ("klein", "chroma"):
            return (32 if self.tiny else 512), cfg.context_dim, 0
        if self.kind == "sd3":
            return (24 if self.tiny else 333), cfg.context_dim, cfg.pooled_dim
        if cfg.adm_in_channels == 0:            # SD1.5: no pooled / size conditioning
            return 77, cfg.context_dim, 0
        return 77, cfg.context_dim, cfg.adm_in_channels - 6 * 256 if not self.tiny else cfg.adm_in_channels

    # ---- phases -------------------------------------------------------------------------------------------------
    def _read_caps(self, path: str, prompt: str, T: int, D: int, P: int):
        if path and os.path.isfile(path):
            d = load_safetensors(path)
            pooled = d["pooled"].float() if "pooled" in d else torch.zeros(1, max(P, 1))
            return d["text_embedding"].float(), pooled, "pre-encoded"
        txt, pooled = prompt_embedding(prompt, T, D, max(P, 1))
        return txt, pooled, "hash-embedding"

    def _encode(self, p: JobParams) -> None:
        self.cfg = cfg = self._model_config()
        T, D, P = self._text_shape(cfg)
        self.use_cfg = p.cfg > 1.0
        if self._encode_in_child(p, D, P):
            return
        self.txt, self.pooled, self.text_kind = self._read_caps(p.sample_caps_pos, p.prompt, T, D, P)
        if self.use_cfg:
            self.txt_neg, self.pooled_neg, _ = self._read_caps(p.sample_caps_neg, p.negative, self.txt.shape[1], D, P)

    def _encode_in_child(self, p: JobParams, D: int, P: int) -> bool:
        """Real text encoders in a child process that exits afterwards (``MDB_ENCODERS_DIR=<dir>``; with the tiny
        architectures ``MDB_ENCODE_SUBPROCESS=1`` runs tiny random-weight encoders through the same protocol). Pre-encoded
        caption files still win. Returns False when this path is not configured for the family."""
        from .encode_subprocess import FAMILY_ENCODERS, encode_in_child
        enc_dir = os.environ.get("MDB_ENCODERS_DIR", "")
        tiny_child = self.tiny and os.environ.get("MDB_ENCODE_SUBPROCESS", "") == "1"
        if self.kind not in FAMILY_ENCODERS or not (enc_dir or tiny_child) or (p.sample_caps_pos and os.path.isfile(p.sample_caps_pos)):
            return False
        res = encode_in_child(self.kind, p.prompt, p.negative if self.use_cfg else None, enc_dir, tiny_child,
                              device="cpu" if self.device.type == "cpu" else "")

        def fit(t, width):                      # tiny encoders are narrower than the tiny backbones' text inputs
            return t if t.shape[-1] == width else torch.nn.functional.pad(t, (0, width - t.shape[-1])) if t.shape[-1] < width else t[..., :width]
        self.txt, self.pooled = fit(res["text_embedding"].float(), D), fit(res["pooled"].float(), max(P, 1))
        if self.use_cfg:
            self.txt_neg, self.pooled_neg = fit(res["neg_text_embedding"].float(), D), fit(res["neg_pooled"].float(), max(P, 1))
            n = min(self.txt.shape[1], self.txt_neg.shape[1])
            self.txt, self.txt_neg = self.txt[:, :n], self.txt_neg[:, :n]
        self.text_kind = "encoder-subprocess"
        self.encoder_pid = int(res["child_pid"][0])
        return True

    def _load(self, p: JobParams) -> None:
        from ..models.vae import AutoencoderKL
        if self.model is not None and self.loaded_name == p.model:
            return
        self.model = self.vae = None
        self.trim()
        if self.kind == "zimage":
            from ..models.single_dit import SingleStreamDiT as Cls
        elif self.kind == "qwenimage":
            from ..models.qwen_image import QwenImageDiT as Cls
        elif self.kind == "ltx2":
            from ..models.video_dit import VideoDiT as Cls
        elif self.kind == "sd3":
            from ..models.sd3 import SD3MMDiT as Cls
        elif self.kind == "klein":
            from ..models.flux2 import Flux2DiT as Cls
        elif self.kind == "chroma":
            from ..models.chroma import ChromaDiT as Cls
        else:
            from ..models.unet import UNet as Cls
        model = Cls(self.cfg, self.dtype, self.device)
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
        if self.kind == "ltx2":
            from ..models.video_vae import VideoVAE, ltx2_vae_config, tiny_video_vae_config
            vcfg = dataclasses.replace(tiny_video_vae_config(), latent_channels=self.cfg.in_channels) if self.tiny else ltx2_vae_config()
            vae = VideoVAE(vcfg, self.dtype, self.device)
        elif self.tiny or self.kind not in ("klein", "qwenimage", "zimage"):
            vae = AutoencoderKL(self._vae_config(), self.dtype, self.device, with_encoder=False)
        else:                                   # families whose autoencoder is not the plain LDM one
            from ..models.vae_factory import build_family_vae
            vae = build_family_vae(self.kind, self.dtype, self.device, False)
        vpath = os.path.join(root, p.vae) if (root and p.vae) else ""
        if vpath and os.path.isfile(vpath):
            from ..models.vae_factory import load_vae_weights
            load_vae_weights(vae, vpath, self.device, self.dtype)
        else:
            vae.init_weights(seed=1)
        self.model, self.vae = model.eval(), vae.eval()
        self.loaded_name = p.model

    def _prepare(self, p: JobParams) -> None:
        from ..models.mmdit import pack_latents
        dev, dt = self.device, self.dtype
        g = torch.Generator().manual_seed(int(p.seed) & 0x7FFFFFFFFFFFFFFF)
        self.txt_d = self.txt.to(dev, dt)
        if self.use_cfg:
            self.txt_neg_d = self.txt_neg.to(dev, dt)
        self.t = torch.empty(1, device=dev)
        if self.kind == "ltx2":
            ft, fs = self.vae.expansion()
            frames = 9
            try:
                frames = int(json.loads(p.params_json).get("frames", frames)) if p.params_json else frames
            except (ValueError, AttributeError):
                pass
            if p.width % fs or p.height % fs:
                raise UnsupportedParam(f"ltx2: width/height must be multiples of {fs}")
            F_lat = 1 + max(frames - 1, 0) // ft
            self.grid = (F_lat, p.height // fs, p.width // fs)
            C = self.cfg.in_channels
            noise = torch.randn(1, self.grid[0] * self.grid[1] * self.grid[2], C, generator=g)
            self.sigmas = fm.ltx2_linear_quadratic_sigmas(p.steps)
            self.x = noise.float().to(dev)
            return
        from ..models.vae_factory import latent_geometry
        C, f = latent_geometry(self.vae)
        h, w = p.height // f, p.width // f
        noise = torch.randn(1, C, h, w, generator=g)
        if self.kind == "sdxl":
            from ..sampling.ddpm import SDXLEulerScheduler
            self.sched = SDXLEulerScheduler(p.steps)
            self.x = (noise * self.sched.init_noise_sigma).float().to(dev)
            if self.cfg.adm_in_channels == 0:
                self.y = self.y_neg = None
            elif self.tiny:
                self.y = self.pooled.to(dev, dt)
                self.y_neg = self.pooled_neg.to(dev, dt) if self.use_cfg else None
            else:
                ids = _size_ids((p.height, p.width, 0, 0, p.height, p.width))
                self.y = torch.cat((self.pooled, ids), 1).to(dev, dt)
                self.y_neg = torch.cat((self.pooled_neg, ids), 1).to(dev, dt) if self.use_cfg else None
            return
        if self.kind == "sd3":
            self.sigmas = fm.sd3_sigmas(p.steps, p.sigma_shift if p.sigma_shift > 0 else 3.0)
            self.x = noise.float().to(dev)
            self.y = self.pooled.to(dev, dt)
            self.y_neg = self.pooled_neg.to(dev, dt) if self.use_cfg else None
            return
        self.hw = (h // 2, w // 2)
        S_img = self.hw[0] * self.hw[1]
        if self.kind == "qwenimage":
            self.sigmas = fm.qwen_image_sigmas(p.steps, S_img)
        elif self.kind == "klein":
            self.sigmas = fm.flux2_klein_sigmas(p.steps, S_img)
        elif self.kind == "chroma":
            self.sigmas = fm.shifted_sigmas(p.steps, 1.15)
        else:
            self.sigmas = fm.shifted_sigmas(p.steps, p.sigma_shift if p.sigma_shift > 0 else 3.0)
        self.x = pack_latents(noise).float().to(dev)

    @torch.no_grad()
    def _denoise_step(self, p: JobParams) -> None:
        i = self.i
        if self.kind == "sdxl":
            t = self.sched.timesteps[i]
            self.t.fill_(float(t))
            xin = self.sched.scale_model_input(self.x, i).to(self.dtype)
            eps = self.model(xin, self.t, self.txt_d, self.y).float()
            if self.use_cfg:
                eu = self.model(xin, self.t, self.txt_neg_d, self.y_neg).float()
                eps = cfg_textbook(eps, eu, p.cfg)
            self.x = self.sched.step(self.x, eps, i)
            return
        s, s_next = float(self.sigmas[i]), float(self.sigmas[i + 1])
        xb = self.x.to(self.dtype)
        if self.kind == "ltx2":
            self.t.fill_(s)
            v = self.model(xb, self.txt_d, self.t, self.grid).float()
            if self.use_cfg:
                v = cfg_textbook(v, self.model(xb, self.txt_neg_d, self.t, self.grid).float(), p.cfg)
            last = i == p.steps - 1
            self.x = self.x + ((0.0 - s) if last else (s_next - s)) * v       # the final step lands on x - v * sigma
            return
        if self.kind == "sd3":
            self.t.fill_(s)
            v = self.model(xb, self.txt_d, self.t, self.y).float()
            if self.use_cfg:
                v = cfg_textbook(v, self.model(xb, self.txt_neg_d, self.t, self.y_neg).float(), p.cfg)
            self.x = self.x + (s_next - s) * v
            return
        if self.kind == "zimage":
            self.t.fill_(1.0 - s)                         # the model's clock runs from noise (0) to image (1)
            v = -self.model(xb, self.txt_d, self.t, self.hw).float()
            if self.use_cfg:
                vu = -self.model(xb, self.txt_neg_d, self.t, self.hw).float()
                v = cfg_textbook(v, vu, p.cfg)
        else:
            self.t.fill_(s)
            v = self.model(xb, self.txt_d, self.t, self.hw).float()
            if self.use_cfg:
                vu = self.model(xb, self.txt_neg_d, self.t, self.hw).float()
                v = cfg_true_with_norm_rescale(v, vu, p.cfg) if self.kind == "qwenimage" else cfg_textbook(v, vu, p.cfg)
        self.x = self.x + (s_next - s) * v

    @torch.no_grad()
    def _decode_and_save(self, p: JobParams) -> str:
        from ..models.mmdit import unpack_latents
        if self.kind == "ltx2":
            return self._decode_video(p)
        z = self.x if self.kind in ("sdxl", "sd3") else unpack_latents(self.x, self.hw[0], self.hw[1])
        from ..models.vae_factory import decode_latent
        img = decode_latent(self.vae, z)
        arr = tensor_to_uint8(img[0].float().permute(1, 2, 0).cpu()).numpy()
        os.makedirs(p.out_dir or ".", exist_ok=True)
        path = p.output_path()
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(encode_png(arr, {"serenity.genparams.v1": p.genparams_text()}))
        os.replace(tmp, path)
        return path

    def _decode_video(self, p: JobParams) -> str:
        Fl, H, W = self.grid
        z = self.x.reshape(1, Fl, H, W, -1).permute(0, 4, 1, 2, 3)
        vid = self.vae.decode(z.to(self.dtype))[0].float().permute(1, 2, 3, 0).cpu()       # [T, H, W, 3]
        os.makedirs(p.out_dir or ".", exist_ok=True)
        path = p.output_path()
        fdir = path[:-4] + ".frames"
        os.makedirs(fdir, exist_ok=True)
        self.frames_written = int(vid.shape[0])
        for t in range(vid.shape[0]):
            arr = tensor_to_uint8(vid[t]).numpy()
            with open(os.path.join(fdir, f"{t:04d}.png"), "wb") as f:
                f.write(encode_png(arr, {}))
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(encode_png(tensor_to_uint8(vid[0]).numpy(), {"serenity.genparams.v1": p.genparams_text()}))
        os.replace(tmp, path)
        return path

    def _write_sidecar(self, p: JobParams, path: str) -> None:
        peak = torch.cuda.max_memory_allocated() if self.device.type == "cuda" else 0
        side = {"schema": f"serenity.{self.variant}.daemon_result.v1", "job_id": p.job_id, "model": p.model,
                "weights": self.weights_kind, "text": self.text_kind, "encoder_pid": getattr(self, "encoder_pid", 0),
                "cfg": p.cfg if self.use_cfg else 1.0,
                "stage_seconds": {k: round(v, 4) for k, v in self.stage_s.items()}, "peak_device_bytes": int(peak),
                "steps_run": p.steps, "sampler": "euler", "device": str(self.device)}
        if self.kind == "ltx2":
            side["frames"] = self.frames_written
            side["frames_dir"] = path[:-4] + ".frames"
        with open(path + ".worker_result.json", "w") as f:
            json.dump(side, f)
