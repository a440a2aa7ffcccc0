"""Model manifests: one record per model id that names everything a pipeline, a trainer or a worker needs to know about
a checkpoint family without opening it: backbone class and configuration, latent layout, text-conditioning shape and
encoders, sampler schedule and guidance defaults, LoRA key scheme, block-swap plan, worker kind, and whether the profile
is admitted for serving.

Plays the role of the reference's ``ModelManifest`` and its per-model defaults
(serenitymojo/runtime/model_manifest.mojo:47-526), ``default_manifest_by_id`` (serenitymojo/registry/checkpoints.mojo:578),
``ExecutionConfig`` / ``ShapeProfile`` (serenitymojo/runtime/) and the production guard that refuses blocked profiles
loudly (serenity-server/crates/server/src/capabilities.rs:17-39). Shapes are runtime values here: a manifest lists the
resolution buckets a family is exercised on, not one binary per bucket.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class LatentSpec:
    channels: int                  # VAE latent channels
    vae_factor: int                # pixels per latent cell (8 for the LDM family, 32 for the LTX-2 video VAE)
    patch: int = 2                 # DiT patch size (tokens = (h / patch) * (w / patch)); 1 for UNet / patch-in-model
    packed: bool = True            # True: the model consumes [B, tokens, channels * patch^2]; False: [B, C, h, w]
    temporal_factor: int = 1       # frames per latent frame (video)
    scale: float = 1.0             # latent = (z - shift) * scale on the way into the model
    shift: float = 0.0


@dataclass(frozen=True)
class TextSpec:
    tokens: int
    dim: int
    pooled_dim: int = 0
    encoders: Tuple[str, ...] = ()   # "clip_l", "clip_g", "t5_xxl", "umt5", "qwen3", "qwen25_vl", "gemma"
    key_mask: bool = False           # padded text keys are masked in joint attention


@dataclass(frozen=True)
class ScheduleSpec:
    kind: str                      # flux1 | flux2_klein | qwen_image | shifted | sd3 | ltx2_linear_quadratic | sdxl_ddpm
    steps: int = 20
    cfg: float = 1.0               # default guidance scale (1.0 = single forward)
    shift: float = 3.0
    cfg_rule: str = "textbook"     # textbook | true_norm_rescale | distilled (guidance fed to the model)
    prediction: str = "flow"       # flow (velocity eps - x0) | epsilon


@dataclass(frozen=True)
class LoraSpec:
    injector: str                  # function of training.lora
    layout: str                    # onetrainer | peft
    state_layout: str = "peft"     # key scheme of the train-state sidecar


@dataclass(frozen=True)
class ModelManifest:
    model_id: str
    family: str                    # worker kind / adapter name: flux, klein, qwenimage, zimage, sd3, chroma, sdxl, ltx2, wan22
    module: str                    # python module of the backbone
    model_class: str
    config_fn: str
    tiny_config_fn: str
    latent: LatentSpec
    text: TextSpec
    schedule: ScheduleSpec
    lora: Optional[LoraSpec]
    vae_config_fn: str = "flux_vae_config"
    offload_plan: str = ""         # builder in offload.plan
    param_billions: float = 0.0
    buckets: Tuple[Tuple[int, int], ...] = ((1024, 1024),)   # (width, height) the family is exercised on
    blocked: str = ""              # non-empty: the profile is refused for serving, with this reason
    full_finetune: bool = False    # a runnable full-finetune loop exists
    notes: str = ""

    # ---- constructors -------------------------------------------------------------------------------------
    def _mod(self):
        return importlib.import_module(self.module)

    def config(self, tiny: bool = False):
        return getattr(self._mod(), self.tiny_config_fn if tiny else self.config_fn)()

    def build(self, tiny: bool = False, dtype=None, device=None, cfg=None):
        import torch
        cfg = cfg if cfg is not None else self.config(tiny)
        dtype = dtype if dtype is not None else torch.float32
        return getattr(self._mod(), self.model_class)(cfg, dtype, device)

    def tokens_for(self, width: int, height: int, frames: int = 1) -> int:
        f = self.latent.vae_factor * self.latent.patch
        t = 1 + max(frames - 1, 0) // self.latent.temporal_factor if self.latent.temporal_factor > 1 else 1
        return (height // f) * (width // f) * t


# ---- registry ---------------------------------------------------------------------------------------------------
_REG: Dict[str, ModelManifest] = {}
_ALIASES: Dict[str, str] = {}


def register(m: ModelManifest, *aliases: str) -> ModelManifest:
    _REG[m.model_id] = m
    for a in aliases:
        _ALIASES[a] = m.model_id
    return m


def manifest_ids() -> List[str]:
    return sorted(_REG)


def default_manifest_by_id(model_id: str) -> ModelManifest:
    """Manifest for a model id or one of its aliases (family names, checkpoint file stems). Raises KeyError with the
    list of known ids otherwise: an unknown model must never fall through to some default family."""
    key = model_id.strip()
    low = key.lower().replace("_", "-")
    for cand in (key, low, _ALIASES.get(key, ""), _ALIASES.get(low, "")):
        if cand in _REG:
            return _REG[cand]
    stem = low.rsplit("/", 1)[-1].removesuffix(".safetensors")
    for a, mid in _ALIASES.items():
        if stem.startswith(a):
            return _REG[mid]
    raise KeyError(f"no manifest for model '{model_id}'; known: {', '.join(manifest_ids())}")


def manifest_for_family(family: str) -> ModelManifest:
    for m in _REG.values():
        if m.family == family:
            return m
    raise KeyError(f"no manifest of family '{family}'")


_M = "mojodiffusion_b200.models."

register(ModelManifest(
    "flux1-dev", "flux", _M + "mmdit", "MMDiT", "flux1_dev_config", "tiny_mmdit_config",
    LatentSpec(16, 8, 2, True, scale=0.3611, shift=0.1159), TextSpec(512, 4096, 768, ("clip_l", "t5_xxl")),
    ScheduleSpec("flux1", 20, 3.5, cfg_rule="distilled"), LoraSpec("inject_flux_lora", "onetrainer"),
    "flux_vae_config", "flux_plan", 12.0, ((1024, 1024), (768, 1344), (1344, 768), (512, 512))),
    "flux", "flux1", "flux.1-dev", "flux1-schnell")
register(ModelManifest(
    "flux2-klein-9b", "klein", _M + "flux2", "Flux2DiT", "klein_9b_config", "tiny_flux2_config",
    LatentSpec(32, 8, 2, True), TextSpec(512, 12288, 0, ("qwen3",)),
    ScheduleSpec("flux2_klein", 20, 4.0), LoraSpec("inject_klein_lora", "peft"),
    "flux2_vae_config", "klein_plan", 9.0, ((1024, 1024), (512, 512))),
    "klein", "flux2", "klein-9b", "flux2-klein")
register(ModelManifest(
    "flux2-klein-4b", "klein", _M + "flux2", "Flux2DiT", "klein_4b_config", "tiny_flux2_config",
    LatentSpec(32, 8, 2, True), TextSpec(512, 7680, 0, ("qwen3",)),
    ScheduleSpec("flux2_klein", 20, 4.0), LoraSpec("inject_klein_lora", "peft"),
    "flux2_vae_config", "klein_plan", 4.0, ((1024, 1024), (512, 512))),
    "klein-4b")
register(ModelManifest(
    "qwen-image", "qwenimage", _M + "qwen_image", "QwenImageDiT", "qwen_image_config", "tiny_qwen_image_config",
    LatentSpec(16, 8, 2, True), TextSpec(256, 3584, 0, ("qwen25_vl",), key_mask=True),
    ScheduleSpec("qwen_image", 20, 4.0, cfg_rule="true_norm_rescale"), LoraSpec("inject_qwen_lora", "onetrainer"),
    "flux_vae_config", "qwenimage_plan", 20.0, ((1024, 1024), (1328, 1328)), full_finetune=True),
    "qwenimage", "qwen_image", "qwen")
register(ModelManifest(
    "z-image", "zimage", _M + "single_dit", "SingleStreamDiT", "zimage_config", "tiny_single_dit_config",
    LatentSpec(16, 8, 2, True, scale=0.3611, shift=0.1159), TextSpec(128, 2560, 0, ("qwen3",)),
    ScheduleSpec("shifted", 28, 3.5, shift=3.0), LoraSpec("inject_zimage_lora", "peft"),
    "flux_vae_config", "zimage_plan", 6.15, ((1024, 1024), (512, 512)), full_finetune=True),
    "zimage", "z_image", "zimage-turbo")
register(ModelManifest(
    "sd35-large", "sd3", _M + "sd3", "SD3MMDiT", "sd35_large_config", "tiny_sd3_config",
    LatentSpec(16, 8, 1, False, scale=1.5305, shift=0.0609), TextSpec(333, 4096, 2048, ("clip_l", "clip_g", "t5_xxl")),
    ScheduleSpec("sd3", 28, 4.5, shift=3.0), None, "sd3_vae_config", "sd35_plan", 8.1),
    "sd3", "sd35", "sd3.5-large")
register(ModelManifest(
    "sd35-medium", "sd3", _M + "sd3", "SD3MMDiT", "sd35_medium_config", "tiny_sd3_config",
    LatentSpec(16, 8, 1, False, scale=1.5305, shift=0.0609), TextSpec(333, 4096, 2048, ("clip_l", "clip_g", "t5_xxl")),
    ScheduleSpec("sd3", 28, 4.5, shift=3.0), None, "sd3_vae_config", "sd35_plan", 2.5),
    "sd3.5-medium")
register(ModelManifest(
    "chroma", "chroma", _M + "chroma", "ChromaDiT", "chroma_config", "tiny_chroma_config",
    LatentSpec(16, 8, 2, True, scale=0.3611, shift=0.1159), TextSpec(512, 4096, 0, ("t5_xxl",)),
    ScheduleSpec("shifted", 26, 4.0, shift=1.15), None, "flux_vae_config", "chroma_plan", 8.9,
    blocked="profile kept off the serving allow-list (fails loudly), as in the reference's capability table"),
    "chroma1-hd")
register(ModelManifest(
    "sdxl", "sdxl", _M + "unet", "UNet", "sdxl_config", "tiny_unet_config",
    LatentSpec(4, 8, 1, False, scale=0.13025), TextSpec(77, 2048, 1280, ("clip_l", "clip_g")),
    ScheduleSpec("sdxl_ddpm", 30, 7.0, cfg_rule="textbook", prediction="epsilon"), LoraSpec("inject_sdxl_lora", "onetrainer"),
    "sdxl_vae_config", "sdxl_plan", 2.6, ((1024, 1024), (832, 1216), (1216, 832))),
    "sdxl-base", "sd_xl")
register(ModelManifest(
    "sd15", "sdxl", _M + "unet", "UNet", "sd15_config", "tiny_sd15_config",
    LatentSpec(4, 8, 1, False, scale=0.18215), TextSpec(77, 768, 0, ("clip_l",)),
    ScheduleSpec("sdxl_ddpm", 30, 7.5, cfg_rule="textbook", prediction="epsilon"), LoraSpec("inject_sdxl_lora", "onetrainer"),
    "sdxl_vae_config", "sdxl_plan", 0.86, ((512, 512), (512, 768), (768, 512)),
    notes="the SDXL worker family with the SD1.5 UNet shape (no size / pooled conditioning)"),
    "sd-v1-5", "v1-5", "stable-diffusion-v1-5")
register(ModelManifest(
    "ltx2", "ltx2", _M + "video_dit", "VideoDiT", "ltx2_config", "tiny_video_dit_config",
    LatentSpec(128, 32, 1, True, temporal_factor=8), TextSpec(256, 4096, 0, ("gemma",)),
    ScheduleSpec("ltx2_linear_quadratic", 40, 3.0), LoraSpec("inject_ltx2_lora", "peft"),
    "", "ltx2_plan", 22.0, ((768, 512),)),
    "ltx-2", "ltx2.3", "ltx-2.3")
register(ModelManifest(
    "wan22-ti2v-5b", "wan22", _M + "wan", "WanDiT", "wan22_ti2v_5b_config", "tiny_wan_config",
    LatentSpec(48, 16, 2, True, temporal_factor=4), TextSpec(512, 4096, 0, ("umt5",)),
    ScheduleSpec("shifted", 40, 5.0, shift=5.0), None, "", "wan22_plan", 5.0, ((1280, 704),)),
    "wan22", "wan2.2")
register(ModelManifest(
    "ernie-image", "ernie", _M + "ernie", "ErnieImage", "ernie_config", "tiny_ernie_config",
    LatentSpec(128, 16, 1, False), TextSpec(256, 3072, 0, ("mistral3b",), key_mask=True),
    ScheduleSpec("shifted", 50, 4.0, shift=3.0), LoraSpec("inject_ernie_lora", "peft"),
    "klein_vae_config", "", 8.0, ((1024, 1024),), notes="latents are the packed 128-channel FLUX.2 VAE latents at 1/16"),
    "ernie", "ernie-image-8b")
register(ModelManifest(
    "anima", "anima", _M + "anima", "Anima", "anima_config", "tiny_anima_config",
    LatentSpec(16, 8, 1, False), TextSpec(256, 1024, 0, ("qwen3", "t5_adapter")),
    ScheduleSpec("shifted", 30, 4.0, shift=3.0), LoraSpec("inject_anima_lora", "peft"),
    "flux_vae_config", "", 2.0, ((1024, 1024),), notes="2 x 2 patches and the mask channel are added inside the model"),
    "anima-minitraindit")

_NO_PIPELINE = "the backbone and its parity tests exist; no sampler adapter, serving backend or trainer adapter is wired"
register(ModelManifest(
    "ideogram-4", "ideogram4", _M + "ideogram4", "Ideogram4DiT", "Ideogram4Config", "tiny_ideogram4_config",
    LatentSpec(128, 16, 1, True), TextSpec(512, 53248, 0, ("qwen3_vl_stacked",)),
    ScheduleSpec("logit_normal", 30, 1.0), None, "klein_vae_config", "", 10.6, ((1024, 1024),), blocked=_NO_PIPELINE,
    notes="text and image tokens share one sequence; an indicator per position selects the embedding path"),
    "ideogram4")
register(ModelManifest(
    "hunyuan-video-1.5", "hunyuan15", _M + "hunyuan15", "Hunyuan15DiT", "Hunyuan15Config", "tiny_hunyuan15_config",
    LatentSpec(32, 16, 1, False, temporal_factor=4), TextSpec(1000, 2048, 0, ("qwen25_vl", "byt5")),
    ScheduleSpec("shifted", 50, 6.0, shift=7.0), None, "", "", 8.3, ((1280, 720),), blocked=_NO_PIPELINE,
    notes="65 input channels: latent, condition latent and mask are concatenated by the caller; text arrives projected"),
    "hunyuan15", "hunyuanvideo-1.5")
register(ModelManifest(
    "kandinsky-5-t2v-lite", "kandinsky5", _M + "kandinsky5", "Kandinsky5DiT", "Kandinsky5Config", "tiny_kandinsky5_config",
    LatentSpec(16, 8, 2, False, temporal_factor=4), TextSpec(256, 3584, 768, ("qwen25_vl", "clip_l")),
    ScheduleSpec("shifted", 50, 5.0, shift=5.0), None, "", "", 2.0, ((768, 512),), blocked=_NO_PIPELINE),
    "kandinsky5", "kandinsky-5")
register(ModelManifest(
    "cosmos-predict2.5-2b", "cosmos", _M + "cosmos", "CosmosDiT", "CosmosConfig", "tiny_cosmos_config",
    LatentSpec(16, 8, 2, False, temporal_factor=4), TextSpec(512, 100352, 0, ("cosmos_reason1",)),
    ScheduleSpec("rectified_flow_unipc", 35, 7.0), None, "", "", 2.0, ((1280, 704),), blocked=_NO_PIPELINE),
    "cosmos", "cosmos-predict25")
register(ModelManifest(
    "wan21-vace-14b", "wan_vace", _M + "wan", "WanVaceDiT", "wan21_vace_14b_config", "tiny_wan_vace_config",
    LatentSpec(16, 8, 2, False, temporal_factor=4), TextSpec(512, 4096, 0, ("umt5",)),
    ScheduleSpec("shifted", 50, 5.0, shift=5.0), None, "", "", 14.0, ((832, 480),), blocked=_NO_PIPELINE,
    notes="control latent + mask (96 channels) enter through the VACE branch; hints feed every second base layer"),
    "wan-vace", "vace")
register(ModelManifest(
    "nucleus-image", "nucleus", _M + "nucleus", "NucleusDiT", "NucleusConfig", "tiny_nucleus_config",
    LatentSpec(16, 8, 2, True), TextSpec(512, 4096, 0, ("qwen3_vl",)),
    ScheduleSpec("shifted", 30, 4.0, shift=3.0), None, "flux_vae_config", "", 17.0, ((1024, 1024),), blocked=_NO_PIPELINE,
    notes="29 of 32 blocks are expert-choice mixtures of 64 experts plus a shared expert"),
    "nucleus")
register(ModelManifest(
    "ace-step-1.5", "acestep", _M + "acestep", "AceStepDiT", "AceStepConfig", "tiny_acestep_config",
    LatentSpec(64, 1, 2, False), TextSpec(512, 2048, 0, ("qwen3_embedding", "lyric", "timbre")),
    ScheduleSpec("shifted", 8, 1.0, shift=3.0), None, "", "", 2.0, ((1, 1),), blocked=_NO_PIPELINE,
    notes="audio: a 1-D token sequence of acoustic latents; the acoustic VAE and the condition encoder are not built"),
    "acestep", "ace-step")
register(ModelManifest(
    "krea-2", "krea2", _M + "krea2", "Krea2DiT", "Krea2Config", "tiny_krea2_config",
    LatentSpec(16, 8, 2, True), TextSpec(512, 2560, 0, ("qwen3_vl_4b_12_layers",)),
    ScheduleSpec("krea2_exp_shift", 20, 4.5, cfg_rule="cond_anchored"), LoraSpec("inject_krea2_lora", "peft"), "qwen_image_vae_config", "", 13.0,
    ((1024, 1024),),
    blocked="cli.sample, cli.train (LoRA on the single-stream blocks) and the validation sampler are wired (text features: twelve "
            "stacked encoder layers per token, flattened); no serving backend",
    notes="`models.krea2.krea2_sample` is the stand-alone sampling loop"),
    "krea2")
register(ModelManifest(
    "zimage-l2p", "zimage_l2p", _M + "zimage_l2p", "ZImageL2P", "zimage_l2p_config", "tiny_zimage_l2p_config",
    LatentSpec(3, 1, 16, False), TextSpec(512, 2560, 0, ("qwen3",)),
    ScheduleSpec("shifted", 30, 2.0, shift=3.0), None, "", "", 6.2, ((1024, 1024),),
    blocked="cli.sample and the validation sampler run the model's own pixel-space loop (no VAE); no serving backend or trainer adapter",
    notes="`models.zimage_l2p.l2p_sample` is the sampling loop"),
    "l2p")
register(ModelManifest(
    "lens", "lens", _M + "lens", "LensDiT", "LensConfig", "tiny_lens_config",
    LatentSpec(32, 8, 2, True), TextSpec(415, 11520, 0, ("gpt_oss_layers_5_11_17_23",)),
    ScheduleSpec("lens_exp_shift", 20, 5.0), LoraSpec("inject_lens_lora", "peft"), "flux2_vae_config", "", 3.1, ((1024, 1024),),
    blocked="cli.sample, cli.train (LoRA on both streams' projections) and the validation sampler are wired (text features: four "
            "encoder layers concatenated); no serving backend",
    notes="each of the four text layers is normalised by its own weight inside the model"),
    "microsoft-lens")
register(ModelManifest(
    "lance-3b-video", "lance", _M + "lance", "LanceT2V", "LanceConfig", "tiny_lance_config",
    LatentSpec(48, 16, 1, True, temporal_factor=4), TextSpec(512, 2048, 0, ()),
    ScheduleSpec("lance_shifted", 30, 4.0, shift=3.0), None, "", "", 6.5, ((848, 480),), blocked=_NO_PIPELINE,
    notes="token ids and latent tokens share one decoder; generated rows use the *_moe_gen weights; see runtime/lance_kv_plan.py"),
    "lance")
register(ModelManifest(
    "magihuman-15b", "magihuman", _M + "magihuman", "MagiHumanDiT", "MagiHumanConfig", "tiny_magihuman_config",
    LatentSpec(48, 16, 2, True, temporal_factor=4), TextSpec(512, 3584, 0, ("t5gemma",)),
    ScheduleSpec("shifted", 8, 1.0, shift=5.0), None, "", "", 30.6, ((448, 256),), blocked=_NO_PIPELINE,
    notes="video, audio and text tokens in one stream; the 1080p super-resolution checkpoint loads through remap_magihuman_sr_keys"),
    "magihuman", "magihuman-sr")
register(ModelManifest(
    "sensenova-u1-8b", "sensenova_u1", _M + "sensenova_u1", "SenseNovaU1", "SenseNovaU1Config", "tiny_sensenova_u1_config",
    LatentSpec(3, 1, 32, True), TextSpec(512, 4096, 0, ()),
    ScheduleSpec("shifted", 30, 4.0, shift=3.0), None, "", "", 17.0, ((1024, 1024),),
    blocked="cli.sample and the validation sampler run the model's own pixel-space loop (no VAE, token ids in); no serving backend or trainer adapter",
    notes="the prompt's token ids run through the base weights once (key / value cache), image tokens through the _mot_gen weights; `SenseNovaU1.sample` is the loop"),
    "sensenova-u1", "sensenova")
register(ModelManifest(
    "boogu-image-0.1", "boogu", _M + "boogu", "BooguDiT", "BooguConfig", "tiny_boogu_config",
    LatentSpec(16, 8, 2, False), TextSpec(512, 4096, 0, ("qwen3_vl",)),
    ScheduleSpec("shifted", 30, 4.0, shift=3.0), None, "flux_vae_config", "", 10.0, ((1024, 1024),), blocked=_NO_PIPELINE,
    notes="head width 120: attention runs on the library kernel on the GPU (the tcgen05 kernel covers 64 and 128)"),
    "boogu")
register(ModelManifest(
    "nava", "nava", _M + "nava", "NavaDiT", "NavaConfig", "tiny_nava_config",
    LatentSpec(48, 16, 2, False, temporal_factor=4), TextSpec(512, 4096, 0, ("umt5",)),
    ScheduleSpec("shifted", 50, 5.0, shift=5.0), None, "", "", 5.9, ((832, 480),), blocked=_NO_PIPELINE,
    notes="video and audio latents in one sequence; fp8 checkpoint rows are dequantised by remap_nava_keys"),
    "nava-av")
register(ModelManifest(
    "pid-sr4x", "pid", _M + "pid", "PidNet", "PidConfig", "tiny_pid_config",
    LatentSpec(3, 1, 16, False), TextSpec(300, 2304, 0, ("gemma2_2b",)),
    ScheduleSpec("pid_distill", 4, 1.0), None, "", "", 1.4, ((2048, 2048),), blocked=_NO_PIPELINE,
    notes="pixel-space super-resolution decoder conditioned on a low-quality 16-channel latent; `sampling.family_schedules.pid_distill_sample` is its sampler"),
    "pid", "pixeldit")
register(ModelManifest(
    "hidream-o1", "hidream_o1", _M + "hidream_o1", "HiDreamO1", "HiDreamO1Config", "tiny_hidream_o1_config",
    LatentSpec(3, 1, 32, True), TextSpec(512, 4096, 0, ()),
    ScheduleSpec("hidream_o1", 28, 5.0), None, "", "", 8.0, ((1024, 1024),), blocked=_NO_PIPELINE,
    notes="pixel space: 32 x 32 RGB patches and the prompt's token ids run through one language-model spine"),
    "hidream_o1", "hidream")


# ---- execution config / shape profile / guard ------------------------------------------------------------------
@dataclass
class ExecutionConfig:
    """How one process runs a manifest: devices, dtype, residency and the parallel layout."""
    device: str = "cuda"
    dtype: str = "bf16"
    cuda_graph: bool = True
    block_swap: bool = False
    resident_blocks: int = -1            # -1: everything resident
    sequence_parallel: int = 1
    tensor_parallel: int = 1
    data_parallel: int = 1
    fsdp: bool = False

    def world(self) -> int:
        return max(1, self.sequence_parallel) * max(1, self.tensor_parallel) * max(1, self.data_parallel)


@dataclass
class ShapeProfile:
    """Token counts of one request on one manifest (what sizes the attention and the activation buffers)."""
    width: int
    height: int
    frames: int
    image_tokens: int
    text_tokens: int

    @property
    def seq_len(self) -> int:
        return self.image_tokens + self.text_tokens

    @staticmethod
    def of(m: ModelManifest, width: int, height: int, frames: int = 1) -> "ShapeProfile":
        cell = m.latent.vae_factor * m.latent.patch
        if width % cell or height % cell:
            raise ValueError(f"{m.model_id}: width/height must be multiples of {cell}")
        return ShapeProfile(width, height, frames, m.tokens_for(width, height, frames), m.text.tokens)


class ProductionGuard:
    """Admission check shared by the CLIs and the workers: a blocked manifest, a shape off the latent grid, or a parallel
    layout that does not divide heads / tokens is an error raised before any weight is loaded."""

    @staticmethod
    def check(m: ModelManifest, shape: ShapeProfile, ex: Optional[ExecutionConfig] = None, serving: bool = False) -> None:
        if serving and m.blocked:
            raise PermissionError(f"{m.model_id}: {m.blocked}")
        ex = ex or ExecutionConfig()
        if ex.sequence_parallel > 1:
            cfg = m.config()
            heads = getattr(cfg, "heads", getattr(cfg, "num_heads", 0))
            if heads and heads % ex.sequence_parallel:
                raise ValueError(f"{m.model_id}: {heads} heads do not divide over {ex.sequence_parallel} sequence-parallel ranks")
            if shape.image_tokens % ex.sequence_parallel or shape.text_tokens % ex.sequence_parallel:
                raise ValueError(f"{m.model_id}: token counts {shape.image_tokens}+{shape.text_tokens} do not divide over "
                                 f"{ex.sequence_parallel} ranks")
