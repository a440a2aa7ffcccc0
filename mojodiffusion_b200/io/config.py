"""Run configuration: the reference's JSON model/run configs (OneTrainer-shaped keys, nested ``optimizer`` block),
sample-prompt files (``serenity.sample_prompts.v1``) and the free-space guard used before saves.

Keys mirror serenitymojo/configs/*.json as parsed by serenitymojo/io/train_config_reader.mojo:749 into
serenitymojo/training/train_config.mojo:98-400 (defaults :590-610: max_steps 3000, save_every 500, sample_every 250).
Every key found in those 35 files is accepted; unknown keys are kept in ``extra`` instead of being dropped.
"""
from __future__ import annotations

import json
import os
import shutil
from dataclasses import asdict, dataclass, field, fields
from pathlib import Path
from typing import Any, Dict, List, Optional


@dataclass
class OptimizerConfig:
    optimizer: str = "ADAMW"
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.01
    fused: bool = True
    fused_back_pass: bool = False
    stochastic_rounding: bool = False


@dataclass
class TextEncoderConfig:
    train: bool = False
    dropout_probability: float = 0.0


@dataclass
class TrainConfig:
    # ---- paths -----------------------------------------------------------------------------------------
    model_type: str = "flux"
    base_model_name: str = ""
    checkpoint: str = ""
    vae: str = ""
    text_encoder: Any = None
    text_encoder_2: Any = None
    validation_prompts_file: str = ""
    sample_definition_file_name: str = ""
    concept_file_name: str = ""
    dataset_path: str = ""
    dataset_cache_dir: str = ""
    cache_dir: str = ""
    workspace_dir: str = ""
    output_model_destination: str = "output/lora.safetensors"
    output_model_format: str = "SAFETENSORS"
    trigger_word: str = ""
    # ---- architecture ----------------------------------------------------------------------------------
    inner_dim: int = 3072
    in_channels: int = 64
    out_channels: int = 64
    joint_attention_dim: int = 4096
    context_dim: int = 0
    num_double: int = 19
    num_single: int = 38
    num_heads: int = 24
    head_dim: int = 128
    mlp_hidden: int = 12288
    timestep_dim: int = 256
    time_embed_dim: int = 0
    time_scale: float = 1000.0
    rope_theta: float = 10000.0
    rope_axes_dim: Optional[List[int]] = None
    patch_size: int = 2
    norm_eps: float = 1e-6
    final_norm_eps: float = 1e-6
    num_noise_refiner: int = 0
    num_context_refiner: int = 0
    pad_tokens_multiple: int = 0
    min_mod: int = 0
    # UNet family
    model_channels: int = 320
    channel_mult: Optional[List[int]] = None
    num_res_blocks: int = 2
    num_groups: int = 32
    adm_in_channels: int = 2816
    transformer_depth_input: Optional[List[int]] = None
    transformer_depth_middle: int = 10
    transformer_depth_output: Optional[List[int]] = None
    num_train_timesteps: int = 1000
    beta_start: float = 0.00085
    beta_end: float = 0.012
    prediction_type: str = "epsilon"
    controlnet_layers: int = 0
    controlnet_scale: float = 1.0
    # ---- method / dtypes ----------------------------------------------------------------------------------
    training_method: str = "LORA"
    algo: str = "lora"
    lora_rank: int = 16
    lora_alpha: float = 16.0
    lora_weight_dtype: str = "BFLOAT_16"
    lokr_factor: int = -1
    lokr_factor_attn: int = -1
    lokr_factor_ff: int = -1
    lokr_factor_single: int = -1
    lokr_full_matrix: bool = False
    lokr_decompose_both: bool = False
    lokr_targets: Optional[List[str]] = None
    init_lokr_norm: float = 0.0
    train_dtype: str = "BFLOAT_16"
    fallback_train_dtype: str = "BFLOAT_16"
    weight_dtype: str = "BFLOAT_16"
    transformer_weight_dtype: str = "BFLOAT_16"
    text_encoder_weight_dtype: str = "BFLOAT_16"
    vae_weight_dtype: str = "BFLOAT_16"
    embedding_weight_dtype: str = "BFLOAT_16"
    output_dtype: str = "BFLOAT_16"
    quantized_resident: bool = False
    # ---- optimisation -----------------------------------------------------------------------------------
    resolution: str = "1024"
    batch_size: int = 1
    learning_rate: float = 1e-4
    lr_scheduler: str = "constant"
    learning_rate_scheduler: str = ""
    lr_warmup_steps: int = 0
    learning_rate_warmup_steps: int = 0
    max_grad_norm: float = 1.0
    max_steps: int = 3000
    train_num_steps: int = 0
    stop_training_after: int = 0
    stop_training_after_unit: str = "STEP"
    seed: int = 42
    loss_fn: str = "mse"
    huber_delta: float = 1.0
    smooth_l1_beta: float = 1.0
    min_snr_gamma_flow: float = 0.0
    timestep_distribution: str = "LOGIT_NORMAL"
    timestep_shift: float = 1.0
    timestep_noising_weight: float = 0.0
    timestep_noising_bias: float = 0.0
    sample_shift: float = 0.0
    caption_dropout_prob: float = 0.0
    gradient_checkpointing: str = "ON"
    layer_offload_fraction: float = 0.0
    enable_activation_offloading: bool = False
    enable_async_offloading: bool = True
    ema: str = "OFF"
    ema_decay: float = 0.999
    ema_min_decay: float = 0.0
    ema_update_after_step: int = 0
    ema_update_step_interval: int = 1
    non_ema_sampling: bool = True
    # ---- cadence ------------------------------------------------------------------------------------------
    save_every: int = 500
    save_every_unit: str = "STEP"
    save_skip_first: int = 0
    save_before_sample: bool = True
    sample_every: int = 250
    sample_after: int = 0
    sample_after_unit: str = "STEP"
    sample_at_start: bool = False
    sample_skip_first: int = 0
    continue_last_backup: bool = False
    optimizer: OptimizerConfig = field(default_factory=OptimizerConfig)
    extra: Dict[str, Any] = field(default_factory=dict)

    # ---- derived ----------------------------------------------------------------------------------------
    @property
    def total_steps(self) -> int:
        return self.train_num_steps or self.stop_training_after or self.max_steps

    @property
    def scheduler_name(self) -> str:
        return (self.learning_rate_scheduler or self.lr_scheduler).lower()

    @property
    def warmup_steps(self) -> int:
        return self.learning_rate_warmup_steps or self.lr_warmup_steps

    def to_dict(self) -> Dict[str, Any]:
        return asdict(self)


def _build(cls, d: Dict[str, Any]):
    names = {f.name for f in fields(cls)}
    return cls(**{k: v for k, v in d.items() if k in names})


def read_model_config(path_or_dict) -> TrainConfig:
    """JSON file (or already-parsed dict) -> :class:`TrainConfig`. Keys starting with ``_comment`` / ``comment``
    are documentation and ignored."""
    d = path_or_dict if isinstance(path_or_dict, dict) else json.loads(Path(path_or_dict).read_text())
    d = dict(d)
    opt = d.pop("optimizer", None)
    names = {f.name for f in fields(TrainConfig)}
    known, extra = {}, {}
    for k, v in d.items():
        if k.startswith("_comment") or k.startswith("comment"):
            continue
        (known if k in names else extra)[k] = v
    cfg = TrainConfig(**known)
    if isinstance(opt, dict):
        cfg.optimizer = _build(OptimizerConfig, opt)
    elif isinstance(opt, str):
        cfg.optimizer = OptimizerConfig(optimizer=opt)
    cfg.extra = extra
    return cfg


# ---------------------------------------------------------------------------------------------------------
# sample prompts (serenity.sample_prompts.v1; serenitymojo/training/sample_prompt_config.mojo)
# ---------------------------------------------------------------------------------------------------------
@dataclass
class SamplePrompt:
    id: str
    prompt: str
    seed: int
    negative: str
    width: int
    height: int
    frames: int
    fps: int
    steps: int
    cfg: float
    caps_positive: str = ""
    caps_negative: str = ""


@dataclass
class SamplePromptFile:
    sample_every: int = 250
    sample_at_start: bool = False
    save_before_sample: bool = True
    precache_required: bool = False
    prompts: List[SamplePrompt] = field(default_factory=list)

    def by_id(self, pid: str) -> SamplePrompt:
        for p in self.prompts:
            if p.id == pid:
                return p
        raise KeyError(pid)


def read_sample_prompts(path_or_dict) -> SamplePromptFile:
    d = path_or_dict if isinstance(path_or_dict, dict) else json.loads(Path(path_or_dict).read_text())
    if d.get("schema") != "serenity.sample_prompts.v1":
        raise ValueError(f"unsupported sample prompt schema {d.get('schema')!r}")
    df = {"sample_every": 250, "sample_at_start": False, "save_before_sample": True, "precache_required": False,
          "width": 1024, "height": 1024, "frames": 1, "fps": 24, "steps": 20, "cfg": 4.0, "seed": 42, "negative": ""}
    df.update(d.get("defaults", {}))
    out = SamplePromptFile(df["sample_every"], df["sample_at_start"], df["save_before_sample"], df["precache_required"])
    seen = set()
    for p in d.get("prompts", []):
        if "id" not in p or "prompt" not in p:
            raise ValueError("every prompt needs 'id' and 'prompt'")
        if p["id"] in seen:
            raise ValueError(f"duplicate prompt id {p['id']}")
        seen.add(p["id"])
        caps = p.get("caps", {}) or {}
        out.prompts.append(SamplePrompt(p["id"], p["prompt"], int(p.get("seed", df["seed"])),
                                        p.get("negative", df["negative"]), int(p.get("width", df["width"])),
                                        int(p.get("height", df["height"])), int(p.get("frames", df["frames"])),
                                        int(p.get("fps", df["fps"])), int(p.get("steps", df["steps"])),
                                        float(p.get("cfg", df["cfg"])), caps.get("positive", ""), caps.get("negative", "")))
    return out


# ---------------------------------------------------------------------------------------------------------
# disk guard (serenitymojo/io/disk_check.mojo:155-169)
# ---------------------------------------------------------------------------------------------------------
def free_bytes(path) -> int:
    p = Path(path)
    while not p.exists() and p != p.parent:
        p = p.parent
    return shutil.disk_usage(p).free


def guard_free_space(path, need_bytes: int, margin: float = 1.1) -> None:
    """Raise before a save that would not fit (needed bytes x margin must be free on the target filesystem)."""
    have = free_bytes(path)
    if have < need_bytes * margin:
        raise OSError(f"not enough free space under {path}: need {int(need_bytes * margin)} bytes, have {have}")
