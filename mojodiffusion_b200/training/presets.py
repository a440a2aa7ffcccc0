"""Training preset catalogue and product-run contracts (no GPU involved anywhere in this module).

``preset_entry(id_or_alias)`` resolves a OneTrainer-style preset id to a catalogue row: recipe family, variant (lora /
finetune / inpaint_lora / deturbo_lora), the memory tier the preset was written for, model type, training method, optimizer
and whether a runnable loop exists for it here. ``apply_preset`` stamps those choices onto a ``TrainConfig``;
``dry_run_report`` is the lifecycle check a front-end calls before launching (paths, cadence, resume contract);
``lifecycle_paths`` spells the file naming policy (step files, final file, state sidecar).

Catalogue ids, aliases, the memory tiers, the per-preset optimizer (AdamW for the LoRA presets, Adafactor for the finetune
presets) and the rejection of plain "sd3" follow serenitymojo/training/onetrainer_preset_catalog.mojo:55-125,160-300;
naming policy serenitymojo/training/onetrainer_train_loop_policy.mojo:247-311; resume contract
serenitymojo/training/onetrainer_resume_contract.mojo:40-160. The 8 / 16 / 24 GB tiers are kept as labels: on a 180 GB part
they all run fully resident, and ``layer_offload_fraction`` stays at the preset's value only if the config asks for offload.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

from ..io.config import TrainConfig


@dataclass(frozen=True)
class PresetEntry:
    preset_id: str
    display_name: str
    recipe_family: str
    variant: str
    vram_tier_gb: int
    model_type: str
    training_method: str      # LORA | FINE_TUNE
    optimizer: str            # ADAMW | ADAFACTOR
    runnable: bool            # a train loop for this (family, method) exists in cli.train


def _mk(pid, name, family, model_type, method, optimizer, runnable, tier=0, variant=""):
    if not variant:
        variant = "finetune" if method == "FINE_TUNE" else "lora"
    return PresetEntry(pid, name, family, variant, tier, model_type, method, optimizer, runnable)


_ROWS: List[PresetEntry] = [
    _mk("qwen_lora_16gb", "Qwen Image LoRA 16GB", "qwenimage", "qwenimage", "LORA", "ADAMW", True, 16),
    _mk("qwen_lora_24gb", "Qwen Image LoRA 24GB", "qwenimage", "qwenimage", "LORA", "ADAMW", True, 24),
    _mk("qwen_finetune_16gb", "Qwen Image Finetune 16GB", "qwenimage", "qwenimage", "FINE_TUNE", "ADAFACTOR", True, 16),
    _mk("qwen_finetune_24gb", "Qwen Image Finetune 24GB", "qwenimage", "qwenimage", "FINE_TUNE", "ADAFACTOR", True, 24),
    _mk("ernie_lora_8gb", "ERNIE Image LoRA 8GB", "ernie", "ernie_image", "LORA", "ADAMW", False, 8),
    _mk("ernie_lora_16gb", "ERNIE Image LoRA 16GB", "ernie", "ernie_image", "LORA", "ADAMW", False, 16),
    _mk("anima_lora", "Anima LoRA", "anima", "anima", "LORA", "ADAMW", False),
    _mk("anima_finetune", "Anima Finetune", "anima", "anima", "FINE_TUNE", "ADAFACTOR", False),
    _mk("sd35_lora", "SD 3.5 LoRA", "sd35", "STABLE_DIFFUSION_35", "LORA", "ADAMW", False),
    _mk("sdxl_1_0_lora", "SDXL 1.0 LoRA", "sdxl", "sdxl", "LORA", "ADAMW", True),
    _mk("sdxl_1_0_finetune", "SDXL 1.0 Finetune", "sdxl", "sdxl", "FINE_TUNE", "ADAFACTOR", True),
    _mk("sdxl_1_0_inpaint_lora", "SDXL 1.0 Inpaint LoRA", "sdxl", "STABLE_DIFFUSION_XL_10_BASE_INPAINTING", "LORA", "ADAMW", False,
        variant="inpaint_lora"),
    _mk("flux1_dev_lora", "FLUX.1-dev LoRA", "flux1", "flux", "LORA", "ADAMW", True),
    _mk("flux2_lora_8gb", "FLUX.2 LoRA 8GB", "flux2_klein", "klein", "LORA", "ADAMW", True, 8),
    _mk("flux2_klein9b_lora_16gb", "FLUX.2 Klein 9B LoRA 16GB", "flux2_klein", "klein", "LORA", "ADAMW", True, 16),
    _mk("flux2_finetune_16gb", "FLUX.2 Finetune 16GB", "flux2_klein", "klein", "FINE_TUNE", "ADAFACTOR", True, 16),
    _mk("flux2_finetune_24gb", "FLUX.2 Finetune 24GB", "flux2_klein", "klein", "FINE_TUNE", "ADAFACTOR", True, 24),
    _mk("chroma_lora_8gb", "Chroma LoRA 8GB", "chroma", "chroma", "LORA", "ADAMW", False, 8),
    _mk("chroma_lora_16gb", "Chroma LoRA 16GB", "chroma", "chroma", "LORA", "ADAMW", False, 16),
    _mk("chroma_lora_24gb", "Chroma LoRA 24GB", "chroma", "chroma", "LORA", "ADAMW", False, 24),
    _mk("chroma_finetune_8gb", "Chroma Finetune 8GB", "chroma", "chroma", "FINE_TUNE", "ADAFACTOR", True, 8),
    _mk("chroma_finetune_16gb", "Chroma Finetune 16GB", "chroma", "chroma", "FINE_TUNE", "ADAFACTOR", True, 16),
    _mk("chroma_finetune_24gb", "Chroma Finetune 24GB", "chroma", "chroma", "FINE_TUNE", "ADAFACTOR", True, 24),
    _mk("zimage_lora_8gb", "Z-Image LoRA 8GB", "zimage", "zimage", "LORA", "ADAMW", True, 8),
    _mk("zimage_lora_16gb", "Z-Image LoRA 16GB", "zimage", "zimage", "LORA", "ADAMW", True, 16),
    _mk("zimage_deturbo_lora_8gb", "Z-Image De-Turbo LoRA 8GB", "zimage", "zimage", "LORA", "ADAMW", True, 8, "deturbo_lora"),
    _mk("zimage_deturbo_lora_16gb", "Z-Image De-Turbo LoRA 16GB", "zimage", "zimage", "LORA", "ADAMW", True, 16, "deturbo_lora"),
    _mk("zimage_finetune_16gb", "Z-Image Finetune 16GB", "zimage", "zimage", "FINE_TUNE", "ADAFACTOR", True, 16),
    _mk("zimage_finetune_24gb", "Z-Image Finetune 24GB", "zimage", "zimage", "FINE_TUNE", "ADAFACTOR", True, 24),
]
_BY_ID: Dict[str, PresetEntry] = {r.preset_id: r for r in _ROWS}
_ALIASES = {
    "qwen": "qwen_lora_16gb", "qwen_lora": "qwen_lora_16gb", "qwenimage": "qwen_lora_16gb", "QWEN": "qwen_lora_16gb",
    "qwen_finetune": "qwen_finetune_16gb", "ernie": "ernie_lora_16gb", "ernie_lora": "ernie_lora_16gb",
    "ernie_image": "ernie_lora_16gb", "ERNIE": "ernie_lora_16gb", "anima": "anima_lora", "ANIMA": "anima_lora",
    "sd35": "sd35_lora", "sd3.5": "sd35_lora", "STABLE_DIFFUSION_35": "sd35_lora", "sdxl": "sdxl_1_0_lora", "sdxl_lora": "sdxl_1_0_lora",
    "sdxl_finetune": "sdxl_1_0_finetune", "flux": "flux1_dev_lora", "flux1": "flux1_dev_lora", "flux_lora": "flux1_dev_lora",
    "klein": "flux2_klein9b_lora_16gb", "flux2": "flux2_klein9b_lora_16gb", "flux2_lora": "flux2_lora_8gb",
    "flux2_finetune": "flux2_finetune_16gb", "chroma": "chroma_lora_16gb", "chroma_lora": "chroma_lora_16gb",
    "chroma_finetune": "chroma_finetune_16gb", "zimage": "zimage_lora_16gb", "zimage_lora": "zimage_lora_16gb",
    "zimage_deturbo": "zimage_deturbo_lora_16gb", "zimage_finetune": "zimage_finetune_16gb",
}
# plain SD3 is a different checkpoint family from SD3.5 and is refused instead of being mapped onto it
_REJECTED = {"sd3": "plain SD3 (STABLE_DIFFUSION_3) is not a target; the SD 3.5 preset is 'sd35_lora'",
             "STABLE_DIFFUSION_3": "plain SD3 is not a target; use 'sd35_lora'"}


def preset_ids() -> List[str]:
    return [r.preset_id for r in _ROWS]


def preset_entry(preset: str) -> PresetEntry:
    if preset in _REJECTED:
        raise ValueError(_REJECTED[preset])
    pid = preset if preset in _BY_ID else _ALIASES.get(preset, "")
    if pid not in _BY_ID:
        raise KeyError(f"unknown training preset '{preset}'; known: {', '.join(preset_ids())}")
    return _BY_ID[pid]


def apply_preset(cfg: TrainConfig, preset: str) -> PresetEntry:
    e = preset_entry(preset)
    cfg.model_type = {"STABLE_DIFFUSION_35": "sd3", "STABLE_DIFFUSION_XL_10_BASE_INPAINTING": "sdxl"}.get(e.model_type, e.model_type)
    cfg.training_method = e.training_method
    cfg.optimizer.optimizer = e.optimizer
    if e.training_method == "FINE_TUNE":
        cfg.output_dtype = cfg.output_dtype or "BFLOAT_16"
    cfg.extra["preset_id"] = e.preset_id
    cfg.extra["vram_tier_gb"] = e.vram_tier_gb
    return e


# ---- lifecycle / naming / resume contracts -------------------------------------------------------------------------
def lifecycle_paths(cfg: TrainConfig, step: Optional[int] = None) -> Dict[str, str]:
    """File naming policy of a run: final file, its state sidecar, and the ``<base>_step<N>`` step file for ``step``."""
    final = cfg.output_model_destination
    ws = cfg.workspace_dir or "."
    dst = final if os.path.isabs(final) else os.path.join(ws, final)
    base, ext = os.path.splitext(dst)
    out = {"final": dst, "state_sidecar": base + ".state" + (ext or ".safetensors"), "workspace": ws,
           "backup_dir": os.path.join(ws, "backup"), "save_dir": os.path.join(ws, "save"), "samples_dir": os.path.join(ws, "samples")}
    if step is not None:
        out["step_file"] = f"{base}_step{step}{ext or '.safetensors'}"
    return out


def should_save_at(cfg: TrainConfig, step: int) -> bool:
    return cfg.save_every > 0 and cfg.save_every_unit.upper() == "STEP" and step > 0 and step % cfg.save_every == 0


def dry_run_report(cfg: TrainConfig, preset: str = "") -> Dict:
    """What a front-end shows before launching: resolved preset, paths, cadence, and every reason the run cannot start."""
    problems: List[str] = []
    entry = None
    if preset:
        try:
            entry = preset_entry(preset)
            if not entry.runnable:
                problems.append(f"preset {entry.preset_id}: no runnable loop for ({entry.recipe_family}, {entry.variant}) in this build")
        except (KeyError, ValueError) as ex:
            problems.append(str(ex))
    if not cfg.output_model_destination:
        problems.append("output_model_destination is empty")
    cache = cfg.cache_dir or cfg.dataset_cache_dir or cfg.dataset_path
    if not cache:
        problems.append("no cache directory configured (cache_dir / dataset_cache_dir / dataset_path)")
    elif not os.path.isdir(cache):
        problems.append(f"cache directory does not exist: {cache}")
    if cfg.total_steps <= 0:
        problems.append("total step count is not positive")
    if cfg.training_method.upper() == "LORA" and cfg.lora_rank <= 0:
        problems.append("lora_rank must be positive")
    resume = {"requested": bool(cfg.continue_last_backup), "found": None}
    if cfg.continue_last_backup:
        from .loop import find_last_backup
        resume["found"] = find_last_backup(cfg.workspace_dir or ".")
        if resume["found"] and not os.path.isfile(os.path.join(resume["found"], "optimizer", "optimizer.safetensors")):
            problems.append("resume: the last backup has no optimizer state beside the weights")
    return {"schema": "mdb200.train_dry_run.v1", "preset": entry.preset_id if entry else "", "paths": lifecycle_paths(cfg, cfg.save_every or None),
            "cadence": {"save_every": cfg.save_every, "save_unit": cfg.save_every_unit, "sample_every": cfg.sample_after or cfg.sample_every,
                        "sample_unit": cfg.sample_after_unit}, "resume": resume, "ok": not problems, "problems": problems}
