"""Generation backend contract and the job-parameter record.

A backend is a cooperative state machine: ``start(params)`` accepts a job, every ``step()`` advances it by one unit of
work (one phase change or one denoise step) and returns what to report, ``cancel()`` makes the next ``step()`` return
"cancelled", ``trim()`` releases cached device memory between jobs. The worker loop interleaves ``step()`` with reads of
the control socket, so a cancel or a closed socket is seen within one step. A backend announces a phase BEFORE the long
tick that performs it ("encode", "load", "denoise", "decode"), so the UI shows what is running rather than what finished
(serenitymojo/serve/backend.mojo:40-398; per-model state machines in serve/*_backend.mojo; wire defaults
serenity-server/crates/wire/src/lib.rs:88-166)."""
from __future__ import annotations

import json
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional


@dataclass
class LoraSpec:
    name: str
    weight: float = 1.0


@dataclass
class JobParams:
    job_id: str = ""
    model: str = ""
    prompt: str = ""
    negative: str = ""
    width: int = 512
    height: int = 512
    steps: int = 20
    seed: int = 0
    cfg: float = 4.5
    cfg_override: float = -1.0
    cfg_override_start_percent: float = 0.0
    cfg_override_end_percent: float = 1.0
    sampler: str = ""
    scheduler: str = ""
    sigma_shift: float = 3.0
    variation_seed: int = 0
    variation_strength: float = 0.0
    images: int = 1
    image_index: int = 0
    image_count: int = 1
    workflow_save_prefix: str = ""
    init_image: str = ""
    mask_image: str = ""
    lanpaint_mask_channel: str = ""
    inpaint_conditioning_image: str = ""
    inpaint_conditioning_mask: str = ""
    inpaint_conditioning_noise_mask: bool = False
    qwen_edit_conditioning_image: str = ""
    sample_caps_pos: str = ""
    sample_caps_neg: str = ""
    conditioning_mask_image: str = ""
    conditioning_mask_channel: str = ""
    conditioning_mask_strength: float = -1.0
    conditioning_mask_set_area_to_bounds: bool = False
    outpaint_left: int = -1
    outpaint_top: int = -1
    outpaint_right: int = -1
    outpaint_bottom: int = -1
    outpaint_feathering: int = -1
    threshold_mask_value: float = -1.0
    threshold_mask_operator: str = ""
    lanpaint_mask_blend_overlap: int = -1
    lanpaint_num_steps: int = -1
    lanpaint_lambda: float = -1.0
    lanpaint_step_size: float = -1.0
    lanpaint_beta: float = -1.0
    lanpaint_friction: float = -1.0
    lanpaint_prompt_mode: str = ""
    lanpaint_inpainting_mode: str = ""
    lanpaint_add_noise: str = ""
    lanpaint_noise_seed: int = -1
    lanpaint_start_at_step: int = -1
    lanpaint_end_at_step: int = -1
    lanpaint_return_with_leftover_noise: str = ""
    lanpaint_early_stop: int = -1
    lanpaint_inner_threshold: float = -1.0
    lanpaint_inner_patience: int = -1
    reference_image: str = ""
    reference_latent_method: str = ""
    reference_latent_count: int = 0
    creativity: float = 0.5
    clip_skip: int = 0
    eta: float = -1.0
    sigma_min: float = -1.0
    sigma_max: float = -1.0
    restart_sampling: bool = False
    vae: str = ""
    out_dir: str = ""
    params_json: str = ""
    loras: List[LoraSpec] = field(default_factory=list)

    @classmethod
    def from_wire(cls, obj: Dict[str, Any]) -> "JobParams":
        p = cls()
        for f in fields(cls):
            if f.name == "loras":
                continue
            if f.name in obj and obj[f.name] is not None:
                v = obj[f.name]
                cur = getattr(p, f.name)
                if isinstance(cur, bool):
                    v = bool(v)
                elif isinstance(cur, int):
                    v = int(v)
                elif isinstance(cur, float):
                    v = float(v)
                else:
                    v = str(v)
                setattr(p, f.name, v)
        p.loras = [LoraSpec(str(e["name"]), float(e.get("weight", 1.0))) for e in obj.get("lora", []) or []]
        return p

    def to_wire(self) -> Dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self) if f.name != "loras"}
        d["lora"] = [{"name": l.name, "weight": l.weight} for l in self.loras]
        return d

    def start_line(self) -> str:
        return json.dumps({"cmd": "start", **self.to_wire()}, separators=(",", ":"))

    def output_path(self) -> str:
        return f"{self.out_dir}/{self.job_id}.png"

    def genparams_text(self) -> str:
        """The JSON embedded in the output image (tEXt keyword ``serenity.genparams.v1``)."""
        if self.params_json:
            try:
                self.params_json.encode("latin-1")
                return self.params_json
            except UnicodeEncodeError:                     # tEXt is Latin-1: re-escape everything beyond it
                return json.dumps(json.loads(self.params_json), separators=(",", ":"))
        d = self.to_wire()
        d.pop("params_json", None)
        d["schema"] = "serenity.genparams.v1"
        return json.dumps(d, separators=(",", ":"))


@dataclass
class StepResult:
    kind: str                      # progress | done | failed | cancelled
    step: int = 0
    total: int = 0
    phase: str = ""
    preview: str = ""
    output_path: str = ""
    error: str = ""

    def event(self) -> Dict[str, Any]:
        if self.kind == "progress":
            return {"ev": "progress", "step": self.step, "total": self.total, "phase": self.phase, "preview": self.preview}
        if self.kind == "done":
            return {"ev": "done", "output_path": self.output_path}
        if self.kind == "failed":
            return {"ev": "failed", "error": self.error}
        return {"ev": "cancelled"}

    @property
    def terminal(self) -> bool:
        return self.kind != "progress"


class UnsupportedParam(ValueError):
    pass


def reject_unsupported_common(p: JobParams, *, img2img: bool = True, inpaint: bool = True, lora: bool = True,
                              negative: bool = True, variation: bool = True, reference: bool = False) -> None:
    """Fail loudly on request features a backend cannot honour (never silently ignore them)."""
    if p.width % 16 or p.height % 16 or not (64 <= p.width <= 4096 and 64 <= p.height <= 4096):
        raise UnsupportedParam("width/height must be multiples of 16 within [64, 4096]")
    if not 1 <= p.steps <= 4096:
        raise UnsupportedParam("steps out of range")
    if p.init_image and not img2img:
        raise UnsupportedParam("this backend has no img2img")
    if p.mask_image and not inpaint:
        raise UnsupportedParam("this backend has no inpaint")
    if p.loras and not lora:
        raise UnsupportedParam("this backend does not execute LoRA")
    if p.negative and not negative:
        raise UnsupportedParam("this backend takes no negative prompt")
    if p.variation_strength > 0 and not variation:
        raise UnsupportedParam("this backend has no variation noise")
    if p.reference_image and not reference:
        raise UnsupportedParam("this backend takes no reference image")


class GenBackend:
    name = "base"

    def start(self, params: JobParams) -> None:
        raise NotImplementedError

    def step(self) -> StepResult:
        raise NotImplementedError

    def cancel(self) -> None:
        self._cancel = True

    def trim(self) -> None:
        """Release cached device memory between jobs (the resident model stays)."""

    def resident_model(self) -> str:
        return ""
