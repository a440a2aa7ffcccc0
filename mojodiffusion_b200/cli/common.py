"""Shared set-up of the command-line entry points: manifest lookup, model construction (checkpoint or seeded random
weights, stated in every result), LoRA attach / load."""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from ..io.config import TrainConfig
from ..io.safetensors_io import load_safetensors
from ..runtime import ModelManifest, adapter_for, default_manifest_by_id


def pick_device(name: str = "") -> torch.device:
    if name:
        return torch.device(name)
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


def manifest_from_config(cfg: TrainConfig, model_arg: str = "") -> ModelManifest:
    for cand in (model_arg, cfg.model_type, cfg.base_model_name):
        if cand:
            try:
                return default_manifest_by_id(cand)
            except KeyError:
                continue
    raise KeyError(f"cannot resolve a model manifest from '{model_arg}' / model_type '{cfg.model_type}' / "
                   f"base_model_name '{cfg.base_model_name}'")


def build_model(m: ModelManifest, cfg: TrainConfig, device: torch.device, tiny: bool) -> Tuple[torch.nn.Module, str]:
    """Backbone on ``device``; weights from ``cfg.checkpoint`` when that file exists, else seeded random init.
    Returns (model, "checkpoint" | "random-init")."""
    dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    model = m.build(tiny=tiny, dtype=dtype, device=device)
    ck = cfg.checkpoint or cfg.base_model_name
    if ck and os.path.isfile(ck):
        sd = load_safetensors(ck, device=str(device), dtype=dtype)
        missing = [k for k in model.state_dict() if k not in sd]
        if missing:
            raise KeyError(f"{ck}: checkpoint lacks {len(missing)} tensors of {m.model_class}, e.g. {missing[:3]}")
        model.load_state_dict(sd, strict=False)
        return model, "checkpoint"
    model.init_weights(seed=0)
    return model, "random-init"


def attach_lora(m: ModelManifest, model, rank: int, alpha: float, path: Optional[str] = None):
    """Attach the family's adapter slots (runtime overlay: base weights are never modified) and load ``path`` into them."""
    from ..training import lora as L
    a = adapter_for(m)
    if path and os.path.isfile(path):
        sd = load_safetensors(path)
        for k, v in sd.items():
            if k.endswith("lora_down.weight") or k.endswith("lora_A.weight"):
                rank = int(v.shape[0])
                break
        alpha = float(rank) if not any(k.endswith(".alpha") for k in sd) else alpha
    slots = a.inject_lora(model, rank, alpha)
    if path and os.path.isfile(path):
        n = L.load_lora(path, slots, strict=False)
        if n == 0:
            raise KeyError(f"{path}: none of its keys match the {m.family} adapter names")
    elif path and path != "-":
        raise FileNotFoundError(path)
    return slots
