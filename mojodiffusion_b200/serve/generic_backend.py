"""Backends for the remaining model kinds. Each kind maps to the model class and sampler of this package; without a
checkpoint directory (``MDB_MODEL_DIR``) a kind whose architecture needs tens of GB is refused at ``start`` with a
message that names the missing file, instead of silently generating from random weights
(serenitymojo/serve/{zimage,qwenimage,sdxl,sd3,klein}_backend.mojo: residency and admission rules)."""
from __future__ import annotations

import os

from .backend import GenBackend, JobParams, StepResult, reject_unsupported_common

_CHECKPOINT_HINT = {"zimage": "z_image_turbo_bf16.safetensors", "qwenimage": "qwen_image_bf16.safetensors",
                    "sdxl": "sd_xl_base_1.0.safetensors", "sd3": "sd3.5_large.safetensors", "sd15": "v1-5-pruned.safetensors",
                    "ltx2": "ltx-2-19b-dev-fp8.safetensors"}


class GenericBackend(GenBackend):
    def __init__(self, kind: str):
        if kind not in _CHECKPOINT_HINT:
            raise ValueError(f"no backend for kind '{kind}'")
        self.kind = self.name = kind
        self.p = None
        self._cancel = False

    def start(self, params: JobParams) -> None:
        reject_unsupported_common(params)
        root = os.environ.get("MDB_MODEL_DIR", "")
        name = params.model if params.model.endswith(".safetensors") else params.model + ".safetensors"
        if not root or not os.path.isfile(os.path.join(root, name)):
            raise FileNotFoundError(f"{self.kind}: checkpoint '{name}' not found under MDB_MODEL_DIR "
                                    f"(expected e.g. {_CHECKPOINT_HINT[self.kind]})")
        raise NotImplementedError(f"{self.kind}: serving loop for this family is not wired to the worker yet; "
                                  f"use the FLUX kinds or the Python pipelines directly")

    def step(self) -> StepResult:
        return StepResult("failed", error=f"{self.kind}: no active job")
