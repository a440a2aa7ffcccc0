"""Sampler entry point with the reference's argument contract:

    python -m mojodiffusion_b200.cli.sample <model> <config.json> <lora|-> <sample_prompts.json> <prompt_id> <out.png>

``<model>`` is a manifest id or family name (flux, klein, zimage, qwenimage, sdxl, sd3, chroma, ltx2); the config is the
reference's JSON run config (checkpoint / vae paths, LoRA rank); ``-`` means no adapter; the prompt file follows
``serenity.sample_prompts.v1``. Honoured from the prompt entry: prompt, negative, width, height, frames, steps, cfg, seed,
pre-encoded caption files. Stages: text -> load -> denoise -> VAE decode -> PNG with the generation parameters embedded,
plus ``<out>.json`` stating where weights and text conditioning came from. Options: ``--tiny`` (tiny architecture, for
smoke runs without checkpoints), ``--device``.

Contract and stages: serenitymojo/pipeline/flux_sample_cli.mojo:7-27,247-307,359; sibling CLIs klein / qwenimage / sdxl /
sd3 / chroma (serenitymojo/sampling/klein_sample_cli.mojo, serenitymojo/pipeline/*_sample_cli.mojo).
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import torch

from ..io.config import read_model_config, read_sample_prompts
from ..training.validation_sampler import ValidationSampler
from .common import attach_lora, build_model, manifest_from_config, pick_device


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mojodiffusion_b200.cli.sample")
    ap.add_argument("model")
    ap.add_argument("config")
    ap.add_argument("lora")
    ap.add_argument("prompts")
    ap.add_argument("prompt_id")
    ap.add_argument("out")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--device", default="")
    a = ap.parse_args(argv)
    if not a.out.lower().endswith(".png"):
        ap.error("the output path must end in .png")
    cfg = read_model_config(a.config)
    m = manifest_from_config(cfg, a.model)
    sp = read_sample_prompts(a.prompts).by_id(a.prompt_id)
    dev = pick_device(a.device)
    t0 = time.perf_counter()
    model, weights = build_model(m, cfg, dev, a.tiny)
    lora = "none"
    if a.lora != "-":
        slots = attach_lora(m, model, cfg.lora_rank, cfg.lora_alpha, a.lora)
        lora = f"{a.lora} ({len(slots)} adapters, runtime overlay)"
    model.eval()
    for p in model.parameters():
        p.requires_grad_(False)
    t_load = time.perf_counter() - t0
    vs = ValidationSampler(m, model, dev, tiny=a.tiny, vae_path=cfg.vae)
    path = vs.sample(sp, a.out, {"lora": a.lora})
    report = {"schema": "mdb200.sample_cli_result.v1", "model": m.model_id, "family": m.family, "weights": weights, "lora": lora,
              "load_s": round(t_load, 4), "device": str(dev), "output": path, **vs.last_report}
    with open(a.out[:-4] + ".json", "w") as f:
        json.dump(report, f)
    print(json.dumps(report))
    return 0


if __name__ == "__main__":
    sys.exit(main())
