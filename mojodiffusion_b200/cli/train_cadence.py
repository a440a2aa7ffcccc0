"""Process-separated train / sample cadence:

    python -m mojodiffusion_b200.cli.train_cadence <config.json> --chunk N [--tiny] [--device D]

Repeats: run the trainer as a child process for ``N`` more steps (it resumes from the last complete backup) -> it exits and
its device memory is gone -> run the sampler CLI as a child once per prompt of the sample-prompt file with the LoRA the
trainer just wrote -> next chunk, until the configured step count is reached. A trainer that dies is restarted from the
last backup up to ``--retries`` times. This is the supervisor of serenitymojo/training/train_klein_cadence.mojo:1-216
(train chunk -> exit -> one sampler process per prompt -> repeat; restart from the latest step checkpoint :64-75).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys

from ..io.config import read_model_config, read_sample_prompts
from ..training.loop import find_last_backup, read_backup


def _steps_done(workspace: str) -> int:
    last = find_last_backup(workspace)
    if last is None:
        return 0
    return read_backup(last)[0].global_step


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mojodiffusion_b200.cli.train_cadence")
    ap.add_argument("config")
    ap.add_argument("--chunk", type=int, required=True, help="optimizer steps per trainer process")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--device", default="")
    ap.add_argument("--retries", type=int, default=2)
    a = ap.parse_args(argv)
    raw = json.load(open(a.config))
    cfg = read_model_config(raw)
    ws = cfg.workspace_dir or "."
    os.makedirs(ws, exist_ok=True)
    run_cfg = os.path.join(ws, "cadence_run_config.json")
    raw = dict(raw)
    raw["continue_last_backup"] = True
    raw["sample_after_unit"] = "NEVER"            # sampling happens in separate processes here
    with open(run_cfg, "w") as f:
        json.dump(raw, f)
    pfile = cfg.validation_prompts_file or cfg.sample_definition_file_name
    prompts = read_sample_prompts(pfile).prompts if pfile and os.path.isfile(pfile) else []
    final = cfg.output_model_destination
    lora_path = final if os.path.isabs(final) else os.path.join(ws, final)
    extra = (["--tiny"] if a.tiny else []) + (["--device", a.device] if a.device else [])
    events = []
    failures = 0
    while True:
        done = _steps_done(ws)
        if done >= cfg.total_steps:
            break
        rc = subprocess.call([sys.executable, "-m", "mojodiffusion_b200.cli.train", run_cfg, "--max-steps", str(a.chunk), "--quiet"] + extra)
        now = _steps_done(ws)
        events.append({"event": "train_chunk", "from": done, "to": now, "rc": rc})
        if rc != 0 or now <= done:
            failures += 1
            if failures > a.retries:
                print(json.dumps({"schema": "mdb200.cadence_result.v1", "ok": False, "events": events}))
                return 1
            continue
        for sp in prompts:
            out = os.path.join(ws, "samples", f"cadence-step{now}-{sp.id}.png")
            src = cfg.model_type or cfg.base_model_name
            rc = subprocess.call([sys.executable, "-m", "mojodiffusion_b200.cli.sample", src, run_cfg,
                                  lora_path if os.path.isfile(lora_path) else "-", pfile, sp.id, out] + extra,
                                 stdout=subprocess.DEVNULL)
            events.append({"event": "sample", "step": now, "prompt": sp.id, "rc": rc, "png": out})
    print(json.dumps({"schema": "mdb200.cadence_result.v1", "ok": True, "steps": _steps_done(ws), "events": events}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
