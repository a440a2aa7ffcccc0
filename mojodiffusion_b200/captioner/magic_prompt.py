"""Idea -> structured Ideogram-4 caption with a local language model, as a throw-away process.

    python -m mojodiffusion_b200.captioner.magic_prompt <model> <aspect> <idea...>

``model`` is a directory holding a Qwen3-style checkpoint (``config.json``, ``*.safetensors``, ``tokenizer.json``) or
``stub:<file>`` (the file's text stands in for the model's reply: tests and dry runs). The process loads the model,
generates one reply, repairs it with the caption glue and prints ONE line of JSON on stdout; exit status 1 with the reason
on stderr otherwise. The control plane calls it per request (POST /v1/magic_prompt), so the language model never holds
device memory while an image worker runs (serenity-server/crates/server/src/magic.rs:1-125).
"""
from __future__ import annotations

import glob
import json
import os
import sys
from typing import List, Optional

from .glue import caption_from_idea_reply, upsample_caption_prompt


def list_llms(models_dir: str) -> List[dict]:
    """Language models under ``models_dir`` (one level of sub-directories is scanned): ``*.gguf`` files and directories
    that hold a ``config.json`` next to safetensors weights. Sorted by name."""
    out = []

    def add(path: str, size: int):
        out.append({"id": path, "name": os.path.splitext(os.path.basename(path.rstrip("/")))[0], "path": path, "size": size})

    def scan(d: str, deep: bool):
        try:
            names = sorted(os.listdir(d))
        except OSError:
            return
        if "config.json" in names and any(n.endswith(".safetensors") for n in names):
            add(d, sum(os.path.getsize(os.path.join(d, n)) for n in names if n.endswith(".safetensors")))
            return
        for n in names:
            p = os.path.join(d, n)
            if os.path.isdir(p) and deep:
                scan(p, False)
            elif n.endswith(".gguf"):
                add(p, os.path.getsize(p))
    scan(models_dir, True)
    return sorted(out, key=lambda e: e["name"])


def generate_reply(model: str, prompt: str, max_new_tokens: int = 1024, seed: int = 0) -> str:
    if model.startswith("stub:"):
        with open(model[5:], "r", encoding="utf-8") as f:
            return f.read()
    if model.endswith(".gguf"):
        raise RuntimeError("GGUF checkpoints are not readable here: point to a safetensors Qwen3 directory")
    import torch
    from ..io.safetensors_io import SafeTensors
    from ..llm.decoder import Qwen3Decoder
    from ..llm.sampler import SamplerConfig
    from ..models.text.qwen3 import Qwen3Config, Qwen3Encoder
    from ..models.text.tokenizers import ByteLevelBPE
    with open(os.path.join(model, "config.json"), "r", encoding="utf-8") as f:
        hf = json.load(f)
    fields = {k: hf[k] for k in Qwen3Config.__dataclass_fields__ if k in hf}
    cfg = Qwen3Config(**fields)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    enc = Qwen3Encoder(cfg, torch.bfloat16 if dev == "cuda" else torch.float32, dev)
    sd, head = {}, None
    for path in sorted(glob.glob(os.path.join(model, "*.safetensors"))):
        st = SafeTensors(path)
        for name in st.keys():
            if name == "lm_head.weight":
                head = st.tensor(name).to(dev)
            else:
                sd[name] = st.tensor(name)
    enc.load_state_dict(sd, strict=False)
    tok = ByteLevelBPE.from_tokenizer_json(os.path.join(model, "tokenizer.json"))
    text = f"<|im_start|>user\n{prompt}<|im_end|>\n<|im_start|>assistant\n"
    eos = [i for i in (hf.get("eos_token_id"),) if isinstance(i, int)]
    ids = Qwen3Decoder(enc, head).generate(tok.encode(text), max_new_tokens, SamplerConfig(temperature=0.7, top_p=0.9, seed=seed), eos)
    return tok.decode(ids)


def magic_prompt(model: str, aspect: str, idea: str, creative: bool = True) -> Optional[str]:
    return caption_from_idea_reply(generate_reply(model, upsample_caption_prompt(aspect, idea.strip(), creative=creative)))


def main(argv: List[str]) -> int:
    if len(argv) < 3:
        sys.stderr.write("usage: magic_prompt <model dir | stub:file> <aspect> <idea...>\n")
        return 2
    try:
        caption = magic_prompt(argv[0], argv[1], " ".join(argv[2:]))
    except Exception as ex:                      # one line for the caller's error body
        sys.stderr.write(f"{type(ex).__name__}: {ex}\n")
        return 1
    if not caption:
        sys.stderr.write("the model's reply held no JSON caption\n")
        return 1
    sys.stdout.write(caption + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
