"""Text encoding in a throw-away child process.

The text encoders of a family (CLIP-L / CLIP-G / T5-XXL / Qwen3) are needed for a fraction of a second per job and can be
larger than the denoiser's free memory. Running them in a child that exits after writing its result gives their device
memory back to the driver through process exit, the only release the allocator cannot hold on to
(serenitymojo/serve/zimage_encode_subprocess.mojo, serenitymojo/serve/qwenimage_encode_subprocess.mojo).

    parent:  encode_in_child(family, prompt, negative, encoders_dir, ...) -> {"text_embedding", "pooled", "text_mask", "neg_*"}
    child:   python -m mojodiffusion_b200.serve.encode_subprocess --family F --out caps.safetensors --prompt ... [--negative ...]
                    [--encoders-dir DIR] [--tiny] [--device cuda|cpu]

``encoders_dir`` layout (any subset; a missing encoder of the family is an error unless ``--tiny``):
    clip_l/{model.safetensors,vocab.json,merges.txt}   clip_g/{...}   t5_xxl/{model.safetensors,spiece.model}
    qwen3/{model.safetensors,tokenizer.json}
``--tiny`` builds small random-weight encoders and a byte tokenizer instead: the same process protocol and file contract
without checkpoints (CPU tests).

Per family: flux -> T5 hidden [1, 512, 4096] + CLIP-L pooled [1, 768]; sd3 -> CLIP-L + CLIP-G hidden (padded to 4096)
followed by T5 hidden, pooled = CLIP-L | CLIP-G pooled; sdxl -> penultimate CLIP-L | CLIP-G hidden [1, 77, 2048], pooled =
CLIP-G pooled; zimage / qwenimage / klein -> Qwen3 hidden of the chat-framed prompt (second-to-last layer, no final
norm) with its token mask.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
from typing import Dict, Optional

import torch

FAMILY_ENCODERS = {"flux": ("t5_xxl", "clip_l"), "chroma": ("t5_xxl",), "sd3": ("clip_l", "clip_g", "t5_xxl"), "sdxl": ("clip_l", "clip_g"),
                   "zimage": ("qwen3",), "qwenimage": ("qwen3",), "klein": ("qwen3",)}


class _ByteTokenizer:
    """Bytes of the prompt as ids (tiny mode only): deterministic, needs no vocabulary file."""

    def __init__(self, vocab_size: int, max_length: int, eos: int):
        self.v, self.n, self.eos = vocab_size, max_length, eos

    def __call__(self, text: str):
        ids = [(b % (self.v - 2)) + 1 for b in text.encode("utf-8")][: self.n - 1] + [self.eos]
        mask = [1] * len(ids) + [0] * (self.n - len(ids))
        return ids + [self.eos] * (self.n - len(ids)), mask


def _load_weights(model, path: str, device, dtype):
    from ..io.safetensors_io import load_safetensors
    sd = load_safetensors(path, device=str(device), dtype=dtype)
    own = model.state_dict()
    hit = {k: v for k, v in sd.items() if k in own and tuple(v.shape) == tuple(own[k].shape)}
    if len(hit) < len(own) // 2:
        raise ValueError(f"{path}: only {len(hit)} of {len(own)} encoder tensors match")
    model.load_state_dict(hit, strict=False)


def _build(name: str, enc_dir: str, tiny: bool, device, dtype):
    """-> (encoder, tokenizer)."""
    from ..models.text import clip as C, qwen3 as Q, t5 as T, tokenizers as K
    sub = os.path.join(enc_dir, name) if enc_dir else ""
    if name in ("clip_l", "clip_g"):
        cfg = C.clip_l_config() if name == "clip_l" else C.clip_g_config()
        if tiny:
            cfg = C.CLIPTextConfig(vocab_size=300, hidden_size=32 if name == "clip_l" else 48, intermediate_size=64, num_hidden_layers=2,
                                   num_attention_heads=4, max_position_embeddings=16, eos_token_id=299, hidden_act=cfg.hidden_act)
        enc = C.CLIPTextEncoder(cfg, dtype, device)
        tok = _ByteTokenizer(cfg.vocab_size, cfg.max_position_embeddings, cfg.eos_token_id) if tiny else \
            K.CLIPTokenizer.from_files(os.path.join(sub, "vocab.json"), os.path.join(sub, "merges.txt"), pad_with_eos=name == "clip_l")
    elif name == "t5_xxl":
        cfg = T.T5Config(vocab_size=300, d_model=64, d_kv=16, d_ff=96, num_layers=2, num_heads=4) if tiny else T.t5_xxl_config()
        enc = T.T5Encoder(cfg, dtype, device)
        tok = _ByteTokenizer(cfg.vocab_size, 24, 1) if tiny else K.T5Tokenizer(os.path.join(sub, "spiece.model"), 512)
    elif name == "qwen3":
        cfg = Q.Qwen3Config(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2,
                            head_dim=16) if tiny else Q.Qwen3Config()
        enc = Q.Qwen3Encoder(cfg, dtype, device)
        tok = _ByteTokenizer(cfg.vocab_size, 32, 2) if tiny else K.ByteLevelBPE.from_tokenizer_json(os.path.join(sub, "tokenizer.json"))
    else:
        raise KeyError(name)
    if tiny:
        from ..models.layers import init_module_weights
        with torch.no_grad():
            init_module_weights(enc, seed=7, std=0.05)
    else:
        _load_weights(enc, os.path.join(sub, "model.safetensors"), device, dtype)
    return enc.eval(), tok


@torch.no_grad()
def encode_family(family: str, prompt: str, enc_dir: str, tiny: bool, device, dtype, max_tokens: int = 512) -> Dict[str, torch.Tensor]:
    names = FAMILY_ENCODERS[family]
    out: Dict[str, torch.Tensor] = {}
    hidden, pooled, masks = {}, {}, {}
    for name in names:
        enc, tok = _build(name, enc_dir, tiny, device, dtype)
        if name == "qwen3":
            if isinstance(tok, _ByteTokenizer):
                ids, mask = tok(prompt)
            else:
                ids = tok.encode(tok.chat_template(prompt))[:max_tokens]
                mask = [1] * len(ids)
            t_ids, t_mask = torch.tensor([ids], device=device), torch.tensor([mask], device=device)
            hidden[name] = enc(t_ids, t_mask, layer=-2, final_norm=False).float().cpu()
            masks[name] = t_mask.float().cpu()
        elif name == "t5_xxl":
            ids, mask = tok(prompt)
            t_ids, t_mask = torch.tensor([ids], device=device), torch.tensor([mask], device=device)
            hidden[name] = enc(t_ids, t_mask).float().cpu()
            masks[name] = t_mask.float().cpu()
        else:
            ids, mask = tok(prompt)
            h, p = enc(torch.tensor([ids], device=device), clip_skip=1 if family == "sdxl" else 0)
            hidden[name], pooled[name], masks[name] = h.float().cpu(), p.float().cpu(), torch.tensor([mask]).float()
        del enc                                         # one encoder resident at a time
        if device.type == "cuda":
            torch.cuda.empty_cache()
    if family in ("flux", "chroma"):
        out["text_embedding"], out["text_mask"] = hidden["t5_xxl"], masks["t5_xxl"]
        out["pooled"] = pooled.get("clip_l", torch.zeros(1, 1))
    elif family == "sdxl":
        out["text_embedding"] = torch.cat((hidden["clip_l"], hidden["clip_g"]), dim=-1)
        out["text_mask"], out["pooled"] = masks["clip_l"], pooled["clip_g"]
    elif family == "sd3":
        clip = torch.cat((hidden["clip_l"], hidden["clip_g"]), dim=-1)
        t5 = hidden["t5_xxl"]
        clip = torch.nn.functional.pad(clip, (0, t5.shape[-1] - clip.shape[-1])) if clip.shape[-1] < t5.shape[-1] else clip[..., :t5.shape[-1]]
        out["text_embedding"] = torch.cat((clip, t5), dim=1)
        out["text_mask"] = torch.cat((masks["clip_l"], masks["t5_xxl"]), dim=1)
        out["pooled"] = torch.cat((pooled["clip_l"], pooled["clip_g"]), dim=-1)
    else:
        out["text_embedding"], out["text_mask"] = hidden["qwen3"], masks["qwen3"]
        out["pooled"] = torch.zeros(1, 1)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mojodiffusion_b200.serve.encode_subprocess")
    ap.add_argument("--family", required=True, choices=sorted(FAMILY_ENCODERS))
    ap.add_argument("--out", required=True)
    ap.add_argument("--prompt", default="")
    ap.add_argument("--negative", default=None)
    ap.add_argument("--encoders-dir", default="")
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--device", default="")
    a = ap.parse_args(argv)
    dev = torch.device(a.device or ("cuda" if torch.cuda.is_available() else "cpu"))
    dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    if not a.tiny and not a.encoders_dir:
        print(json.dumps({"error": "no --encoders-dir and not --tiny"}))
        return 2
    from ..io.safetensors_io import save_safetensors
    res = encode_family(a.family, a.prompt, a.encoders_dir, a.tiny, dev, dtype)
    if a.negative is not None:
        for k, v in encode_family(a.family, a.negative, a.encoders_dir, a.tiny, dev, dtype).items():
            res["neg_" + k] = v
    tmp = a.out + ".tmp"
    save_safetensors(tmp, {k: v.contiguous() for k, v in res.items()}, {"family": a.family, "pid": str(os.getpid()), "tiny": str(int(a.tiny))})
    os.replace(tmp, a.out)
    print(json.dumps({"ok": True, "out": a.out, "tokens": int(res["text_embedding"].shape[1]), "pid": os.getpid()}))
    return 0


def encode_in_child(family: str, prompt: str, negative: Optional[str] = None, encoders_dir: str = "", tiny: bool = False,
                    device: str = "", timeout_s: float = 600.0, workdir: Optional[str] = None) -> Dict[str, torch.Tensor]:
    """Run the child, read its result, delete the file. Raises RuntimeError with the child's stderr tail on failure. The
    returned dict carries ``child_pid`` (an int tensor) so callers and tests can see that another process did the work."""
    from ..io.safetensors_io import SafeTensors, load_safetensors
    fd, path = tempfile.mkstemp(suffix=".caps.safetensors", dir=workdir)
    os.close(fd)
    os.unlink(path)
    cmd = [sys.executable, "-m", "mojodiffusion_b200.serve.encode_subprocess", "--family", family, "--out", path, "--prompt", prompt]
    if negative is not None:
        cmd += ["--negative", negative]
    if encoders_dir:
        cmd += ["--encoders-dir", encoders_dir]
    if tiny:
        cmd += ["--tiny"]
    if device:
        cmd += ["--device", device]
    env = dict(os.environ)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env["PYTHONPATH"] = root + os.pathsep + env.get("PYTHONPATH", "")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s, env=env)
    if r.returncode != 0 or not os.path.isfile(path):
        raise RuntimeError(f"text-encoder child failed (exit {r.returncode}): {r.stderr[-800:] or r.stdout[-400:]}")
    try:
        out = dict(load_safetensors(path))
        st = SafeTensors(path)
        try:
            out["child_pid"] = torch.tensor([int(st.metadata.get("pid", "0"))])
        finally:
            st.close()
    finally:
        os.unlink(path)
    return out


if __name__ == "__main__":
    sys.exit(main())
