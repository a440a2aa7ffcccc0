"""Full fine-tune: every model tensor trains, bf16 storage with fp32 masters in the optimizer. Two artifacts:

* the model file: the tensors under their own names, storage dtype preserved byte for byte;
* the resume state file: ``param.<i>`` fp32 masters for i in manifest order, then ``adam_m.<i>``, ``adam_v.<i>``
  interleaved, then ``__meta__`` = fp32 [t_step, accum_count]; the tensor-name manifest (newline-joined UTF-8 names, as
  a U8 tensor) under ``__full_finetune_tensor_names_utf8__`` binds index i to a name

(serenitymojo/training/full_finetune_contract.mojo:26-33,320-405, full_finetune_state_binding.mojo:5,75-135,
full_finetune_save.mojo:1-13)."""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, List, Sequence, Tuple

import torch
from torch import nn

from ..io.safetensors_io import load_safetensors, save_safetensors
from .optim import FusedAdamW

MANIFEST_KEY = "__full_finetune_tensor_names_utf8__"
META_KEY = "__meta__"


def trainable_inventory(model: nn.Module) -> List[Tuple[str, nn.Parameter]]:
    """Deterministic (module registration) order of every floating-point parameter."""
    return [(n, p) for n, p in model.named_parameters() if p.is_floating_point()]


def prepare_full_finetune(model: nn.Module, lr: float, **opt_kw) -> Tuple[List[Tuple[str, nn.Parameter]], FusedAdamW]:
    inv = trainable_inventory(model)
    for _, p in inv:
        p.requires_grad_(True)
    opt = FusedAdamW([p for _, p in inv], lr, master_weights=True, **opt_kw)
    return inv, opt


def save_model_tensors(path, inventory: Sequence[Tuple[str, torch.Tensor]], metadata=None) -> None:
    save_safetensors(path, OrderedDict((n, p.detach().contiguous()) for n, p in inventory), metadata)


def state_keys(n: int) -> List[str]:
    keys = [f"param.{i}" for i in range(n)]
    for i in range(n):
        keys += [f"adam_m.{i}", f"adam_v.{i}"]
    return keys + [META_KEY]


def save_state(path, inventory, optimizer, t_step: int, accum_count: int = 0) -> None:
    n = len(inventory)
    out = OrderedDict()
    masters = getattr(optimizer, "masters", None)
    for i, (_, p) in enumerate(inventory):
        src = masters[i] if masters is not None else p.detach()
        out[f"param.{i}"] = src.float().contiguous()
    for i, (_, p) in enumerate(inventory):
        m, v = optimizer.moments(p)
        out[f"adam_m.{i}"] = m.float().contiguous()
        out[f"adam_v.{i}"] = v.float().contiguous()
    out[META_KEY] = torch.tensor([float(t_step), float(accum_count)], dtype=torch.float32)
    names = "\n".join(nm for nm, _ in inventory).encode("utf-8")
    out[MANIFEST_KEY] = torch.frombuffer(bytearray(names), dtype=torch.uint8).clone()
    assert list(out.keys())[:-1] == state_keys(n)
    save_safetensors(path, out)


def load_state(path, inventory, optimizer) -> Tuple[int, int]:
    """Re-binds by NAME through the manifest: a reordered or renamed inventory fails loudly."""
    sd = load_safetensors(path)
    if MANIFEST_KEY not in sd or META_KEY not in sd:
        raise KeyError("full-finetune state file lacks the tensor-name manifest or __meta__")
    names = bytes(sd[MANIFEST_KEY].tolist()).decode("utf-8").split("\n")
    if names != [n for n, _ in inventory]:
        raise ValueError("full-finetune resume: param.N order does not match the tensor-name manifest")
    meta = sd[META_KEY]
    if meta.dtype != torch.float32 or meta.numel() != 2:
        raise ValueError("full-finetune resume metadata must be F32 [t_step, accum_count]")
    masters = getattr(optimizer, "masters", None)
    with torch.no_grad():
        for i, (n, p) in enumerate(inventory):
            for k in (f"param.{i}", f"adam_m.{i}", f"adam_v.{i}"):
                if k not in sd:
                    raise KeyError(k)
                if sd[k].dtype != torch.float32 or sd[k].numel() != p.numel():
                    raise ValueError(f"{k}: fp32 tensor of {p.numel()} elements expected")
            w = sd[f"param.{i}"].view_as(p)
            if masters is not None:
                masters[i].copy_(w.to(masters[i].device))
            p.copy_(w.to(p.device, p.dtype))
            optimizer.set_moments(p, sd[f"adam_m.{i}"].view_as(p), sd[f"adam_v.{i}"].view_as(p))
    optimizer.step_count = int(meta[0])
    return int(meta[0]), int(meta[1])
