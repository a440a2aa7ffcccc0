"""LoRA injection, key layouts and checkpoint formats.

Five key schemes are written / read (serenitymojo/training/lora_save.mojo:83-380):
* OneTrainer raw layout (FLUX, Qwen-Image): ``<prefix>.alpha`` (scalar), ``<prefix>.lora_down.weight`` [rank, in],
  ``<prefix>.lora_up.weight`` [out, rank]
* PEFT layout (Klein, Z-Image, LTX-2): ``<module>.lora_A.weight`` [rank, in], ``<module>.lora_B.weight`` [out, rank]
* train-state sidecar ``*.state.safetensors``: the PEFT pair in bf16 plus ``.lora_A.adam_m/.adam_v`` and
  ``.lora_B.adam_m/.adam_v`` in fp32 per module.
Prefix tables: FLUX.1 (serenitymojo/models/flux/flux_stack_lora.mojo:1232-1365), Klein
(serenitymojo/models/klein/klein_stack_lora.mojo:2468-2511), Qwen-Image (serenitymojo/models/qwenimage/qwenimage_stack_lora.mojo:205-234),
Z-Image (serenitymojo/models/zimage/zimage_stack_lora.mojo:1655-1700), LTX-2 (serenitymojo/training/ltx2/lora_surface.mojo:25-90).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Iterable, List, Optional, Sequence

import torch
import torch.nn as nn

from ..io.safetensors_io import SafeTensors, save_safetensors
from ..models.layers import Linear, LoRASlot

FLUX_DOUBLE_IMG = ("attn_to_q", "attn_to_k", "attn_to_v", "attn_to_out_0", "ff_net_0_proj", "ff_net_2")
FLUX_DOUBLE_TXT = ("attn_add_q_proj", "attn_add_k_proj", "attn_add_v_proj", "attn_to_add_out",
                   "ff_context_net_0_proj", "ff_context_net_2")
FLUX_SINGLE = ("attn_to_q", "attn_to_k", "attn_to_v", "proj_mlp", "proj_out")


def flux_lora_prefixes(depth_double: int = 19, depth_single: int = 38) -> List[str]:
    """All FLUX.1 adapter prefixes in checkpoint order: doubles (img 6 then txt 6) then singles (5)."""
    out = []
    for i in range(depth_double):
        out += [f"lora_transformer_transformer_blocks_{i}_{s}" for s in FLUX_DOUBLE_IMG]
        out += [f"lora_transformer_transformer_blocks_{i}_{s}" for s in FLUX_DOUBLE_TXT]
    for i in range(depth_single):
        out += [f"lora_transformer_single_transformer_blocks_{i}_{s}" for s in FLUX_SINGLE]
    return out


def inject_flux_lora(model, rank: int = 16, alpha: float = 16.0, targets: Optional[Sequence[str]] = None,
                     seed: int = 0) -> List[LoRASlot]:
    """Attach adapters to every attention / MLP linear of an :class:`MMDiT`. Fused projections get one adapter
    per logical matrix (to_q / to_k / to_v are row ranges of ``qkv``; single blocks split ``linear1`` into
    q, k, v, proj_mlp). Base weights are frozen; returns the slots in checkpoint order."""
    D = model.cfg.hidden
    F_ = model.cfg.mlp_hidden
    want = set(targets) if targets is not None else None
    slots: List[LoRASlot] = []

    def add(lin: Linear, key: str, rows=None):
        short = key.split("_blocks_", 1)[1].split("_", 1)[1]
        if want is not None and short not in want:
            return
        slots.append(lin.add_lora(key, rank, alpha, rows, seed))

    for p in model.parameters():
        p.requires_grad_(False)
    for i, blk in enumerate(model.double_blocks):
        pre = f"lora_transformer_transformer_blocks_{i}_"
        add(blk.img_attn.qkv, pre + "attn_to_q", (0, D))
        add(blk.img_attn.qkv, pre + "attn_to_k", (D, 2 * D))
        add(blk.img_attn.qkv, pre + "attn_to_v", (2 * D, 3 * D))
        add(blk.img_attn.proj, pre + "attn_to_out_0")
        add(blk.img_mlp["0"], pre + "ff_net_0_proj")
        add(blk.img_mlp["2"], pre + "ff_net_2")
        add(blk.txt_attn.qkv, pre + "attn_add_q_proj", (0, D))
        add(blk.txt_attn.qkv, pre + "attn_add_k_proj", (D, 2 * D))
        add(blk.txt_attn.qkv, pre + "attn_add_v_proj", (2 * D, 3 * D))
        add(blk.txt_attn.proj, pre + "attn_to_add_out")
        add(blk.txt_mlp["0"], pre + "ff_context_net_0_proj")
        add(blk.txt_mlp["2"], pre + "ff_context_net_2")
    for i, blk in enumerate(model.single_blocks):
        pre = f"lora_transformer_single_transformer_blocks_{i}_"
        add(blk.linear1, pre + "attn_to_q", (0, D))
        add(blk.linear1, pre + "attn_to_k", (D, 2 * D))
        add(blk.linear1, pre + "attn_to_v", (2 * D, 3 * D))
        add(blk.linear1, pre + "proj_mlp", (3 * D, 3 * D + F_))
        add(blk.linear2, pre + "proj_out")
    for s in slots:
        s.down.requires_grad_(True)
        s.up.requires_grad_(True)
    return slots


KLEIN_DOUBLE = ("attn.to_q", "attn.to_k", "attn.to_v", "attn.to_out.0", "ff.linear_in", "ff.linear_out", "attn.add_q_proj",
                "attn.add_k_proj", "attn.add_v_proj", "attn.to_add_out", "ff_context.linear_in", "ff_context.linear_out")
KLEIN_SINGLE = ("attn.to_qkv_mlp_proj", "attn.to_out")
QWEN_BLOCK = ("attn.to_q", "attn.to_k", "attn.to_v", "attn.to_out.0", "img_mlp.net.0.proj", "img_mlp.net.2", "attn.add_q_proj",
              "attn.add_k_proj", "attn.add_v_proj", "attn.to_add_out", "txt_mlp.net.0.proj", "txt_mlp.net.2")
ZIMAGE_BLOCK = ("attention.to_q", "attention.to_k", "attention.to_v", "attention.to_out.0", "feed_forward.w1",
                "feed_forward.w3", "feed_forward.w2")
LTX2_ATTN = ("to_q", "to_k", "to_v", "to_out.0")


def _finish(model: nn.Module, slots: List[LoRASlot]) -> List[LoRASlot]:
    for s in slots:
        s.down.requires_grad_(True)
        s.up.requires_grad_(True)
    return slots


def _freeze(model: nn.Module) -> None:
    for p in model.parameters():
        p.requires_grad_(False)


def inject_klein_lora(model, rank: int = 16, alpha: float = 16.0, seed: int = 0) -> List[LoRASlot]:
    """FLUX.2 Klein adapters under the diffusers-style names the reference saves
    (``transformer.transformer_blocks.{i}.attn.to_q`` ... ``transformer.single_transformer_blocks.{i}.attn.to_qkv_mlp_proj``);
    to_q / to_k / to_v are row ranges of the fused ``qkv`` weight, the single block's whole ``linear1`` is one adapter."""
    D = model.cfg.hidden
    _freeze(model)
    slots: List[LoRASlot] = []
    for i, b in enumerate(model.double_blocks):
        pre = f"transformer.transformer_blocks.{i}."
        table = {"attn.to_q": (b.img_attn.qkv, (0, D)), "attn.to_k": (b.img_attn.qkv, (D, 2 * D)), "attn.to_v": (b.img_attn.qkv, (2 * D, 3 * D)),
                 "attn.to_out.0": (b.img_attn.proj, None), "ff.linear_in": (b.img_mlp["0"], None), "ff.linear_out": (b.img_mlp["2"], None),
                 "attn.add_q_proj": (b.txt_attn.qkv, (0, D)), "attn.add_k_proj": (b.txt_attn.qkv, (D, 2 * D)),
                 "attn.add_v_proj": (b.txt_attn.qkv, (2 * D, 3 * D)), "attn.to_add_out": (b.txt_attn.proj, None),
                 "ff_context.linear_in": (b.txt_mlp["0"], None), "ff_context.linear_out": (b.txt_mlp["2"], None)}
        for n in KLEIN_DOUBLE:
            lin, rows = table[n]
            slots.append(lin.add_lora(pre + n, rank, alpha, rows, seed))
    for i, b in enumerate(model.single_blocks):
        pre = f"transformer.single_transformer_blocks.{i}."
        slots.append(b.linear1.add_lora(pre + "attn.to_qkv_mlp_proj", rank, alpha, None, seed))
        slots.append(b.linear2.add_lora(pre + "attn.to_out", rank, alpha, None, seed))
    return _finish(model, slots)


def klein_lora_prefixes(depth_double: int, depth_single: int) -> List[str]:
    out = []
    for i in range(depth_double):
        out += [f"transformer.transformer_blocks.{i}.{n}" for n in KLEIN_DOUBLE]
    for i in range(depth_single):
        out += [f"transformer.single_transformer_blocks.{i}.{n}" for n in KLEIN_SINGLE]
    return out


def inject_qwen_lora(model, rank: int = 16, alpha: float = 16.0, seed: int = 0) -> List[LoRASlot]:
    """Qwen-Image adapters: twelve per block under ``transformer.transformer_blocks.{i}.<module path>``."""
    _freeze(model)
    mods = dict(model.named_modules())
    slots = []
    for i in range(len(model.transformer_blocks)):
        for n in QWEN_BLOCK:
            slots.append(mods[f"transformer_blocks.{i}.{n}"].add_lora(f"transformer.transformer_blocks.{i}.{n}", rank, alpha, None, seed))
    return _finish(model, slots)


def inject_zimage_lora(model, rank: int = 16, alpha: float = 16.0, refiners: bool = False, seed: int = 0) -> List[LoRASlot]:
    """Z-Image adapters on the attention and feed-forward projections of the main ``layers`` (210 for 30 layers); the
    noise / context refiners only when asked for (the reference's production surface leaves them out)."""
    _freeze(model)
    mods = dict(model.named_modules())
    groups = [("layers", len(model.layers))]
    if refiners:
        groups = [("noise_refiner", len(model.noise_refiner)), ("context_refiner", len(model.context_refiner))] + groups
    slots = []
    for g, n_ in groups:
        for i in range(n_):
            for n in ZIMAGE_BLOCK:
                slots.append(mods[f"{g}.{i}.{n}"].add_lora(f"{g}.{i}.{n}", rank, alpha, None, seed))
    return _finish(model, slots)


def zimage_kohya_name(prefix: str) -> str:
    """``layers.3.attention.to_q`` -> ``lora_unet_layers_3_attention_to_q`` (the Kohya export spelling)."""
    return "lora_unet_" + prefix.replace(".", "_")


def inject_ltx2_lora(model, rank: int = 16, alpha: float = 16.0, cross_attention: bool = True, seed: int = 0) -> List[LoRASlot]:
    """LTX-2 video adapters: ``diffusion_model.transformer_blocks.{i}.{attn1,attn2}.{to_q,to_k,to_v,to_out.0}`` and
    ``ff.net.{0.proj,2}``; saved in the PEFT layout where the scale is the load-time strength (alpha = rank)."""
    _freeze(model)
    mods = dict(model.named_modules())
    slots = []
    for i in range(len(model.transformer_blocks)):
        pre = f"transformer_blocks.{i}."
        names = [f"attn1.{n}" for n in LTX2_ATTN] + ([f"attn2.{n}" for n in LTX2_ATTN] if cross_attention else [])
        names += ["ff.net.0.proj", "ff.net.2"]
        for n in names:
            slots.append(mods[pre + n].add_lora("diffusion_model." + pre + n, rank, alpha, None, seed))
    return _finish(model, slots)


def inject_ernie_lora(model, rank: int = 16, alpha: float = 16.0, seed: int = 0) -> List[LoRASlot]:
    """ERNIE-Image adapters on the attention and gated-MLP projections of every layer, under ``transformer.<module path>``."""
    from ..models.ernie import ernie_lora_targets
    _freeze(model)
    mods = dict(model.named_modules())
    return _finish(model, [mods[n].add_lora("transformer." + n, rank, alpha, None, seed) for n in ernie_lora_targets(len(model.layers))])


def inject_anima_lora(model, rank: int = 16, alpha: float = 16.0, seed: int = 0) -> List[LoRASlot]:
    """Anima adapters on self- / cross-attention and MLP projections, keys = the checkpoint's module paths (``net.blocks.…``)."""
    from ..models.anima import anima_lora_targets
    _freeze(model)
    mods = dict(model.named_modules())
    return _finish(model, [mods[n].add_lora("diffusion_model." + n, rank, alpha, None, seed) for n in anima_lora_targets(len(model.net.blocks))])


KREA2_BLOCK = ("attn.wq", "attn.wk", "attn.wv", "attn.gate", "attn.wo", "mlp.gate", "mlp.up", "mlp.down")
LENS_BLOCK = ("attn.img_qkv", "attn.txt_qkv", "attn.to_out.0", "attn.to_add_out", "img_mlp.w1", "img_mlp.w2", "img_mlp.w3",
              "txt_mlp.w1", "txt_mlp.w2", "txt_mlp.w3")


def inject_krea2_lora(model, rank: int = 16, alpha: float = 16.0, seed: int = 0) -> List[LoRASlot]:
    """Krea-2 adapters: eight per single-stream block (the five attention projections and the three feed-forward ones); the
    embedders, the text fusion and the last layer stay frozen (serenitymojo/models/krea2/krea2_stack.mojo:12-18,124)."""
    _freeze(model)
    mods = dict(model.named_modules())
    slots = [mods[f"blocks.{i}.{n}"].add_lora(f"blocks.{i}.{n}", rank, alpha, None, seed)
             for i in range(len(model.blocks)) for n in KREA2_BLOCK]
    return _finish(model, slots)


def inject_lens_lora(model, rank: int = 16, alpha: float = 16.0, seed: int = 0) -> List[LoRASlot]:
    """Lens adapters on the attention and feed-forward projections of both streams of every block."""
    _freeze(model)
    mods = dict(model.named_modules())
    slots = [mods[f"transformer_blocks.{i}.{n}"].add_lora(f"transformer_blocks.{i}.{n}", rank, alpha, None, seed)
             for i in range(len(model.transformer_blocks)) for n in LENS_BLOCK]
    return _finish(model, slots)


def inject_lora_by_name(model: nn.Module, name_to_key: Dict[str, str], rank: int, alpha: float) -> List[LoRASlot]:
    """Generic injection: ``name_to_key`` maps a module path of a :class:`Linear` to its checkpoint prefix."""
    for p in model.parameters():
        p.requires_grad_(False)
    mods = dict(model.named_modules())
    slots = []
    for name, key in name_to_key.items():
        lin = mods[name]
        assert isinstance(lin, Linear), name
        slots.append(lin.add_lora(key, rank, alpha))
    for s in slots:
        s.down.requires_grad_(True)
        s.up.requires_grad_(True)
    return slots


def collect_slots(model: nn.Module) -> List[LoRASlot]:
    return [m for m in model.modules() if isinstance(m, LoRASlot)]


def lora_parameters(slots: Iterable[LoRASlot]) -> List[nn.Parameter]:
    out = []
    for s in slots:
        out += [s.down, s.up]
    return out


# ------------------------------------------------------------------------------------------------
# checkpoint formats
# ------------------------------------------------------------------------------------------------
def lora_state_onetrainer(slots: Sequence[LoRASlot]) -> "OrderedDict[str, torch.Tensor]":
    sd: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    for s in slots:
        sd[f"{s.key}.alpha"] = torch.tensor(s.alpha, dtype=torch.bfloat16)
        sd[f"{s.key}.lora_down.weight"] = s.down.detach().to(torch.bfloat16).cpu()
        sd[f"{s.key}.lora_up.weight"] = s.up.detach().to(torch.bfloat16).cpu()
    return sd


def lora_state_peft(slots: Sequence[LoRASlot]) -> "OrderedDict[str, torch.Tensor]":
    sd: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    for s in slots:
        sd[f"{s.key}.lora_A.weight"] = s.down.detach().to(torch.bfloat16).cpu()
        sd[f"{s.key}.lora_B.weight"] = s.up.detach().to(torch.bfloat16).cpu()
    return sd


def save_lora(path, slots: Sequence[LoRASlot], layout: str = "onetrainer", metadata=None) -> None:
    sd = lora_state_onetrainer(slots) if layout == "onetrainer" else lora_state_peft(slots)
    save_safetensors(path, sd, metadata)


def save_lora_state_sidecar(path, slots: Sequence[LoRASlot], optimizer, step: int) -> None:
    """``*.state.safetensors``: adapters (bf16) + Adam moments (fp32) per module, plus the step counter."""
    sd: "OrderedDict[str, torch.Tensor]" = OrderedDict()
    for s in slots:
        sd[f"{s.key}.lora_A.weight"] = s.down.detach().to(torch.bfloat16).cpu()
        sd[f"{s.key}.lora_B.weight"] = s.up.detach().to(torch.bfloat16).cpu()
        for tag, p in (("lora_A", s.down), ("lora_B", s.up)):
            m, v = optimizer.moments(p)
            sd[f"{s.key}.{tag}.adam_m"] = m.detach().float().cpu()
            sd[f"{s.key}.{tag}.adam_v"] = v.detach().float().cpu()
    sd["__meta__"] = torch.tensor([float(step), 0.0], dtype=torch.float32)
    save_safetensors(path, sd)


def load_lora(path, slots: Sequence[LoRASlot], strict: bool = True) -> int:
    """Load adapters from either key layout (also accepts ``.alpha``). Returns the number of slots restored."""
    st = SafeTensors(path)
    n = 0
    with torch.no_grad():
        for s in slots:
            for dn, un in ((f"{s.key}.lora_down.weight", f"{s.key}.lora_up.weight"),
                           (f"{s.key}.lora_A.weight", f"{s.key}.lora_B.weight")):
                if dn in st and un in st:
                    s.down.copy_(st.tensor(dn).to(s.down.dtype))
                    s.up.copy_(st.tensor(un).to(s.up.dtype))
                    if f"{s.key}.alpha" in st:
                        s.alpha = float(st.tensor(f"{s.key}.alpha").float())
                    n += 1
                    break
            else:
                if strict:
                    raise KeyError(f"{path}: no adapter for {s.key}")
    return n


def load_lora_state_sidecar(path, slots: Sequence[LoRASlot], optimizer) -> int:
    """Faithful resume: adapters + moments + bias-correction step. Returns the restored step."""
    st = SafeTensors(path)
    with torch.no_grad():
        for s in slots:
            s.down.copy_(st.tensor(f"{s.key}.lora_A.weight").to(s.down.dtype))
            s.up.copy_(st.tensor(f"{s.key}.lora_B.weight").to(s.up.dtype))
            for tag, p in (("lora_A", s.down), ("lora_B", s.up)):
                optimizer.set_moments(p, st.tensor(f"{s.key}.{tag}.adam_m"), st.tensor(f"{s.key}.{tag}.adam_v"))
    step = int(st.tensor("__meta__")[0].item()) if "__meta__" in st else 0
    optimizer.step_count = step
    return step


@torch.no_grad()
def merge_lora_into_weights(model: nn.Module, multiplier: float = 1.0) -> None:
    """Fold every adapter into a resident copy of its host weight and drop the slots (inference-time merge;
    saved base checkpoints are never touched: serenitymojo/lora.mojo:680-722)."""
    for m in model.modules():
        if isinstance(m, Linear) and len(m.slots):
            for s in m.slots:
                delta = (s.up.float() @ s.down.float()) * (s.scale * multiplier)
                m.weight[s.row0:s.row1] += delta.to(m.weight.dtype)
            m.slots = nn.ModuleList()


def sdxl_kohya_name(module_path: str) -> str:
    """LDM module path of a UNet linear -> Kohya SDXL key prefix (``lora_unet_`` + the path with dots as underscores)."""
    return "lora_unet_" + module_path.replace(".", "_")


def inject_sdxl_lora(model, rank: int = 16, alpha: float = 16.0, seed: int = 0) -> List[LoRASlot]:
    """SDXL UNet adapters on every linear of the SpatialTransformers (attn1 / attn2 q, k, v, out and the GEGLU feed-forward),
    the surface the reference trains (serenitymojo/models/sdxl/sdxl_unet_stack_lora.mojo; real-dims step
    serenitymojo/models/sdxl/sdxl_real_train.mojo:289,462), saved under Kohya's ``lora_unet_*`` names
    (serenitymojo/lora.mojo:61-75 ``FMT_KOHYA_SDXL``)."""
    names = {n: sdxl_kohya_name(n) for n in model.lora_target_names()}
    return inject_lora_by_name(model, names, rank, alpha)
