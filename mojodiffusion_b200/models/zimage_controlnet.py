"""Z-Image ControlNet (the DiT pattern, not the UNet zero-convolution pattern): every control block is a copy of one main
transformer block plus zero-initialised projections.

    control tokens -> control_all_x_embedder -> control_noise_refiner blocks (image rope, adaLN)
    c = cat(control tokens, caption features of the base)                       (same unified order as the base)
    block 0:  c = before_proj(c) + unified            unified = the base's input to its main layers
    block i:  c = TransformerBlock_i(c);  hint_i = after_proj_i(c)
    base:     unified = layer_p(unified);  unified += scale * hint_i            for p = places[i]

Places are evenly spaced ``i * depth // n`` (always containing 0). A fresh network copies the base's ``layers[place]``,
``noise_refiner[j]`` and ``all_x_embedder`` weights; projections start at zero, so step 0 reproduces the base exactly.
Checkpoint keys: ``control_layers.{i}.<block keys>``, ``control_layers.{i}.{before_proj (i = 0),after_proj}.{weight,bias}``,
``control_noise_refiner.{j}.*``, ``control_all_x_embedder.2-1.{weight,bias}``
(serenitymojo/models/zimage/controlnet_block.mojo:13-52, serenitymojo/training/controlnet_zimage.mojo:14-50).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
from torch import nn

from .layers import Linear
from .single_dit import Block, SingleDiTConfig, SingleStreamDiT


def control_places(depth: int, n: int) -> List[int]:
    return [i * depth // n for i in range(n)]


class ControlBlock(Block):
    def __init__(self, cfg: SingleDiTConfig, first: bool, dtype, device):
        super().__init__(cfg, True, dtype, device)
        D = cfg.hidden
        if first:
            self.before_proj = Linear(D, D, True, dtype, device)
        self.after_proj = Linear(D, D, True, dtype, device)


class ZImageControlNet(nn.Module):
    def __init__(self, cfg: SingleDiTConfig, n_layers: int, control_in_dim: Optional[int] = None, n_refiner: Optional[int] = None,
                 dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.places = control_places(cfg.depth, n_layers)
        assert 0 in self.places and len(set(self.places)) == n_layers, "control places must be distinct and contain layer 0"
        cin = control_in_dim or cfg.in_channels
        self.control_all_x_embedder = nn.ModuleDict({"2-1": Linear(cin, cfg.hidden, True, dtype, device)})
        nr = cfg.depth_noise_refiner if n_refiner is None else n_refiner
        self.control_noise_refiner = nn.ModuleList([Block(cfg, True, dtype, device) for _ in range(nr)])
        self.control_layers = nn.ModuleList([ControlBlock(cfg, i == 0, dtype, device) for i in range(n_layers)])

    @torch.no_grad()
    def init_from_base(self, base: SingleStreamDiT):
        """Copy-from-base initialisation; zero projections."""
        def copy_block(dst, src):
            sd = src.state_dict()
            dst.load_state_dict({k: v for k, v in sd.items()}, strict=False)
        for i, p in enumerate(self.places):
            copy_block(self.control_layers[i], base.layers[p])
            blk = self.control_layers[i]
            for proj in ([blk.before_proj] if i == 0 else []) + [blk.after_proj]:
                proj.weight.zero_()
                proj.bias.zero_()
        for j, blk in enumerate(self.control_noise_refiner):
            copy_block(blk, base.noise_refiner[min(j, len(base.noise_refiner) - 1)])
        src = base.all_x_embedder["2-1"]
        dst = self.control_all_x_embedder["2-1"]
        if dst.weight.shape == src.weight.shape:
            dst.weight.copy_(src.weight)
            dst.bias.copy_(src.bias)
        return self

    def forward(self, base: SingleStreamDiT, st: dict, control: torch.Tensor, scale: float = 1.0) -> Dict[int, torch.Tensor]:
        """st: the dict returned by ``base.embed``; control [B, S_img, control_in] (packed, normalised control latent).
        Returns {main layer index: hint [B, S_img + S_cap, D]} already multiplied by ``scale``."""
        c = self.control_all_x_embedder["2-1"](control.to(st["dt"]))
        for blk in self.control_noise_refiner:
            c = base._run(blk, c, st["cos_img"], st["sin_img"], st["c"])
        c = torch.cat((c, st["cap"]), dim=1)
        hints: Dict[int, torch.Tensor] = {}
        for i, blk in enumerate(self.control_layers):
            if i == 0:
                c = blk.before_proj(c) + st["h"]
            c = base._run(blk, c, st["cos"], st["sin"], st["c"], st["kv_len"])
            hint = blk.after_proj(c)
            hints[self.places[i]] = hint * scale if scale != 1.0 else hint
        return hints

    def trainable_parameters(self):
        return [p for p in self.parameters()]


class ControlledZImage(nn.Module):
    """The frozen base and its control branch as one module with the base's call signature plus ``control``: what the
    family trainer and the samplers drive."""

    def __init__(self, base: SingleStreamDiT, net: ZImageControlNet, scale: float = 1.0):
        super().__init__()
        self.base, self.controlnet, self.scale = base, net, scale
        self.cfg = base.cfg
        for p in base.parameters():
            p.requires_grad_(False)

    def forward(self, img, cap, t, hw=None, cap_len=None, control=None):
        if control is None:
            return self.base(img, cap, t, hw, cap_len)
        return self.base(img, cap, t, hw, cap_len, control=(self.controlnet, control), control_scale=self.scale)


def save_controlnet(net: ZImageControlNet, path: str, metadata: Optional[dict] = None):
    from ..io.safetensors_io import save_safetensors
    save_safetensors(path, {k: v.detach().cpu().contiguous() for k, v in net.state_dict().items()}, metadata or {})


def load_controlnet(net: ZImageControlNet, path: str):
    from ..io.safetensors_io import load_safetensors
    sd = load_safetensors(path)
    missing, unexpected = net.load_state_dict({k: v.to(next(net.parameters()).dtype) for k, v in sd.items()}, strict=False)
    if missing or unexpected:
        raise ValueError(f"control checkpoint does not match: missing {missing[:4]}, unexpected {unexpected[:4]}")
    return net
