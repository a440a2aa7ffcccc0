"""HunyuanVideo-1.5 DiT: 54 double-stream blocks (no single-stream stage) over video tokens and pre-projected text.

Width 2048 (16 heads x 128), patch 1 x 1 x 1 over a 65-channel input (32 latent + 32 condition + 1 mask channels are
concatenated by the caller), per-stream adaLN (shift, scale, gate) x 2 from ``silu(time MLP)``, separate q / k / v
projections with per-head QK-RMSNorm, half-split three-axis rotary (16, 56, 56; theta 256) on the video tokens only,
joint attention over [video, text], GELU-tanh MLP, final adaLN + linear to 32 channels. In the joint attention buffer the
text rows come first here (attention without a mask does not depend on the row order); their rotary rows are identity.

Behaviour and checkpoint keys: serenitymojo/models/dit/hunyuan15_dit.mojo:19-534.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops.conv import patchify_3d, unpatchify_3d
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class Hunyuan15Config:
    in_channels: int = 65
    out_channels: int = 32
    hidden: int = 2048
    heads: int = 16
    head_dim: int = 128
    depth: int = 54
    mlp_ratio: int = 4
    patch: Tuple[int, int, int] = (1, 1, 1)
    axes_dim: Tuple[int, int, int] = (16, 56, 56)
    theta: float = 256.0
    eps: float = 1e-6
    name: str = "hunyuan-video-1.5"


def tiny_hunyuan15_config() -> Hunyuan15Config:
    return Hunyuan15Config(in_channels=9, out_channels=4, hidden=128, heads=2, head_dim=64, depth=2,
                           axes_dim=(16, 24, 24), name="tiny-hunyuan15")


class _Mod(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        self.linear = Linear(dim, 6 * dim, True, dtype, device)


class _Mlp(nn.Module):
    def __init__(self, dim, hidden, dtype, device):
        super().__init__()
        self.fc1 = Linear(dim, hidden, True, dtype, device)
        self.fc2 = Linear(hidden, dim, True, dtype, device)


class Hunyuan15Block(nn.Module):
    def __init__(self, cfg: Hunyuan15Config, dtype, device):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        for s in ("img", "txt"):
            setattr(self, f"{s}_mod", _Mod(D, dtype, device))
            for p in ("q", "k", "v"):
                setattr(self, f"{s}_attn_{p}", Linear(D, D, True, dtype, device))
            setattr(self, f"{s}_attn_q_norm", RMSNorm(cfg.head_dim, cfg.eps, dtype, device))
            setattr(self, f"{s}_attn_k_norm", RMSNorm(cfg.head_dim, cfg.eps, dtype, device))
            setattr(self, f"{s}_attn_proj", Linear(D, D, True, dtype, device))
            setattr(self, f"{s}_mlp", _Mlp(D, cfg.mlp_ratio * D, dtype, device))

    def forward(self, img, txt, vec_silu, cos, sin):
        cfg = self.cfg
        D, S_txt, S_img = cfg.hidden, txt.shape[1], img.shape[1]
        mi = self.img_mod.linear(vec_silu)
        mt = self.txt_mod.linear(vec_silu)
        i_sh1, i_sc1, i_g1, i_sh2, i_sc2, i_g2 = (mi[:, j * D:(j + 1) * D] for j in range(6))
        t_sh1, t_sc1, t_g1, t_sh2, t_sc2, t_g2 = (mt[:, j * D:(j + 1) * D] for j in range(6))
        img_n = ops.norm_modulate(img, scale=i_sc1, shift=i_sh1, eps=cfg.eps)
        txt_n = ops.norm_modulate(txt, scale=t_sc1, shift=t_sh1, eps=cfg.eps)
        qkv = torch.cat((packed_projection(txt_n, (self.txt_attn_q, self.txt_attn_k, self.txt_attn_v)),
                         packed_projection(img_n, (self.img_attn_q, self.img_attn_k, self.img_attn_v))), dim=1)
        attn = ops.qkv_attention(qkv, cfg.heads, cfg.head_dim, self.img_attn_q_norm.weight, self.img_attn_k_norm.weight,
                                 cos, sin, split=S_txt, wq_first=self.txt_attn_q_norm.weight,
                                 wk_first=self.txt_attn_k_norm.weight, interleaved=False, eps=cfg.eps)
        img = self.img_attn_proj(attn[:, S_txt:], residual=img, gate=i_g1, rows_per_group=S_img)
        txt = self.txt_attn_proj(attn[:, :S_txt], residual=txt, gate=t_g1, rows_per_group=S_txt)
        h = self.img_mlp.fc1(ops.norm_modulate(img, scale=i_sc2, shift=i_sh2, eps=cfg.eps), act="gelu_tanh")
        img = self.img_mlp.fc2(h, residual=img, gate=i_g2, rows_per_group=S_img)
        h = self.txt_mlp.fc1(ops.norm_modulate(txt, scale=t_sc2, shift=t_sh2, eps=cfg.eps), act="gelu_tanh")
        txt = self.txt_mlp.fc2(h, residual=txt, gate=t_g2, rows_per_group=S_txt)
        return img, txt


class _PatchIn(nn.Module):
    def __init__(self, cfg: Hunyuan15Config, dtype, device):
        super().__init__()
        self.proj = nn.Conv3d(cfg.in_channels, cfg.hidden, cfg.patch, cfg.patch, dtype=dtype, device=device)


class _TimeIn(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        self.mlp = nn.ModuleDict({"0": Linear(256, dim, True, dtype, device), "2": Linear(dim, dim, True, dtype, device)})


class _Final(nn.Module):
    def __init__(self, cfg: Hunyuan15Config, dtype, device):
        super().__init__()
        pt, ph, pw = cfg.patch
        self.adaLN_modulation = nn.ModuleDict({"1": Linear(cfg.hidden, 2 * cfg.hidden, True, dtype, device)})
        self.linear = Linear(cfg.hidden, cfg.out_channels * pt * ph * pw, True, dtype, device)


class Hunyuan15DiT(nn.Module):
    """forward(latent [B, C_in, F, H, W], text [B, S_txt, hidden] (already projected), t [B] in [0, 1]) ->
    velocity [B, C_out, F, H, W]."""

    def __init__(self, cfg: Hunyuan15Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        assert sum(cfg.axes_dim) == cfg.head_dim and cfg.heads * cfg.head_dim == cfg.hidden
        self.img_in = _PatchIn(cfg, dtype, device)
        self.time_in = _TimeIn(cfg.hidden, dtype, device)
        self.double_blocks = nn.ModuleList([Hunyuan15Block(cfg, dtype, device) for _ in range(cfg.depth)])
        self.final_layer = _Final(cfg, dtype, device)
        self.gradient_checkpointing = False

    def rope(self, f: int, h: int, w: int, n_txt: int, device):
        """cos / sin [n_txt + f h w, head_dim / 2]: identity rows for the text, (t, y, x) positions for the video."""
        t = torch.arange(f, device=device, dtype=torch.float32)[:, None, None].expand(f, h, w)
        y = torch.arange(h, device=device, dtype=torch.float32)[None, :, None].expand(f, h, w)
        x = torch.arange(w, device=device, dtype=torch.float32)[None, None, :].expand(f, h, w)
        cos, sin = ops.rope_table(torch.stack((t, y, x), -1).reshape(-1, 3).contiguous(), list(self.cfg.axes_dim), self.cfg.theta)
        return (torch.cat((torch.ones(n_txt, cos.shape[1], device=device), cos), 0),
                torch.cat((torch.zeros(n_txt, sin.shape[1], device=device), sin), 0))

    def forward(self, z, text, timesteps):
        cfg = self.cfg
        B, C, F_, Hh, Ww = z.shape
        pt, ph, pw = cfg.patch
        grid = (F_ // pt, Hh // ph, Ww // pw)
        dt = self.img_in.proj.weight.dtype
        img = ops.linear(patchify_3d(z, pt, ph, pw).to(dt), self.img_in.proj.weight.flatten(1), self.img_in.proj.bias)
        te = self.time_in.mlp
        vec = te["2"](te["0"](timestep_embedding(timesteps, 256).to(dt), act="silu"))
        vec_silu = ops.activation(vec, "silu")
        txt = text.to(dt)
        cos, sin = self.rope(*grid, txt.shape[1], z.device)
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.double_blocks:
            if ckpt:
                img, txt = torch.utils.checkpoint.checkpoint(blk, img, txt, vec_silu, cos, sin, use_reentrant=False, preserve_rng_state=False)
            else:
                img, txt = blk(img, txt, vec_silu, cos, sin)
        m = self.final_layer.adaLN_modulation["1"](vec_silu)
        D = cfg.hidden
        out = self.final_layer.linear(ops.norm_modulate(img, scale=m[:, D:], shift=m[:, :D], eps=cfg.eps))
        return unpatchify_3d(out, grid, cfg.out_channels, pt, ph, pw)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
