"""Qwen-Image-shaped MMDiT: 60 double-stream blocks (no single blocks), D=3072, 24 heads x 128, text context 3584,
GELU-tanh MLP x4, per-head QK-RMSNorm, interleaved 3-axis RoPE (16,56,56), text-first joint attention with a padded-text
key mask. Facts: serenitymojo/models/dit/qwenimage_dit.mojo:10-53,87-107; forward variants :904-1194. Parameter names
are the diffusers transformer keys (serenitymojo/models/qwenimage/weights.mojo:95-223), which are also the full-finetune
payload keys (serenitymojo/models/zimage/full_finetune_checkpoint.mojo:52-77 describes the sibling layout).

The joint sequence is laid out image-first inside this implementation: attention is permutation invariant over keys
once RoPE has been applied per token, and with the text at the end a padded prompt becomes a plain key-length mask.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class QwenImageConfig:
    in_channels: int = 64
    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    depth: int = 60
    context_dim: int = 3584
    mlp_ratio: float = 4.0
    axes_dim: Tuple[int, ...] = (16, 56, 56)
    theta: float = 10000.0
    name: str = "qwen-image"


def qwen_image_config() -> QwenImageConfig:
    return QwenImageConfig()


def tiny_qwen_image_config() -> QwenImageConfig:
    return QwenImageConfig(hidden=256, heads=4, head_dim=64, depth=2, context_dim=128, axes_dim=(16, 24, 24),
                           name="tiny-qwen-image")


class JointAttention(nn.Module):
    def __init__(self, cfg: QwenImageConfig, dtype, device):
        super().__init__()
        D, Dh = cfg.hidden, cfg.head_dim
        self.cfg = cfg
        self.to_q, self.to_k, self.to_v = [Linear(D, D, True, dtype, device) for _ in range(3)]
        self.add_q_proj, self.add_k_proj, self.add_v_proj = [Linear(D, D, True, dtype, device) for _ in range(3)]
        self.to_out = nn.ModuleList([Linear(D, D, True, dtype, device)])
        self.to_add_out = Linear(D, D, True, dtype, device)
        self.norm_q, self.norm_k = RMSNorm(Dh, 1e-6, dtype, device), RMSNorm(Dh, 1e-6, dtype, device)
        self.norm_added_q, self.norm_added_k = RMSNorm(Dh, 1e-6, dtype, device), RMSNorm(Dh, 1e-6, dtype, device)

    def forward(self, img, txt, cos, sin, kv_len=None):
        cfg = self.cfg
        B, S_img, D = img.shape
        S_txt = txt.shape[1]
        H, Dh = cfg.heads, cfg.head_dim
        qi = packed_projection(img, (self.to_q, self.to_k, self.to_v))
        qt = packed_projection(txt, (self.add_q_proj, self.add_k_proj, self.add_v_proj))
        qi = ops.qk_norm_rope(qi, H, Dh, self.norm_q.weight, self.norm_k.weight, cos, sin, pos_offset=0)
        qt = ops.qk_norm_rope(qt, H, Dh, self.norm_added_q.weight, self.norm_added_k.weight, cos, sin, pos_offset=S_img)
        qkv = torch.cat((qi, qt), dim=1)
        q, k, v = [qkv[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3)]
        o = ops.attention(q, k, v, kv_len=kv_len).reshape(B, S_img + S_txt, D)
        return o[:, :S_img], o[:, S_img:]


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden: int, dtype, device):
        super().__init__()
        proj = nn.Module()
        proj.proj = Linear(dim, hidden, True, dtype, device)
        self.net = nn.ModuleDict({"0": proj, "2": Linear(hidden, dim, True, dtype, device)})

    def forward(self, x, residual, gate, rows):
        h = self.net["0"].proj(x, act="gelu_tanh")
        return self.net["2"](h, residual=residual, gate=gate, rows_per_group=rows)


class QwenBlock(nn.Module):
    def __init__(self, cfg: QwenImageConfig, dtype, device):
        super().__init__()
        D, F_ = cfg.hidden, int(cfg.hidden * cfg.mlp_ratio)
        self.img_mod = nn.ModuleDict({"1": Linear(D, 6 * D, True, dtype, device)})
        self.txt_mod = nn.ModuleDict({"1": Linear(D, 6 * D, True, dtype, device)})
        self.attn = JointAttention(cfg, dtype, device)
        self.img_mlp = FeedForward(D, F_, dtype, device)
        self.txt_mlp = FeedForward(D, F_, dtype, device)

    def forward(self, img, txt, temb_silu, cos, sin, kv_len=None):
        D = img.shape[-1]
        S_img, S_txt = img.shape[1], txt.shape[1]
        mi, mt = self.img_mod["1"](temb_silu), self.txt_mod["1"](temb_silu)
        i_sh1, i_sc1, i_g1, i_sh2, i_sc2, i_g2 = [mi[:, j * D:(j + 1) * D] for j in range(6)]
        t_sh1, t_sc1, t_g1, t_sh2, t_sc2, t_g2 = [mt[:, j * D:(j + 1) * D] for j in range(6)]
        a_img, a_txt = self.attn(ops.norm_modulate(img, scale=i_sc1, shift=i_sh1, eps=1e-6),
                                 ops.norm_modulate(txt, scale=t_sc1, shift=t_sh1, eps=1e-6), cos, sin, kv_len)
        img = self.attn.to_out[0](a_img, residual=img, gate=i_g1, rows_per_group=S_img)
        txt = self.attn.to_add_out(a_txt, residual=txt, gate=t_g1, rows_per_group=S_txt)
        img = self.img_mlp(ops.norm_modulate(img, scale=i_sc2, shift=i_sh2, eps=1e-6), img, i_g2, S_img)
        txt = self.txt_mlp(ops.norm_modulate(txt, scale=t_sc2, shift=t_sh2, eps=1e-6), txt, t_g2, S_txt)
        return img, txt


class QwenImageDiT(nn.Module):
    """forward(img [B,S_img,64], txt [B,S_txt,3584], t [B] in [0,1], txt_len=None) -> velocity [B,S_img,64]."""

    def __init__(self, cfg: QwenImageConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        self.img_in = Linear(cfg.in_channels, D, True, dtype, device)
        self.txt_norm = RMSNorm(cfg.context_dim, 1e-6, dtype, device)
        self.txt_in = Linear(cfg.context_dim, D, True, dtype, device)
        te = nn.Module()
        te.linear_1 = Linear(256, D, True, dtype, device)
        te.linear_2 = Linear(D, D, True, dtype, device)
        self.time_text_embed = nn.ModuleDict({"timestep_embedder": te})
        self.transformer_blocks = nn.ModuleList([QwenBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        no = nn.Module()
        no.linear = Linear(D, 2 * D, True, dtype, device)
        self.norm_out = no
        self.proj_out = Linear(D, cfg.in_channels, True, dtype, device)
        self.gradient_checkpointing = False

    @staticmethod
    def make_ids(h: int, w: int, n_txt: int, device=None) -> torch.Tensor:
        """image tokens first: (0, row - h/2, col - w/2) centred grid; text token i at (max(h,w)/2 + i) on all axes."""
        ids = torch.zeros(h * w + n_txt, 3, dtype=torch.float32, device=device)
        ids[:h * w, 1] = (torch.arange(h, device=device, dtype=torch.float32) - h // 2)[:, None].expand(h, w).reshape(-1)
        ids[:h * w, 2] = (torch.arange(w, device=device, dtype=torch.float32) - w // 2)[None, :].expand(h, w).reshape(-1)
        base = max(h, w) // 2
        ids[h * w:] = (base + torch.arange(n_txt, device=device, dtype=torch.float32))[:, None]
        return ids

    def forward(self, img, txt, t, hw: Optional[Tuple[int, int]] = None, txt_len: Optional[torch.Tensor] = None):
        cfg = self.cfg
        S_img, S_txt = img.shape[1], txt.shape[1]
        if hw is None:
            side = int(round(S_img ** 0.5))
            hw = (side, S_img // side)
        dt = self.img_in.weight.dtype
        cos, sin = ops.rope_table(self.make_ids(hw[0], hw[1], S_txt, img.device), cfg.axes_dim, cfg.theta)
        te = self.time_text_embed["timestep_embedder"]
        temb = te.linear_2(te.linear_1(timestep_embedding(t, 256).to(dt), act="silu"))
        temb_silu = ops.activation(temb, "silu")
        img = self.img_in(img.to(dt))
        txt = self.txt_in(self.txt_norm(txt.to(dt)))
        kv_len = (S_img + txt_len).to(torch.int32) if txt_len is not None else None
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.transformer_blocks:
            if ckpt:
                img, txt = torch.utils.checkpoint.checkpoint(blk, img, txt, temb_silu, cos, sin, kv_len, use_reentrant=False, preserve_rng_state=False)
            else:
                img, txt = blk(img, txt, temb_silu, cos, sin, kv_len)
        D = cfg.hidden
        m = self.norm_out.linear(temb_silu)
        scale, shift = m[:, :D], m[:, D:]
        return self.proj_out(ops.norm_modulate(img, scale=scale, shift=shift, eps=1e-6))

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
