"""Lens DiT: a 48-block double-stream MMDiT of width 1536 (24 heads x 64) on 2 x 2 patches of a 32-channel latent, with the
text stream built from FOUR hidden layers of a GPT-OSS encoder.

Differences from the Qwen-Image block it otherwise follows (joint attention over image + text, text positions starting at
``max(h, w) / 2`` on all three rotary axes, centred image grid, six modulation chunks per stream in the order shift, scale,
gate for attention then for the feed-forward):
* the pre-norms are RMSNorms WITH a learned weight (``img_norm1 / img_norm2 / txt_norm1 / txt_norm2``, eps 1e-6);
* q | k | v of each stream come from one fused projection (``attn.img_qkv``, ``attn.txt_qkv``, with bias);
* the feed-forwards are SwiGLU without biases: ``w2(silu(w1 x) * w3 x)``, 4096 wide;
* rotary axes (8, 28, 28) of the 64-wide head, base 1e4, interleaved pairs;
* text input: hidden layers 5, 11, 17, 23 (2880 wide each) are RMS-normalised by their own weight (``txt_norm.0`` ..
  ``txt_norm.3``, eps 1e-5), concatenated to 11 520 features and projected by ``txt_in``; the first 97 tokens of the
  512-token chat-template encoding are dropped.

Behaviour: serenitymojo/models/lens/lens_contract.mojo:41-93 (sizes, text plan, scheduler constants),
serenitymojo/models/lens/lens_dit_math.mojo:233-266 (rotary angles), :1085-1122 (block order), :1179-1213 (tensor names and
shapes), :1320-1345 (text feature path). The reference verifies block 0 against captures and has no full forward; the parts
outside the block (timestep embedder, output modulation and projection) use the Qwen-Image names that make up the remaining
16 of the checkpoint's 1264 tensors.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, timestep_embedding
from .qwen_image import QwenImageDiT

LENS_TEXT_LAYERS = (5, 11, 17, 23)
LENS_TEXT_OFFSET = 97
LENS_MAX_TEXT_LEN = 512


@dataclass
class LensConfig:
    in_channels: int = 128
    hidden: int = 1536
    heads: int = 24
    head_dim: int = 64
    depth: int = 48
    mlp_hidden: int = 4096
    text_hidden: int = 2880
    text_layers: int = 4
    axes_dim: Tuple[int, ...] = (8, 28, 28)
    theta: float = 10000.0
    name: str = "lens"


def tiny_lens_config() -> LensConfig:
    return LensConfig(in_channels=16, hidden=128, heads=2, head_dim=64, depth=2, mlp_hidden=256, text_hidden=48, text_layers=4,
                      name="tiny-lens")


def lens_text_plan(tokens: int = LENS_MAX_TEXT_LEN, offset: int = LENS_TEXT_OFFSET, latent_hw: Tuple[int, int] = (64, 64)):
    """(text tokens kept, total joint sequence): 415 and 4511 for the 512-token template at 1024^2."""
    kept = tokens - offset
    return kept, kept + latent_hw[0] * latent_hw[1]


class _Attn(nn.Module):
    def __init__(self, cfg: LensConfig, dtype, device):
        super().__init__()
        D, Dh = cfg.hidden, cfg.head_dim
        self.img_qkv = Linear(D, 3 * D, True, dtype, device)
        self.txt_qkv = Linear(D, 3 * D, True, dtype, device)
        self.norm_q, self.norm_k = RMSNorm(Dh, 1e-6, dtype, device), RMSNorm(Dh, 1e-6, dtype, device)
        self.norm_added_q, self.norm_added_k = RMSNorm(Dh, 1e-6, dtype, device), RMSNorm(Dh, 1e-6, dtype, device)
        self.to_out = nn.ModuleList([Linear(D, D, True, dtype, device)])
        self.to_add_out = Linear(D, D, True, dtype, device)


class _SwiGLU(nn.Module):
    def __init__(self, dim, hidden, dtype, device):
        super().__init__()
        self.w1 = Linear(dim, hidden, False, dtype, device)
        self.w2 = Linear(hidden, dim, False, dtype, device)
        self.w3 = Linear(dim, hidden, False, dtype, device)

    def forward(self, x, residual, gate, rows):
        h = self.w1(x, act="silu") * self.w3(x)
        return self.w2(h, residual=residual, gate=gate, rows_per_group=rows)


class LensBlock(nn.Module):
    def __init__(self, cfg: LensConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        self.img_mod = nn.ModuleDict({"1": Linear(D, 6 * D, True, dtype, device)})
        self.txt_mod = nn.ModuleDict({"1": Linear(D, 6 * D, True, dtype, device)})
        self.img_norm1, self.img_norm2 = RMSNorm(D, 1e-6, dtype, device), RMSNorm(D, 1e-6, dtype, device)
        self.txt_norm1, self.txt_norm2 = RMSNorm(D, 1e-6, dtype, device), RMSNorm(D, 1e-6, dtype, device)
        self.attn = _Attn(cfg, dtype, device)
        self.img_mlp = _SwiGLU(D, cfg.mlp_hidden, dtype, device)
        self.txt_mlp = _SwiGLU(D, cfg.mlp_hidden, dtype, device)

    def forward(self, img, txt, temb_silu, cos, sin, kv_len=None):
        cfg, a = self.cfg, self.attn
        B, S_img, D = img.shape
        S_txt = txt.shape[1]
        H, Dh = cfg.heads, cfg.head_dim
        mi, mt = self.img_mod["1"](temb_silu), self.txt_mod["1"](temb_silu)
        i_sh1, i_sc1, i_g1, i_sh2, i_sc2, i_g2 = [mi[:, j * D:(j + 1) * D] for j in range(6)]
        t_sh1, t_sc1, t_g1, t_sh2, t_sc2, t_g2 = [mt[:, j * D:(j + 1) * D] for j in range(6)]
        qi = a.img_qkv(self.img_norm1(img, scale=i_sc1, shift=i_sh1))
        qt = a.txt_qkv(self.txt_norm1(txt, scale=t_sc1, shift=t_sh1))
        qi = ops.qk_norm_rope(qi, H, Dh, a.norm_q.weight, a.norm_k.weight, cos, sin, pos_offset=0)
        qt = ops.qk_norm_rope(qt, H, Dh, a.norm_added_q.weight, a.norm_added_k.weight, cos, sin, pos_offset=S_img)
        qkv = torch.cat((qi, qt), dim=1)
        q, k, v = [qkv[..., j * D:(j + 1) * D].unflatten(-1, (H, Dh)) for j in range(3)]
        o = ops.attention(q, k, v, kv_len=kv_len).reshape(B, S_img + S_txt, D)
        img = a.to_out[0](o[:, :S_img], residual=img, gate=i_g1, rows_per_group=S_img)
        txt = a.to_add_out(o[:, S_img:], residual=txt, gate=t_g1, rows_per_group=S_txt)
        img = self.img_mlp(self.img_norm2(img, scale=i_sc2, shift=i_sh2), img, i_g2, S_img)
        txt = self.txt_mlp(self.txt_norm2(txt, scale=t_sc2, shift=t_sh2), txt, t_g2, S_txt)
        return img, txt


class LensDiT(nn.Module):
    """forward(img [B, S_img, 128], text_layers [B, S_txt, 4, 2880] (or a sequence of four [B, S_txt, 2880]), t [B] in [0, 1],
    hw, txt_len [B] or None) -> velocity [B, S_img, 128]."""

    def __init__(self, cfg: LensConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        self.img_in = Linear(cfg.in_channels, D, True, dtype, device)
        self.txt_norm = nn.ModuleList([RMSNorm(cfg.text_hidden, 1e-5, dtype, device) for _ in range(cfg.text_layers)])
        self.txt_in = Linear(cfg.text_layers * cfg.text_hidden, D, True, dtype, device)
        te = nn.Module()
        te.linear_1 = Linear(256, D, True, dtype, device)
        te.linear_2 = Linear(D, D, True, dtype, device)
        self.time_text_embed = nn.ModuleDict({"timestep_embedder": te})
        self.transformer_blocks = nn.ModuleList([LensBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        no = nn.Module()
        no.linear = Linear(D, 2 * D, True, dtype, device)
        self.norm_out = no
        self.proj_out = Linear(D, cfg.in_channels, True, dtype, device)
        self.gradient_checkpointing = False

    make_ids = staticmethod(QwenImageDiT.make_ids)

    def text_tokens(self, text_layers) -> torch.Tensor:
        dt = self.img_in.weight.dtype
        if isinstance(text_layers, torch.Tensor):
            text_layers = text_layers.unbind(2)
        assert len(text_layers) == self.cfg.text_layers
        return self.txt_in(torch.cat([n(h.to(dt)) for n, h in zip(self.txt_norm, text_layers)], -1))

    def forward(self, img, text_layers, t, hw: Optional[Tuple[int, int]] = None, txt_len: Optional[torch.Tensor] = None):
        cfg = self.cfg
        S_img = img.shape[1]
        if hw is None:
            side = int(round(S_img ** 0.5))
            hw = (side, S_img // side)
        dt = self.img_in.weight.dtype
        txt = self.text_tokens(text_layers)
        S_txt = txt.shape[1]
        cos, sin = ops.rope_table(self.make_ids(hw[0], hw[1], S_txt, img.device), cfg.axes_dim, cfg.theta)
        te = self.time_text_embed["timestep_embedder"]
        temb_silu = ops.activation(te.linear_2(te.linear_1(timestep_embedding(t, 256).to(dt), act="silu")), "silu")
        img = self.img_in(img.to(dt))
        kv_len = (S_img + txt_len).to(torch.int32) if txt_len is not None else None
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.transformer_blocks:
            if ckpt:
                img, txt = torch.utils.checkpoint.checkpoint(blk, img, txt, temb_silu, cos, sin, kv_len, use_reentrant=False, preserve_rng_state=False)
            else:
                img, txt = blk(img, txt, temb_silu, cos, sin, kv_len)
        D = cfg.hidden
        m = self.norm_out.linear(temb_silu)
        return self.proj_out(ops.norm_modulate(img, scale=m[:, :D], shift=m[:, D:], eps=1e-6))

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
