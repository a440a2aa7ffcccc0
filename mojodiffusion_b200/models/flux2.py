"""FLUX.2 Klein-shaped MMDiT: double + single stream blocks like FLUX.1, but with ONE modulation per stream kind shared
by every block (computed once per step from the timestep vector), SwiGLU MLPs (fused gate|up projection), no biases
anywhere, four RoPE axes of 32 dims (theta 2000; image token (0,row,col,0), text token k at (0,0,0,k)), no pooled-vector
or guidance embedder.

Sizes: Klein 9B = 8 double + 24 single, D 4096, 32 heads x 128, MLP 12288, text dim 12288, 128 latent channels per token;
Klein 4B = 5 + 20, D 3072, 24 heads. Parameter names are the BFL checkpoint keys: ``double_blocks.{i}.img_attn.qkv.weight``,
``double_blocks.{i}.img_mlp.{0,2}.weight``, ``single_blocks.{i}.linear{1,2}.weight``,
``double_stream_modulation_{img,txt}.lin.weight``, ``single_stream_modulation.lin.weight``,
``time_in.{in,out}_layer.weight``, ``final_layer.adaLN_modulation.1.weight``.

Facts: serenitymojo/models/dit/klein_dit.mojo:33-48 (sizes), :95-145 (keys), :320-425 (block op order),
:555-610 (RoPE positions); serenitymojo/models/klein/double_block.mojo:52-76.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import native
from .layers import Linear, init_module_weights, timestep_embedding
from .mmdit import QKNorm


@dataclass
class Flux2Config:
    in_channels: int = 128
    context_dim: int = 12288
    hidden: int = 4096
    heads: int = 32
    head_dim: int = 128
    depth_double: int = 8
    depth_single: int = 24
    mlp_hidden: int = 12288
    axes_dim: Tuple[int, ...] = (32, 32, 32, 32)
    theta: float = 2000.0
    time_dim: int = 256
    name: str = "flux2-klein-9b"


def klein_9b_config() -> Flux2Config:
    return Flux2Config()


def klein_4b_config() -> Flux2Config:
    return Flux2Config(context_dim=7680, hidden=3072, heads=24, depth_double=5, depth_single=20, mlp_hidden=9216,
                       name="flux2-klein-4b")


def tiny_flux2_config() -> Flux2Config:
    return Flux2Config(in_channels=32, context_dim=128, hidden=256, heads=4, head_dim=64, depth_double=2, depth_single=2,
                       mlp_hidden=512, axes_dim=(16, 16, 16, 16), name="tiny-flux2")


def _fused(x: torch.Tensor) -> bool:
    return native.use_native(x) and not torch.is_grad_enabled()


class _Attn(nn.Module):
    def __init__(self, cfg: Flux2Config, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.qkv = Linear(D, 3 * D, False, dtype, device)
        self.norm = QKNorm(cfg.head_dim, dtype, device)
        self.proj = Linear(D, D, False, dtype, device)


def _swiglu_mlp(cfg: Flux2Config, dtype, device) -> nn.ModuleDict:
    return nn.ModuleDict({"0": Linear(cfg.hidden, 2 * cfg.mlp_hidden, False, dtype, device),
                          "2": Linear(cfg.mlp_hidden, cfg.hidden, False, dtype, device)})


def _gated_up(lin: Linear, x: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up from the fused [2F, D] projection: one GEMM with the product in its epilogue at inference,
    projection + GLU node (native backward) under autograd or with adapters attached."""
    if _fused(x) and len(lin.slots) == 0:
        return ops.linear_glu(x, lin.weight, None, "silu", False)
    return ops.glu(lin(x), "silu", False)


class Flux2DoubleBlock(nn.Module):
    def __init__(self, cfg: Flux2Config, dtype, device):
        super().__init__()
        self.cfg = cfg
        self.img_attn = _Attn(cfg, dtype, device)
        self.img_mlp = _swiglu_mlp(cfg, dtype, device)
        self.txt_attn = _Attn(cfg, dtype, device)
        self.txt_mlp = _swiglu_mlp(cfg, dtype, device)

    def forward(self, img, txt, mod_img, mod_txt, cos, sin):
        cfg = self.cfg
        B, S_img, D = img.shape
        S_txt = txt.shape[1]
        H, Dh = cfg.heads, cfg.head_dim
        i_shift1, i_scale1, i_gate1, i_shift2, i_scale2, i_gate2 = [mod_img[:, j * D:(j + 1) * D] for j in range(6)]
        t_shift1, t_scale1, t_gate1, t_shift2, t_scale2, t_gate2 = [mod_txt[:, j * D:(j + 1) * D] for j in range(6)]
        img_n = ops.norm_modulate(img, scale=i_scale1, shift=i_shift1, eps=1e-6)
        txt_n = ops.norm_modulate(txt, scale=t_scale1, shift=t_shift1, eps=1e-6)
        wqi, wki = self.img_attn.norm.query_norm.scale, self.img_attn.norm.key_norm.scale
        wqt, wkt = self.txt_attn.norm.query_norm.scale, self.txt_attn.norm.key_norm.scale
        qkv = torch.cat((self.txt_attn.qkv(txt_n), self.img_attn.qkv(img_n)), dim=1)      # txt first on the sequence
        attn = ops.qkv_attention(qkv, H, Dh, wqi, wki, cos, sin, split=S_txt, wq_first=wqt, wk_first=wkt)
        txt_a, img_a = attn[:, :S_txt], attn[:, S_txt:]
        img = self.img_attn.proj(img_a, residual=img, gate=i_gate1, rows_per_group=S_img)
        txt = self.txt_attn.proj(txt_a, residual=txt, gate=t_gate1, rows_per_group=S_txt)
        h = _gated_up(self.img_mlp["0"], ops.norm_modulate(img, scale=i_scale2, shift=i_shift2, eps=1e-6))
        img = self.img_mlp["2"](h, residual=img, gate=i_gate2, rows_per_group=S_img)
        h = _gated_up(self.txt_mlp["0"], ops.norm_modulate(txt, scale=t_scale2, shift=t_shift2, eps=1e-6))
        txt = self.txt_mlp["2"](h, residual=txt, gate=t_gate2, rows_per_group=S_txt)
        return img, txt


class Flux2SingleBlock(nn.Module):
    def __init__(self, cfg: Flux2Config, dtype, device):
        super().__init__()
        self.cfg = cfg
        D, F_ = cfg.hidden, cfg.mlp_hidden
        self.linear1 = Linear(D, 3 * D + 2 * F_, False, dtype, device)      # [q | k | v | gate | up]
        self.linear2 = Linear(D + F_, D, False, dtype, device)              # [attn | silu(gate) * up] -> D
        self.norm = QKNorm(cfg.head_dim, dtype, device)

    def forward(self, x, mod, cos, sin):
        cfg = self.cfg
        B, S, D = x.shape
        H, Dh = cfg.heads, cfg.head_dim
        shift, scale, gate = mod[:, 0:D], mod[:, D:2 * D], mod[:, 2 * D:3 * D]
        xn = ops.norm_modulate(x, scale=scale, shift=shift, eps=1e-6)
        wq, wk = self.norm.query_norm.scale, self.norm.key_norm.scale
        if _fused(x) and len(self.linear1.slots) == 0 and len(self.linear2.slots) == 0:
            w1, w2 = self.linear1.weight, self.linear2.weight
            qkv = ops.linear(xn, w1[:3 * D])
            mlp = ops.linear_glu(xn, w1[3 * D:], None, "silu", False)
            attn = ops.qkv_attention(qkv, H, Dh, wq, wk, cos, sin)
            return ops.linear(attn, w2[:, :D], None, residual=x, gate=gate, rows_per_group=S, extra=[(mlp, w2[:, D:])])
        mid = ops.packed_attention_mlp(self.linear1(xn), H, Dh, wq, wk, cos, sin, act="silu", gated=False)
        return self.linear2(mid, residual=x, gate=gate, rows_per_group=S)


class _Mod(nn.Module):
    def __init__(self, dim: int, n: int, dtype, device):
        super().__init__()
        self.lin = Linear(dim, n * dim, False, dtype, device)

    def forward(self, vec_silu):
        return self.lin(vec_silu)


class _TimeIn(nn.Module):
    def __init__(self, in_dim, hidden, dtype, device):
        super().__init__()
        self.in_layer = Linear(in_dim, hidden, False, dtype, device)
        self.out_layer = Linear(hidden, hidden, False, dtype, device)

    def forward(self, x):
        return self.out_layer(self.in_layer(x, act="silu"))


class _Final(nn.Module):
    def __init__(self, hidden, out_channels, dtype, device):
        super().__init__()
        self.linear = Linear(hidden, out_channels, False, dtype, device)
        self.adaLN_modulation = nn.ModuleDict({"1": Linear(hidden, 2 * hidden, False, dtype, device)})

    def forward(self, x, vec_silu):
        D = x.shape[-1]
        m = self.adaLN_modulation["1"](vec_silu)
        return self.linear(ops.norm_modulate(x, scale=m[:, D:], shift=m[:, :D], eps=1e-6))


class Flux2DiT(nn.Module):
    """forward(img [B,S_img,128], txt [B,S_txt,ctx], t [B] in [0,1], hw) -> velocity [B,S_img,128]."""

    def __init__(self, cfg: Flux2Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert cfg.heads * cfg.head_dim == D and sum(cfg.axes_dim) == cfg.head_dim
        self.img_in = Linear(cfg.in_channels, D, False, dtype, device)
        self.txt_in = Linear(cfg.context_dim, D, False, dtype, device)
        self.time_in = _TimeIn(cfg.time_dim, D, dtype, device)
        self.double_stream_modulation_img = _Mod(D, 6, dtype, device)
        self.double_stream_modulation_txt = _Mod(D, 6, dtype, device)
        self.single_stream_modulation = _Mod(D, 3, dtype, device)
        self.double_blocks = nn.ModuleList([Flux2DoubleBlock(cfg, dtype, device) for _ in range(cfg.depth_double)])
        self.single_blocks = nn.ModuleList([Flux2SingleBlock(cfg, dtype, device) for _ in range(cfg.depth_single)])
        self.final_layer = _Final(D, cfg.in_channels, dtype, device)
        self.gradient_checkpointing = False

    @staticmethod
    def make_ids(h: int, w: int, n_txt: int, device=None) -> torch.Tensor:
        """[n_txt + h*w, 4]: text token k at (0,0,0,k), image token at (0,row,col,0)."""
        ids = torch.zeros(n_txt + h * w, 4, dtype=torch.float32, device=device)
        ids[:n_txt, 3] = torch.arange(n_txt, device=device, dtype=torch.float32)
        ids[n_txt:, 1] = torch.arange(h, device=device, dtype=torch.float32)[:, None].expand(h, w).reshape(-1)
        ids[n_txt:, 2] = torch.arange(w, device=device, dtype=torch.float32)[None, :].expand(h, w).reshape(-1)
        return ids

    def forward(self, img, txt, timesteps, hw: Optional[Tuple[int, int]] = None):
        cfg = self.cfg
        S_txt, S_img = txt.shape[1], img.shape[1]
        if hw is None:
            side = int(round(S_img ** 0.5))
            hw = (side, S_img // side)
        cos, sin = ops.rope_table(self.make_ids(hw[0], hw[1], S_txt, img.device), cfg.axes_dim, cfg.theta)
        dt = self.img_in.weight.dtype
        img = self.img_in(img.to(dt))
        txt = self.txt_in(txt.to(dt))
        vec_silu = ops.activation(self.time_in(timestep_embedding(timesteps, cfg.time_dim).to(dt)), "silu")
        mod_img = self.double_stream_modulation_img(vec_silu)
        mod_txt = self.double_stream_modulation_txt(vec_silu)
        mod_single = self.single_stream_modulation(vec_silu)
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.double_blocks:
            if ckpt:
                img, txt = torch.utils.checkpoint.checkpoint(blk, img, txt, mod_img, mod_txt, cos, sin, use_reentrant=False, preserve_rng_state=False)
            else:
                img, txt = blk(img, txt, mod_img, mod_txt, cos, sin)
        x = torch.cat((txt, img), dim=1)
        for blk in self.single_blocks:
            if ckpt:
                x = torch.utils.checkpoint.checkpoint(blk, x, mod_single, cos, sin, use_reentrant=False, preserve_rng_state=False)
            else:
                x = blk(x, mod_single, cos, sin)
        return self.final_layer(x[:, S_txt:], vec_silu)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)

    def lora_target_names(self):
        """Module paths of the attention and MLP projections of every block (the reference's Klein LoRA surface)."""
        return [n for n, m in self.named_modules() if isinstance(m, Linear) and (n.startswith("double_blocks.") or n.startswith("single_blocks."))]
