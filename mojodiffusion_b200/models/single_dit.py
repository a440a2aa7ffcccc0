"""Single-stream DiT in the Z-Image / NextDiT style: one token stream (caption tokens + image tokens), SwiGLU MLPs,
QK-RMSNorm, half-split 3-axis RoPE, tanh-gated adaLN with sandwich RMSNorms, separate noise / context refiners.

Shape facts follow serenitymojo/models/dit/zimage_dit.mojo:80-105 (D=3840, 30 heads x 128, 30 main + 2 noise-refiner +
2 context-refiner layers, caption dim 2560, RoPE axes (32,48,48), t_scale 1000); parameter names are the diffusers
keys of serenitymojo/models/zimage/full_finetune_inventory.mojo:15-60 (`layers.{i}.attention.to_q` ...).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class SingleDiTConfig:
    in_channels: int = 64            # 16 latent channels x 2x2 patch
    hidden: int = 3840
    heads: int = 30
    head_dim: int = 128
    depth: int = 30
    depth_noise_refiner: int = 2
    depth_context_refiner: int = 2
    cap_dim: int = 2560
    mlp_hidden: int = 10240
    axes_dim: Tuple[int, ...] = (32, 48, 48)
    theta: float = 256.0
    t_scale: float = 1000.0
    adaln_dim: int = 256
    norm_eps: float = 1e-5
    name: str = "zimage"
    patch_key: str = "2-1"         # name of the patch embedder / final layer ("<patch>-<frame patch>")
    rope_interleaved: bool = False  # True: rotary pairs are (2i, 2i + 1); False: (i, i + Dh / 2)
    final_layer: bool = True       # False: the trunk ends at the hidden image tokens (a pixel head follows elsewhere)


def zimage_config() -> SingleDiTConfig:
    return SingleDiTConfig()


def tiny_single_dit_config() -> SingleDiTConfig:
    return SingleDiTConfig(in_channels=64, hidden=256, heads=4, head_dim=64, depth=2, depth_noise_refiner=1,
                           depth_context_refiner=1, cap_dim=128, mlp_hidden=512, axes_dim=(16, 24, 24), adaln_dim=64,
                           name="tiny-single-dit")


class Attention(nn.Module):
    def __init__(self, cfg: SingleDiTConfig, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.cfg = cfg
        self.to_q = Linear(D, D, False, dtype, device)
        self.to_k = Linear(D, D, False, dtype, device)
        self.to_v = Linear(D, D, False, dtype, device)
        self.to_out = nn.ModuleList([Linear(D, D, False, dtype, device)])
        self.norm_q = RMSNorm(cfg.head_dim, cfg.norm_eps, dtype, device)
        self.norm_k = RMSNorm(cfg.head_dim, cfg.norm_eps, dtype, device)

    def forward(self, x, cos, sin, kv_len=None):
        cfg = self.cfg
        B, S, D = x.shape
        H, Dh = cfg.heads, cfg.head_dim
        qkv = packed_projection(x, (self.to_q, self.to_k, self.to_v))
        qkv = ops.qk_norm_rope(qkv, H, Dh, self.norm_q.weight, self.norm_k.weight, cos, sin, eps=cfg.norm_eps,
                               interleaved=cfg.rope_interleaved)
        q, k, v = [qkv[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3)]
        return self.to_out[0](ops.attention(q, k, v, kv_len=kv_len).reshape(B, S, D))


class FeedForward(nn.Module):
    def __init__(self, dim: int, hidden: int, dtype, device):
        super().__init__()
        self.w1 = Linear(dim, hidden, False, dtype, device)   # gate
        self.w2 = Linear(hidden, dim, False, dtype, device)   # down
        self.w3 = Linear(dim, hidden, False, dtype, device)   # up

    def forward(self, x):
        return self.w2(ops.glu(packed_projection(x, (self.w1, self.w3)), "silu"))


class Block(nn.Module):
    def __init__(self, cfg: SingleDiTConfig, modulation: bool, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.modulation = modulation
        self.attention = Attention(cfg, dtype, device)
        self.feed_forward = FeedForward(D, cfg.mlp_hidden, dtype, device)
        self.attention_norm1 = RMSNorm(D, cfg.norm_eps, dtype, device)
        self.attention_norm2 = RMSNorm(D, cfg.norm_eps, dtype, device)
        self.ffn_norm1 = RMSNorm(D, cfg.norm_eps, dtype, device)
        self.ffn_norm2 = RMSNorm(D, cfg.norm_eps, dtype, device)
        if modulation:
            self.adaLN_modulation = nn.ModuleList([Linear(min(D, cfg.adaln_dim), 4 * D, True, dtype, device)])

    def forward(self, x, cos, sin, adaln_input=None, kv_len=None):
        B, S, D = x.shape
        if self.modulation:
            m = self.adaLN_modulation[0](adaln_input)                     # [B, 4D]
            scale_msa, gate_msa, scale_mlp, gate_mlp = [m[:, i * D:(i + 1) * D] for i in range(4)]
            h = self.attention(self.attention_norm1(x, scale=scale_msa), cos, sin, kv_len)
            x = ops.gate_residual(x, self.attention_norm2(h), gate_msa, S, tanh_gate=True)
            h = self.feed_forward(self.ffn_norm1(x, scale=scale_mlp))
            return ops.gate_residual(x, self.ffn_norm2(h), gate_mlp, S, tanh_gate=True)
        h = self.attention(self.attention_norm1(x), cos, sin, kv_len)
        x = ops.gate_residual(x, self.attention_norm2(h))
        h = self.feed_forward(self.ffn_norm1(x))
        return ops.gate_residual(x, self.ffn_norm2(h))


class TimestepEmbedder(nn.Module):
    def __init__(self, out_dim: int, freq_dim: int, mid: int, dtype, device):
        super().__init__()
        self.freq_dim = freq_dim
        self.mlp = nn.ModuleDict({"0": Linear(freq_dim, mid, True, dtype, device),
                                  "2": Linear(mid, out_dim, True, dtype, device)})

    def forward(self, t, t_scale):
        e = timestep_embedding(t, self.freq_dim, time_factor=t_scale).to(self.mlp["0"].weight.dtype)
        return self.mlp["2"](self.mlp["0"](e, act="silu"))


class FinalLayer(nn.Module):
    def __init__(self, cfg: SingleDiTConfig, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.linear = Linear(D, cfg.in_channels, True, dtype, device)
        self.adaLN_modulation = nn.ModuleDict({"1": Linear(min(D, cfg.adaln_dim), D, True, dtype, device)})

    def forward(self, x, c):
        scale = self.adaLN_modulation["1"](ops.activation(c, "silu"))
        return self.linear(ops.norm_modulate(x, scale=scale, eps=1e-6))


class SingleStreamDiT(nn.Module):
    """forward(img [B, S_img, C], cap [B, S_cap, cap_dim], t [B] in [0, 1]) -> velocity [B, S_img, C]."""

    def __init__(self, cfg: SingleDiTConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert cfg.heads * cfg.head_dim == D and sum(cfg.axes_dim) == cfg.head_dim
        self.t_embedder = TimestepEmbedder(min(D, cfg.adaln_dim), 256, 1024 if D > 1024 else D, dtype, device)
        self.cap_embedder = nn.ModuleDict({"0": RMSNorm(cfg.cap_dim, cfg.norm_eps, dtype, device),
                                           "1": Linear(cfg.cap_dim, D, True, dtype, device)})
        self.all_x_embedder = nn.ModuleDict({cfg.patch_key: Linear(cfg.in_channels, D, True, dtype, device)})
        if cfg.final_layer:
            self.all_final_layer = nn.ModuleDict({cfg.patch_key: FinalLayer(cfg, dtype, device)})
        self.x_pad_token = nn.Parameter(torch.zeros(1, D, dtype=dtype, device=device))
        self.cap_pad_token = nn.Parameter(torch.zeros(1, D, dtype=dtype, device=device))
        self.noise_refiner = nn.ModuleList([Block(cfg, True, dtype, device) for _ in range(cfg.depth_noise_refiner)])
        self.context_refiner = nn.ModuleList([Block(cfg, False, dtype, device) for _ in range(cfg.depth_context_refiner)])
        self.layers = nn.ModuleList([Block(cfg, True, dtype, device) for _ in range(cfg.depth)])
        self.gradient_checkpointing = False

    @staticmethod
    def make_ids(h: int, w: int, n_cap: int, device=None) -> torch.Tensor:
        """[n_cap + h*w, 3]: caption token i at (i+1, 0, 0), image token at (n_cap+1, row, col)."""
        ids = torch.zeros(n_cap + h * w, 3, dtype=torch.float32, device=device)
        ids[:n_cap, 0] = torch.arange(1, n_cap + 1, device=device, dtype=torch.float32)
        ids[n_cap:, 0] = float(n_cap + 1)
        ids[n_cap:, 1] = torch.arange(h, device=device, dtype=torch.float32)[:, None].expand(h, w).reshape(-1)
        ids[n_cap:, 2] = torch.arange(w, device=device, dtype=torch.float32)[None, :].expand(h, w).reshape(-1)
        return ids

    def forward(self, img, cap, t, hw: Optional[Tuple[int, int]] = None, cap_len: Optional[torch.Tensor] = None,
                control=None, control_scale: float = 1.0):
        """``control`` = (ZImageControlNet, control tokens [B, S_img, control_in]): the control branch's per-layer hints are
        added after the main layers it names (serenitymojo/models/zimage/controlnet_block.mojo:20-24)."""
        st = self.embed(img, cap, t, hw, cap_len)
        hints = None
        if control is not None:
            net, ctrl = control
            hints = net(self, st, ctrl, control_scale)
        return self.run_layers(st, hints)

    def _run(self, blk, *a):
        if self.gradient_checkpointing and torch.is_grad_enabled():
            return torch.utils.checkpoint.checkpoint(blk, *a, use_reentrant=False, preserve_rng_state=False)
        return blk(*a)

    def embed(self, img, cap, t, hw=None, cap_len=None) -> dict:
        """Everything before the main layers: embeddings, both refiners and the unified (image-first) sequence."""
        cfg = self.cfg
        B, S_img, _ = img.shape
        S_cap = cap.shape[1]
        if hw is None:
            side = int(round(S_img ** 0.5))
            hw = (side, S_img // side)
        dt = self.all_x_embedder[cfg.patch_key].weight.dtype
        ids = self.make_ids(hw[0], hw[1], S_cap, img.device)
        cos, sin = ops.rope_table(ids, cfg.axes_dim, cfg.theta)
        c = self.t_embedder(t, cfg.t_scale)                                   # [B, adaln_dim]
        x = self.all_x_embedder[cfg.patch_key](img.to(dt))
        y = self.cap_embedder["1"](self.cap_embedder["0"](cap.to(dt)))
        if cap_len is not None:                                             # padded captions -> learned pad token
            pad = torch.arange(S_cap, device=img.device)[None, :] >= cap_len[:, None]
            y = torch.where(pad[..., None], self.cap_pad_token.to(y.dtype)[None], y)
        for blk in self.context_refiner:
            y = self._run(blk, y, cos[:S_cap], sin[:S_cap])
        for blk in self.noise_refiner:
            x = self._run(blk, x, cos[S_cap:], sin[S_cap:], c)
        # image tokens first so a caption padding mask is a pure key-length mask
        h = torch.cat((x, y), dim=1)
        cos_j = torch.cat((cos[S_cap:], cos[:S_cap]), 0).contiguous()
        sin_j = torch.cat((sin[S_cap:], sin[:S_cap]), 0).contiguous()
        kv_len = (S_img + cap_len).to(torch.int32) if cap_len is not None else None
        return dict(h=h, cap=y, c=c, cos=cos_j, sin=sin_j, cos_img=cos[S_cap:], sin_img=sin[S_cap:], kv_len=kv_len, S_img=S_img, dt=dt)

    def run_layers(self, st: dict, hints=None):
        h = st["h"]
        for i, blk in enumerate(self.layers):
            h = self._run(blk, h, st["cos"], st["sin"], st["c"], st["kv_len"])
            if hints is not None and i in hints:
                h = h + hints[i]
        h = h[:, :st["S_img"]]
        return self.all_final_layer[self.cfg.patch_key](h, st["c"]) if self.cfg.final_layer else h

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
