"""Wan2.2-shaped video DiT (TI2V-5B: 30 layers, dim 3072, 24 heads x 128, FFN 14336, 48 latent channels, patch (1,2,2),
UMT5 text width 4096).

Block: ``e = modulation + time_projection(silu(time_embedding(t)))`` chunked into (shift, scale, gate) x 2;
``x += gate_sa * self_attn(LN(x) * (1 + scale_sa) + shift_sa)`` where q and k pass an RMSNorm over the full width and a
3-axis interleaved rotary embedding with the head dim split (44, 42, 42) over (frame, row, column);
``x += cross_attn(norm3(x), text)`` (affine LayerNorm, RMS-normed q / k, no rotary, no gate);
``x += gate_ffn * ffn(LN(x) * (1 + scale_ffn) + shift_ffn)`` with a GELU-tanh MLP. The head applies its own
two-row modulation and projects to ``prod(patch) * out_dim`` values per token, channel innermost.

Parameter names are those of ``WanModel`` checkpoints: ``patch_embedding``, ``text_embedding.{0,2}``,
``time_embedding.{0,2}``, ``time_projection.1``, ``blocks.{i}.{self_attn,cross_attn}.{q,k,v,o,norm_q,norm_k}``,
``blocks.{i}.norm3``, ``blocks.{i}.ffn.{0,2}``, ``blocks.{i}.modulation``, ``head.head``, ``head.modulation``.

Facts: serenitymojo/models/dit/wan22_dit.mojo:7-28 (sizes, block order), :82-122 (rotary axes and positions)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops.conv import patchify_3d
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class WanConfig:
    in_dim: int = 48
    out_dim: int = 48
    dim: int = 3072
    heads: int = 24
    ffn_dim: int = 14336
    depth: int = 30
    text_dim: int = 4096
    freq_dim: int = 256
    patch: Tuple[int, int, int] = (1, 2, 2)
    theta: float = 10000.0
    name: str = "wan2.2-ti2v-5b"

    @property
    def head_dim(self) -> int:
        return self.dim // self.heads

    @property
    def axes_dim(self) -> Tuple[int, int, int]:
        d = self.head_dim
        return (d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6))


def wan22_ti2v_5b_config() -> WanConfig:
    return WanConfig()


def tiny_wan_config() -> WanConfig:
    return WanConfig(in_dim=8, out_dim=8, dim=128, heads=2, ffn_dim=256, depth=2, text_dim=96, freq_dim=64, name="tiny-wan")


class LayerNormAffine(nn.Module):
    def __init__(self, dim, eps, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        return ops.norm_modulate(x, weight=self.weight, bias=self.bias, eps=self.eps)


class _Attn(nn.Module):
    def __init__(self, dim, kv_dim, dtype, device):
        super().__init__()
        self.q = Linear(dim, dim, True, dtype, device)
        self.k = Linear(kv_dim, dim, True, dtype, device)
        self.v = Linear(kv_dim, dim, True, dtype, device)
        self.o = Linear(dim, dim, True, dtype, device)
        self.norm_q, self.norm_k = RMSNorm(dim, 1e-6, dtype, device), RMSNorm(dim, 1e-6, dtype, device)


class WanBlock(nn.Module):
    def __init__(self, cfg: WanConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        D = cfg.dim
        self.self_attn = _Attn(D, D, dtype, device)
        self.cross_attn = _Attn(D, D, dtype, device)
        self.norm3 = LayerNormAffine(D, 1e-6, dtype, device)
        self.ffn = nn.ModuleDict({"0": Linear(D, cfg.ffn_dim, True, dtype, device), "2": Linear(cfg.ffn_dim, D, True, dtype, device)})
        self.modulation = nn.Parameter(torch.zeros(1, 6, D, dtype=dtype, device=device))

    def forward(self, x, ctx, e0, cos, sin, ctx_len=None):
        cfg = self.cfg
        B, S, D = x.shape
        H, Dh = cfg.heads, cfg.head_dim
        e = (self.modulation.float() + e0.float()).to(x.dtype)                       # [B, 6, D]
        sa = self.self_attn
        xn = ops.norm_modulate(x, scale=e[:, 1], shift=e[:, 0], eps=1e-6)
        qkv = packed_projection(xn, (sa.q, sa.k, sa.v))
        q, k = sa.norm_q(qkv[..., 0:D]), sa.norm_k(qkv[..., D:2 * D])
        qk = ops.qk_norm_rope(torch.cat((q, k), dim=-1), H, Dh, None, None, cos, sin, interleaved=True, do_norm=False)
        a = ops.attention(qk[..., 0:D].unflatten(-1, (H, Dh)), qk[..., D:2 * D].unflatten(-1, (H, Dh)),
                          qkv[..., 2 * D:3 * D].unflatten(-1, (H, Dh))).reshape(B, S, D)
        x = sa.o(a, residual=x, gate=e[:, 2], rows_per_group=S)
        ca = self.cross_attn
        q = ca.norm_q(ca.q(self.norm3(x))).unflatten(-1, (H, Dh))
        kv = packed_projection(ctx, (ca.k, ca.v))
        k = ca.norm_k(kv[..., 0:D]).unflatten(-1, (H, Dh))
        a = ops.attention(q, k, kv[..., D:2 * D].unflatten(-1, (H, Dh)), kv_len=ctx_len).reshape(B, S, D)
        x = ca.o(a, residual=x)
        h = self.ffn["0"](ops.norm_modulate(x, scale=e[:, 4], shift=e[:, 3], eps=1e-6), act="gelu_tanh")
        return self.ffn["2"](h, residual=x, gate=e[:, 5], rows_per_group=S)


class _Head(nn.Module):
    def __init__(self, cfg: WanConfig, dtype, device):
        super().__init__()
        self.head = Linear(cfg.dim, cfg.out_dim * cfg.patch[0] * cfg.patch[1] * cfg.patch[2], True, dtype, device)
        self.modulation = nn.Parameter(torch.zeros(1, 2, cfg.dim, dtype=dtype, device=device))


class _Patch(nn.Module):
    def __init__(self, cfg: WanConfig, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cfg.dim, cfg.in_dim, *cfg.patch, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cfg.dim, dtype=dtype, device=device))


class WanDiT(nn.Module):
    """forward(latent [B, C, F, H, W], text [B, T, 4096], t [B] in [0, 1]) -> velocity [B, C, F, H, W]."""

    def __init__(self, cfg: WanConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.dim
        assert sum(cfg.axes_dim) == cfg.head_dim
        self.patch_embedding = _Patch(cfg, dtype, device)
        self.text_embedding = nn.ModuleDict({"0": Linear(cfg.text_dim, D, True, dtype, device), "2": Linear(D, D, True, dtype, device)})
        self.time_embedding = nn.ModuleDict({"0": Linear(cfg.freq_dim, D, True, dtype, device), "2": Linear(D, D, True, dtype, device)})
        self.time_projection = nn.ModuleDict({"1": Linear(D, 6 * D, True, dtype, device)})
        self.blocks = nn.ModuleList([WanBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        self.head = _Head(cfg, dtype, device)
        self.gradient_checkpointing = False

    @staticmethod
    def make_ids(f: int, h: int, w: int, device=None) -> torch.Tensor:
        t = torch.arange(f, device=device, dtype=torch.float32)[:, None, None].expand(f, h, w)
        y = torch.arange(h, device=device, dtype=torch.float32)[None, :, None].expand(f, h, w)
        x = torch.arange(w, device=device, dtype=torch.float32)[None, None, :].expand(f, h, w)
        return torch.stack((t, y, x), -1).reshape(-1, 3)

    def _control_hints(self, x, ctx, e0, cos, sin, text_len, control):
        raise NotImplementedError("this model takes no control input")

    def forward(self, z, text, timesteps, text_len: Optional[torch.Tensor] = None, control: Optional[torch.Tensor] = None,
                control_scale: float = 1.0):
        cfg = self.cfg
        B, C, F_, Hh, Ww = z.shape
        pt, ph, pw = cfg.patch
        f, h, w = F_ // pt, Hh // ph, Ww // pw
        D = cfg.dim
        dt = self.patch_embedding.weight.dtype
        tok = patchify_3d(z, pt, ph, pw)
        x = ops.linear(tok.to(dt), self.patch_embedding.weight.flatten(1), self.patch_embedding.bias)
        cos, sin = ops.rope_table(self.make_ids(f, h, w, z.device), cfg.axes_dim, cfg.theta)
        te = self.time_embedding
        e = te["2"](te["0"](timestep_embedding(timesteps, cfg.freq_dim).to(dt), act="silu"))           # [B, D]
        e0 = self.time_projection["1"](ops.activation(e, "silu")).reshape(B, 6, D)
        tx = self.text_embedding
        ctx = tx["2"](tx["0"](text.to(dt), act="gelu_tanh"))
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        hints = self._control_hints(x, ctx, e0, cos, sin, text_len, control) if control is not None else {}
        for i, blk in enumerate(self.blocks):
            if ckpt:
                x = torch.utils.checkpoint.checkpoint(blk, x, ctx, e0, cos, sin, text_len, use_reentrant=False,
                                                      preserve_rng_state=False)
            else:
                x = blk(x, ctx, e0, cos, sin, text_len)
            if i in hints:
                x = x + hints[i] * control_scale
        m = (self.head.modulation.float() + e[:, None].float()).to(x.dtype)                         # [B, 2, D]
        out = self.head.head(ops.norm_modulate(x, scale=m[:, 1], shift=m[:, 0], eps=1e-6))
        # token vector is (pt, ph, pw, channel): channel innermost
        out = out.reshape(B, f, h, w, pt, ph, pw, cfg.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6)
        return out.reshape(B, cfg.out_dim, F_, Hh, Ww)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        init_module_weights(self, seed, std)
        with torch.no_grad():
            g = torch.Generator().manual_seed(seed + 3)
            for n, prm in self.named_parameters():
                if n.endswith("modulation"):
                    prm.copy_((torch.randn(prm.shape, generator=g) * std).to(prm.dtype))
                if n.endswith("norm_q.weight") or n.endswith("norm_k.weight") or n.endswith("norm3.weight"):
                    prm.fill_(1.0)
        return self


# ---- Wan-VACE: ControlNet-style conditioning on the Wan stack ----------------------------------------------------------
@dataclass
class WanVaceConfig(WanConfig):
    vace_in_dim: int = 96          # control latent + mask channels
    vace_blocks: int = 8           # control block i feeds base layer 2 i


def wan21_vace_14b_config() -> WanVaceConfig:
    return WanVaceConfig(in_dim=16, out_dim=16, dim=5120, heads=40, ffn_dim=13824, depth=40, name="wan2.1-vace-14b")


def tiny_wan_vace_config() -> WanVaceConfig:
    return WanVaceConfig(in_dim=8, out_dim=8, dim=128, heads=2, ffn_dim=256, depth=4, text_dim=96, freq_dim=64,
                         vace_in_dim=12, vace_blocks=2, name="tiny-wan-vace")


class _VacePatch(nn.Module):
    def __init__(self, cfg: WanVaceConfig, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cfg.dim, cfg.vace_in_dim, *cfg.patch, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cfg.dim, dtype=dtype, device=device))


class WanVaceBlock(WanBlock):
    """A Wan block of the control branch: block 0 mixes the control embedding into the base tokens through ``before_proj``,
    every block emits its hint through ``after_proj`` (both zero-initialised, so an untrained branch changes nothing)."""

    def __init__(self, cfg: WanVaceConfig, first: bool, dtype, device):
        super().__init__(cfg, dtype, device)
        self.before_proj = Linear(cfg.dim, cfg.dim, True, dtype, device) if first else None
        self.after_proj = Linear(cfg.dim, cfg.dim, True, dtype, device)


class WanVaceDiT(WanDiT):
    """Wan DiT + VACE control branch. ``forward(z, text, t, control=[B, vace_in_dim, F, H, W], control_scale=s)``: the
    control latent gets its own patch embedding, runs through ``vace_blocks`` Wan blocks (the running hidden state is
    carried block to block) and hint i is added, times ``s``, after base layer 2 i
    (serenitymojo/models/dit/wan_vace_dit.mojo:14-33,118-200)."""

    def __init__(self, cfg: WanVaceConfig, dtype=torch.bfloat16, device=None):
        super().__init__(cfg, dtype, device)
        self.vace_patch_embedding = _VacePatch(cfg, dtype, device)
        self.vace_blocks = nn.ModuleList([WanVaceBlock(cfg, i == 0, dtype, device) for i in range(cfg.vace_blocks)])

    def vace_layer(self, i: int) -> int:
        return 2 * i

    def _control_hints(self, x, ctx, e0, cos, sin, text_len, control):
        cfg = self.cfg
        pt, ph, pw = cfg.patch
        tok = patchify_3d(control, pt, ph, pw)
        c = ops.linear(tok.to(x.dtype), self.vace_patch_embedding.weight.flatten(1), self.vace_patch_embedding.bias)
        if c.shape[1] < x.shape[1]:                       # shorter control clip: zero tokens up to the base length
            c = torch.nn.functional.pad(c, (0, 0, 0, x.shape[1] - c.shape[1]))
        hints = {}
        for i, blk in enumerate(self.vace_blocks):
            if blk.before_proj is not None:
                c = (blk.before_proj(c).float() + x.float()).to(x.dtype)
            c = blk(c, ctx, e0, cos, sin, text_len)
            hints[self.vace_layer(i)] = blk.after_proj(c)
        return hints

    def init_weights(self, seed: int = 0, std: float = 0.02):
        super().init_weights(seed, std)
        with torch.no_grad():
            for blk in self.vace_blocks:
                for lin in (blk.before_proj, blk.after_proj):
                    if lin is not None:
                        lin.weight.zero_()
                        lin.bias.zero_()
        return self
