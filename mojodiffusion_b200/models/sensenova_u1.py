"""SenseNova-U1-8B text-to-image: one 42-layer Qwen3-style decoder (width 4096, 32 query / 8 key-value heads of 128, SwiGLU
12 288 wide) carrying TWO dense weight sets per layer. The prompt runs once, causally, through the base set and leaves a
per-layer key / value cache; every sampling step runs the image tokens through the ``_mot_gen`` set with full attention over
[cached prompt keys, image keys]. The cache is never updated. The model works on RGB pixels: there is no VAE and no separate
text encoder.

* rotary embedding with three axes inside the 128-wide head: columns [0, 64) time (theta 5e6), [64, 96) row and [96, 128)
  column (theta 1e4), each half-split on its own; q and k are RMS-normalised per head in two halves (``q_norm`` on the 64
  time columns, ``q_norm_hw`` on the other 64) before rotation. Prompt tokens sit at (position, 0, 0), so only their time
  part rotates; image tokens sit at (prompt length, row, column);
* image tokens: 16 x 16 pixel patches (channel-first 768 values) -> Linear -> GELU (tanh form) -> a 2-D interleaved-pair rotation (first
  512 features by the patch column, last 512 by the patch row, theta 1e4) -> 2 x 2 spatial merge (feature-major, 4096 values)
  -> Linear to the model width, plus the sum of two sinusoid MLP embeddings: of the time t and of the normalised noise scale;
* head: final ``norm_mot_gen`` -> Linear -> GELU -> Linear giving the 32 x 32 x 3 CLEAN patch in (row, column, channel)
  order; the velocity is ``(x_pred - z) / max(1 - t, 0.05)``;
* noise scale ``min(sqrt(tokens / 64) * 1, 8)`` multiplies the start noise; times follow ``1 - shift * s / (1 + (shift - 1) s)``
  with s = 1 - i / steps; guidance ``v_u + scale * (v_c - v_u)``; Euler ``z += (t_next - t) * v``; image = z / 2 + 1 / 2.

Behaviour: serenitymojo/models/dit/sensenova_u1.mojo:8-48 (design), :81-121 (configuration), :589-640 (tables), :752-843 (prompt
layer), :908-1022 (image layer and rotation), :1108-1237 (patch features, embeddings, head, noise scale);
serenitymojo/pipeline/sensenova_u1_gen_real.mojo:84-150 (patch orders, time table), :189-256 (sampling loop).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, timestep_embedding


@dataclass
class SenseNovaU1Config:
    vocab_size: int = 151936
    hidden_size: int = 4096
    num_layers: int = 42
    intermediate_size: int = 12288
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 5.0e6
    rope_theta_hw: float = 1.0e4
    rope_theta_vision: float = 1.0e4
    patch_size: int = 16
    vision_hidden_size: int = 1024
    merge_size: int = 2
    noise_scale_base_seq: int = 64
    noise_scale_max: float = 8.0
    noise_scale: float = 1.0
    t_eps: float = 0.05
    name: str = "sensenova-u1-8b"

    @property
    def fm_head_out_dim(self) -> int:
        return 3 * (self.patch_size * self.merge_size) ** 2


def tiny_sensenova_u1_config() -> SenseNovaU1Config:
    return SenseNovaU1Config(vocab_size=64, hidden_size=128, num_layers=2, intermediate_size=256, num_heads=4, num_kv_heads=2,
                             head_dim=32, patch_size=4, vision_hidden_size=32, name="tiny-sensenova-u1")


def _axis_table(pos: torch.Tensor, dim: int, theta: float):
    """cos / sin [S, dim / 2] for one axis: inverse frequency theta ** (-2 i / dim)."""
    inv = torch.exp(-math.log(theta) * torch.arange(0, dim, 2, dtype=torch.float32, device=pos.device) / dim)
    ang = pos.float()[:, None] * inv[None]
    return ang.cos(), ang.sin()


def _half_split(x, cos, sin):
    """[B, S, H, d] rotated by tables [S, d / 2]."""
    a, b = x.chunk(2, -1)
    c, s = cos[None, :, None].to(x.dtype), sin[None, :, None].to(x.dtype)
    return torch.cat((a * c - b * s, b * c + a * s), -1)


def _pairs(x, cos, sin):
    """[rows, d] rotated in interleaved pairs by tables [rows, d / 2]."""
    a, b = x[..., 0::2], x[..., 1::2]
    c, s = cos.to(x.dtype), sin.to(x.dtype)
    return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)


def patchify(img: torch.Tensor, p: int, channel_first: bool) -> torch.Tensor:
    """[B, 3, H, W] -> [B, (H / p)(W / p), 3 p p]; value order (channel, row, column) or (row, column, channel)."""
    B, Cn, H, W = img.shape
    x = img.reshape(B, Cn, H // p, p, W // p, p)
    x = x.permute(0, 2, 4, 1, 3, 5) if channel_first else x.permute(0, 2, 4, 3, 5, 1)
    return x.reshape(B, (H // p) * (W // p), Cn * p * p)


def unpatchify(x: torch.Tensor, p: int, H: int, W: int) -> torch.Tensor:
    B = x.shape[0]
    return x.reshape(B, H // p, W // p, p, p, 3).permute(0, 5, 1, 3, 2, 4).reshape(B, 3, H, W)


def time_schedule(steps: int, shift: float) -> List[float]:
    out = []
    for i in range(steps + 1):
        s = 1.0 - i / steps
        out.append(1.0 - shift * s / (1.0 + (shift - 1.0) * s))
    return out


class _Attn(nn.Module):
    def __init__(self, c: SenseNovaU1Config, dtype, device):
        super().__init__()
        D, H, KV, Dh = c.hidden_size, c.num_heads, c.num_kv_heads, c.head_dim
        for sfx in ("", "_mot_gen"):
            setattr(self, "q_proj" + sfx, Linear(D, H * Dh, False, dtype, device))
            setattr(self, "k_proj" + sfx, Linear(D, KV * Dh, False, dtype, device))
            setattr(self, "v_proj" + sfx, Linear(D, KV * Dh, False, dtype, device))
            setattr(self, "o_proj" + sfx, Linear(H * Dh, D, False, dtype, device))
            for n in ("q_norm", "k_norm", "q_norm_hw", "k_norm_hw"):
                setattr(self, n + sfx, RMSNorm(Dh // 2, c.rms_norm_eps, dtype, device))


class _Mlp(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.gate_proj = Linear(c.hidden_size, c.intermediate_size, False, dtype, device)
        self.up_proj = Linear(c.hidden_size, c.intermediate_size, False, dtype, device)
        self.down_proj = Linear(c.intermediate_size, c.hidden_size, False, dtype, device)

    def forward(self, x):
        return self.down_proj(self.gate_proj(x, act="silu") * self.up_proj(x))


class SenseNovaLayer(nn.Module):
    def __init__(self, c: SenseNovaU1Config, dtype, device):
        super().__init__()
        self.c = c
        self.self_attn = _Attn(c, dtype, device)
        self.mlp, self.mlp_mot_gen = _Mlp(c, dtype, device), _Mlp(c, dtype, device)
        for n in ("input_layernorm", "post_attention_layernorm", "input_layernorm_mot_gen", "post_attention_layernorm_mot_gen"):
            setattr(self, n, RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device))

    def _qk(self, x, which: str, sfx: str, tables):
        """Two-half QK norm + rotation of [B, S, heads, Dh]; ``tables`` = (t, h, w) cos / sin pairs (h, w None: not rotated)."""
        a = self.self_attn
        Dh = self.c.head_dim
        xt = getattr(a, f"{which}_norm{sfx}")(x[..., :Dh // 2])
        xhw = getattr(a, f"{which}_norm_hw{sfx}")(x[..., Dh // 2:])
        xt = _half_split(xt, *tables[0])
        if tables[1] is not None:
            xhw = torch.cat((_half_split(xhw[..., :Dh // 4], *tables[1]), _half_split(xhw[..., Dh // 4:], *tables[2])), -1)
        return torch.cat((xt, xhw), -1)

    def forward(self, x, tables, gen: bool, past: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        """Prompt pass (``gen`` False): causal, returns (x, (k, v)) with k / v [B, S, kv heads, Dh] after norm + rotation.
        Image pass: full attention over [past, own] keys, returns (x, None)."""
        c, a = self.c, self.self_attn
        sfx = "_mot_gen" if gen else ""
        B, S, _ = x.shape
        H, KV, Dh = c.num_heads, c.num_kv_heads, c.head_dim
        h = getattr(self, "input_layernorm" + sfx)(x)
        q = self._qk(getattr(a, "q_proj" + sfx)(h).unflatten(-1, (H, Dh)), "q", sfx, tables)
        k = self._qk(getattr(a, "k_proj" + sfx)(h).unflatten(-1, (KV, Dh)), "k", sfx, tables)
        v = getattr(a, "v_proj" + sfx)(h).unflatten(-1, (KV, Dh))
        kv = None if gen else (k, v)
        if past is not None:
            k, v = torch.cat((past[0], k), 1), torch.cat((past[1], v), 1)
        rep = H // KV
        kk, vv = k.repeat_interleave(rep, 2), v.repeat_interleave(rep, 2)
        if gen:
            o = ops.attention(q, kk, vv)
        else:
            o = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True).transpose(1, 2)
        x = x + getattr(a, "o_proj" + sfx)(o.reshape(B, S, H * Dh))
        mlp = self.mlp_mot_gen if gen else self.mlp
        return x + mlp(getattr(self, "post_attention_layernorm" + sfx)(x)), kv


class _Spine(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([SenseNovaLayer(c, dtype, device) for _ in range(c.num_layers)])
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.norm_mot_gen = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)


class _LM(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.model = _Spine(c, dtype, device)


def _mlp2(i, mid, o, dtype, device):
    m = nn.Module()
    m.mlp = nn.ModuleDict({"0": Linear(i, mid, True, dtype, device), "2": Linear(mid, o, True, dtype, device)})
    return m


class _VisionEmbeddings(nn.Module):
    def __init__(self, c: SenseNovaU1Config, dtype, device):
        super().__init__()
        p, vh, mg = c.patch_size, c.vision_hidden_size, c.merge_size
        pe, de = nn.Module(), nn.Module()
        pe.weight = nn.Parameter(torch.zeros(vh, 3, p, p, dtype=dtype, device=device))
        pe.bias = nn.Parameter(torch.zeros(vh, dtype=dtype, device=device))
        de.weight = nn.Parameter(torch.zeros(c.hidden_size, vh, mg, mg, dtype=dtype, device=device))
        de.bias = nn.Parameter(torch.zeros(c.hidden_size, dtype=dtype, device=device))
        self.patch_embedding, self.dense_embedding = pe, de


class _FmModules(nn.Module):
    def __init__(self, c: SenseNovaU1Config, dtype, device):
        super().__init__()
        D = c.hidden_size
        vm = nn.Module()
        vm.embeddings = _VisionEmbeddings(c, dtype, device)
        self.vision_model_mot_gen = vm
        self.timestep_embedder = _mlp2(256, D, D, dtype, device)
        self.noise_scale_embedder = _mlp2(256, D, D, dtype, device)
        self.fm_head = nn.ModuleDict({"0": Linear(D, D, True, dtype, device), "2": Linear(D, c.fm_head_out_dim, True, dtype, device)})


class SenseNovaU1(nn.Module):
    def __init__(self, cfg: SenseNovaU1Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.language_model = _LM(cfg, dtype, device)
        self.fm_modules = _FmModules(cfg, dtype, device)

    # ---- prompt pass -----------------------------------------------------------------------------------------------
    @torch.no_grad()
    def forward_und(self, token_ids: Sequence[int]):
        """-> list over layers of (k, v) [1, S, kv heads, Dh]; the image tokens' time index is ``len(token_ids)``."""
        c, m = self.cfg, self.language_model.model
        dev = m.embed_tokens.weight.device
        x = m.embed_tokens(torch.tensor(list(token_ids), dtype=torch.long, device=dev))[None]
        tables = (_axis_table(torch.arange(len(token_ids), device=dev), c.head_dim // 2, c.rope_theta), None, None)
        cache = []
        for layer in m.layers:
            x, kv = layer(x, tables, False)
            cache.append(kv)
        return cache

    # ---- image pass ------------------------------------------------------------------------------------------------
    def noise_scale(self, grid_h: int, grid_w: int) -> float:
        c = self.cfg
        return min(math.sqrt(grid_h * grid_w / c.merge_size ** 2 / c.noise_scale_base_seq) * c.noise_scale, c.noise_scale_max)

    def image_features(self, pixel_patches: torch.Tensor, grid_h: int, grid_w: int) -> torch.Tensor:
        """[B, grid_h * grid_w, 3 p p] channel-first patches -> [B, tokens, hidden]."""
        c, e = self.cfg, self.fm_modules.vision_model_mot_gen.embeddings
        B, N, _ = pixel_patches.shape
        vh, mg = c.vision_hidden_size, c.merge_size
        dt = e.patch_embedding.weight.dtype
        x = ops.linear(pixel_patches.to(dt), e.patch_embedding.weight.flatten(1), e.patch_embedding.bias, "gelu_tanh")
        idx = torch.arange(N, device=x.device)
        cx, sx = _axis_table(idx % grid_w, vh // 2, c.rope_theta_vision)
        cy, sy = _axis_table(idx // grid_w, vh // 2, c.rope_theta_vision)
        x = torch.cat((_pairs(x[..., :vh // 2], cx[None], sx[None]), _pairs(x[..., vh // 2:], cy[None], sy[None])), -1)
        th, tw = grid_h // mg, grid_w // mg
        x = x.reshape(B, th, mg, tw, mg, vh).permute(0, 1, 3, 5, 2, 4).reshape(B, th * tw, vh * mg * mg)
        return ops.linear(x, e.dense_embedding.weight.flatten(1), e.dense_embedding.bias)

    def scalar_embed(self, value: float, which: str, device) -> torch.Tensor:
        emb = self.fm_modules.timestep_embedder if which == "timestep" else self.fm_modules.noise_scale_embedder
        dt = emb.mlp["0"].weight.dtype
        t = torch.tensor([float(value)], dtype=torch.float32, device=device)
        return emb.mlp["2"](emb.mlp["0"](timestep_embedding(t, 256, time_factor=1.0).to(dt), act="silu"))

    @torch.no_grad()
    def forward_gen(self, image_embeds: torch.Tensor, text_len: int, token_h: int, token_w: int, cache) -> torch.Tensor:
        c, m = self.cfg, self.language_model.model
        dev = image_embeds.device
        L = token_h * token_w
        i = torch.arange(L, device=dev)
        tables = (_axis_table(torch.full((L,), text_len, device=dev), c.head_dim // 2, c.rope_theta),
                  _axis_table(i // token_w, c.head_dim // 4, c.rope_theta_hw), _axis_table(i % token_w, c.head_dim // 4, c.rope_theta_hw))
        x = image_embeds
        for layer, past in zip(m.layers, cache):
            x, _ = layer(x, tables, True, past)
        return m.norm_mot_gen(x)

    def fm_head(self, hidden: torch.Tensor) -> torch.Tensor:
        h = self.fm_modules.fm_head
        return h["2"](h["0"](hidden, act="gelu_tanh"))

    @torch.no_grad()
    def predict_clean(self, img: torch.Tensor, t: float, cache, text_len: int) -> torch.Tensor:
        """img [1, 3, H, W] at time t -> predicted clean patches [1, tokens, 3 * (p * merge)^2] in (row, column, channel) order."""
        c = self.cfg
        H, W = img.shape[-2:]
        gh, gw = H // c.patch_size, W // c.patch_size
        emb = self.image_features(patchify(img, c.patch_size, True), gh, gw)
        s_norm = self.noise_scale(gh, gw) / c.noise_scale_max
        emb = emb + (self.scalar_embed(t, "timestep", img.device) + self.scalar_embed(s_norm, "noise", img.device))[:, None]
        return self.fm_head(self.forward_gen(emb, text_len, gh // c.merge_size, gw // c.merge_size, cache))

    @torch.no_grad()
    def sample(self, cond_ids: Sequence[int], uncond_ids: Sequence[int], height: int, width: int, steps: int = 30, cfg_scale: float = 4.0,
               shift: float = 3.0, seed: int = 0, noise: Optional[torch.Tensor] = None) -> torch.Tensor:
        """-> image [1, 3, height, width] in [0, 1] (unclamped)."""
        c = self.cfg
        dev = self.language_model.model.embed_tokens.weight.device
        dt = self.language_model.model.embed_tokens.weight.dtype
        cache_c, cache_u = self.forward_und(cond_ids), self.forward_und(uncond_ids)
        gh, gw = height // c.patch_size, width // c.patch_size
        if noise is None:
            noise = ops.randn((1, 3, height, width), seed, 0, torch.float32, dev)
        img = (noise.float() * self.noise_scale(gh, gw)).to(dt)
        ts = time_schedule(steps, shift)
        pm = c.patch_size * c.merge_size
        for i in range(steps):
            t, t_next = ts[i], ts[i + 1]
            z = patchify(img, pm, False)
            inv = 1.0 / max(1.0 - t, c.t_eps)
            v_c = (self.predict_clean(img, t, cache_c, len(cond_ids)) - z) * inv
            v_u = (self.predict_clean(img, t, cache_u, len(uncond_ids)) - z) * inv
            img = unpatchify(z + (t_next - t) * (v_u + cfg_scale * (v_c - v_u)), pm, height, width)
        return img * 0.5 + 0.5

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
