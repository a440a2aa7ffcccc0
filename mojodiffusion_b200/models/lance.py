"""Lance 3B text-to-video spine: a Qwen2-style decoder (36 layers, width 2048, 16 query / 2 key-value heads of 128, SwiGLU
11 008 wide, q / k / v biases, per-head QK-RMSNorm) in which the GENERATED (visual) rows of the sequence run through a
second set of weights (``*_moe_gen``: layer norms, q / k / v / o projections, QK norms, feed-forward, final norm) while the
text rows use the language model's own.

Sequence: [bos, text, eos | start-of-image, latent tokens ..., end-of-image]. Text rows attend causally among themselves;
every row from the start-of-image token on attends to all rows. Latent tokens enter as ``vae2llm(x_t) + time_embedder(t) +
latent_pos_embed[t * 64 * 64 + h * 64 + w]`` and leave through ``llm2vae`` on the generated rows. Rotary positions have
three axes: the prefix counts 0, 1, 2, ... on all axes; latent (t, h, w) sits at prefix + (2 t, h, w); the end token at one
past the largest position. The full-width rotary table assigns head columns [0, 32) to the time axis, [32, 80) to the row
axis and [80, 128) to the column axis, each column d using inverse frequency ``theta ** (-(d mod 64) / 64)``; the rotation is
half-split.

Behaviour: serenitymojo/models/lance/lance_t2v.mojo:49-84 (configuration), :101-115 (shared tensors), :242-265 (mask),
:274-323 (rotary table), :406-514 (layer), :536-634 (forward), :647-702 (sequence and positions). As in the reference, the
generated rows' q and k are normalised by ``q_norm`` / ``k_norm`` first and then AGAIN by ``q_norm_moe_gen`` /
``k_norm_moe_gen`` (``renorm_gen=False`` applies only the generated-row norm).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.nn as nn

from .. import ops
from ..runtime.lance_kv_plan import LanceInput
from .layers import Linear, RMSNorm, init_module_weights, timestep_embedding


@dataclass
class LanceConfig:
    hidden_size: int = 2048
    num_layers: int = 36
    num_heads: int = 16
    num_kv_heads: int = 2
    head_dim: int = 128
    intermediate_size: int = 11008
    rope_theta: float = 1.0e6
    rms_norm_eps: float = 1e-6
    vocab_size: int = 151936
    timestep_dim: int = 256
    patch_latent_dim: int = 48
    max_latent_size: int = 64
    mrope: tuple = (16, 24, 24)
    tokens_per_second: int = 2
    bos_token_id: int = 151644
    eos_token_id: int = 151645
    start_of_image_id: int = 151652
    end_of_image_id: int = 151653
    video_token_id: int = 151656
    max_latent_frames: int = 32
    name: str = "lance-3b-video"


def tiny_lance_config() -> LanceConfig:
    return LanceConfig(hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32, intermediate_size=256, vocab_size=64,
                       timestep_dim=32, patch_latent_dim=12, max_latent_size=4, mrope=(4, 6, 6), bos_token_id=60, eos_token_id=61,
                       start_of_image_id=62, end_of_image_id=63, video_token_id=59, max_latent_frames=3, name="tiny-lance")


def build_lance_input(cfg: LanceConfig, text_ids: Sequence[int], latent_t: int, latent_h: int, latent_w: int) -> LanceInput:
    full = [cfg.bos_token_id, *text_ids, cfg.eos_token_id]
    split = len(full)
    full.append(cfg.start_of_image_id)
    gen_start, gen_len = len(full), latent_t * latent_h * latent_w
    full += [cfg.video_token_id] * gen_len + [cfg.end_of_image_id]
    prefix = split + 1
    t_pos, h_pos, w_pos = list(range(prefix)), list(range(prefix)), list(range(prefix))
    latent_pos, top = [], prefix
    for tt in range(latent_t):
        for hh in range(latent_h):
            for ww in range(latent_w):
                p = (prefix + tt * cfg.tokens_per_second, prefix + hh, prefix + ww)
                t_pos.append(p[0]), h_pos.append(p[1]), w_pos.append(p[2])
                top = max(top, *p)
                latent_pos.append(tt * cfg.max_latent_size * cfg.max_latent_size + hh * cfg.max_latent_size + ww)
    for axis in (t_pos, h_pos, w_pos):
        axis.append(top + 1)
    return LanceInput(tuple(full), tuple(t_pos), tuple(h_pos), tuple(w_pos), split, gen_start, gen_len, tuple(latent_pos))


def lance_rope_table(inp: LanceInput, head_dim: int, theta: float, mrope: Sequence[int], device=None):
    """cos / sin [S, head_dim] fp32 (full width, for the half-split rotation ``x * cos + rotate_half(x) * sin``)."""
    half = head_dim // 2
    inv = torch.exp(-math.log(theta) * torch.arange(half, dtype=torch.float32) / half)
    pos = torch.tensor([inp.t_pos, inp.h_pos, inp.w_pos], dtype=torch.float32)          # [3, S]
    d = torch.arange(head_dim)
    axis = torch.full((head_dim,), 2, dtype=torch.long)
    axis[d < 2 * (mrope[0] + mrope[1])] = 1
    axis[d < 2 * mrope[0]] = 0
    assert 2 * sum(mrope) == head_dim
    ang = pos[axis, :].t() * inv[d % half][None]                                         # [S, head_dim]
    return ang.cos().to(device), ang.sin().to(device)


def lance_mask(seq: int, text_split_len: int, dtype=torch.float32, device=None) -> torch.Tensor:
    """Additive [1, 1, S, S]: text rows causal among text, the rest see everything; -1e4 blocks."""
    i = torch.arange(seq, device=device)
    allow = (i[:, None] >= text_split_len) | ((i[None, :] < text_split_len) & (i[None, :] <= i[:, None]))
    return torch.where(allow, 0.0, -1.0e4).to(dtype)[None, None]


def _rotate(x, cos, sin):
    a, b = x.chunk(2, -1)
    return x * cos[None, :, None].to(x.dtype) + torch.cat((-b, a), -1) * sin[None, :, None].to(x.dtype)


class _Attn(nn.Module):
    def __init__(self, c: LanceConfig, dtype, device):
        super().__init__()
        D, H, KV, Dh = c.hidden_size, c.num_heads, c.num_kv_heads, c.head_dim
        for suffix in ("", "_moe_gen"):
            setattr(self, "q_proj" + suffix, Linear(D, H * Dh, True, dtype, device))
            setattr(self, "k_proj" + suffix, Linear(D, KV * Dh, True, dtype, device))
            setattr(self, "v_proj" + suffix, Linear(D, KV * Dh, True, dtype, device))
            setattr(self, "o_proj" + suffix, Linear(H * Dh, D, False, dtype, device))
            setattr(self, "q_norm" + suffix, RMSNorm(Dh, c.rms_norm_eps, dtype, device))
            setattr(self, "k_norm" + suffix, RMSNorm(Dh, c.rms_norm_eps, dtype, device))


class _Mlp(nn.Module):
    def __init__(self, c: LanceConfig, dtype, device):
        super().__init__()
        self.gate_proj = Linear(c.hidden_size, c.intermediate_size, False, dtype, device)
        self.up_proj = Linear(c.hidden_size, c.intermediate_size, False, dtype, device)
        self.down_proj = Linear(c.intermediate_size, c.hidden_size, False, dtype, device)

    def forward(self, x):
        return self.down_proj(self.gate_proj(x, act="silu") * self.up_proj(x))


class LanceLayer(nn.Module):
    def __init__(self, c: LanceConfig, dtype, device):
        super().__init__()
        self.c = c
        self.self_attn = _Attn(c, dtype, device)
        self.mlp, self.mlp_moe_gen = _Mlp(c, dtype, device), _Mlp(c, dtype, device)
        for n in ("input_layernorm", "input_layernorm_moe_gen", "post_attention_layernorm", "post_attention_layernorm_moe_gen"):
            setattr(self, n, RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device))

    def forward(self, x, g0: int, g1: int, cos, sin, mask, renorm_gen: bool = True):
        """Rows [g0, g1) are the generated ones."""
        c, a = self.c, self.self_attn
        B, S, _ = x.shape
        H, KV, Dh = c.num_heads, c.num_kv_heads, c.head_dim

        def two_way(fn_text, fn_gen, inp):
            return torch.cat((fn_text(inp[:, :g0]), fn_gen(inp[:, g0:g1]), fn_text(inp[:, g1:])), 1)

        h = two_way(self.input_layernorm, self.input_layernorm_moe_gen, x)
        q = two_way(a.q_proj, a.q_proj_moe_gen, h).unflatten(-1, (H, Dh))
        k = two_way(a.k_proj, a.k_proj_moe_gen, h).unflatten(-1, (KV, Dh))
        v = two_way(a.v_proj, a.v_proj_moe_gen, h).unflatten(-1, (KV, Dh))
        if renorm_gen:
            q = two_way(lambda t: t, a.q_norm_moe_gen, a.q_norm(q))
            k = two_way(lambda t: t, a.k_norm_moe_gen, a.k_norm(k))
        else:
            q, k = two_way(a.q_norm, a.q_norm_moe_gen, q), two_way(a.k_norm, a.k_norm_moe_gen, k)
        q, k = _rotate(q, cos, sin), _rotate(k, cos, sin)
        rep = H // KV
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.repeat_interleave(rep, 2).transpose(1, 2),
                                                             v.repeat_interleave(rep, 2).transpose(1, 2), attn_mask=mask)
        o = o.transpose(1, 2).reshape(B, S, H * Dh)
        x = x + two_way(a.o_proj, a.o_proj_moe_gen, o)
        return x + torch.cat((self.mlp(self.post_attention_layernorm(x[:, :g0])),
                              self.mlp_moe_gen(self.post_attention_layernorm_moe_gen(x[:, g0:g1])),
                              self.mlp(self.post_attention_layernorm(x[:, g1:]))), 1)


class _Spine(nn.Module):
    def __init__(self, c: LanceConfig, dtype, device):
        super().__init__()
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([LanceLayer(c, dtype, device) for _ in range(c.num_layers)])
        self.norm = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.norm_moe_gen = RMSNorm(c.hidden_size, c.rms_norm_eps, dtype, device)


class _LM(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.model = _Spine(c, dtype, device)


class _PosEmbed(nn.Module):
    def __init__(self, rows, dim, dtype, device):
        super().__init__()
        self.pos_embed = nn.Parameter(torch.zeros(rows, dim, dtype=dtype, device=device))


class LanceT2V(nn.Module):
    """forward(inp: LanceInput, x_t [gen_len, 48], t [1] in [0, 1] scaled as the caller's schedule gives it) -> velocity
    [gen_len, 48] on the generated rows."""

    def __init__(self, cfg: LanceConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden_size
        self.language_model = _LM(cfg, dtype, device)
        self.vae2llm = Linear(cfg.patch_latent_dim, D, True, dtype, device)
        self.llm2vae = Linear(D, cfg.patch_latent_dim, True, dtype, device)
        te = nn.Module()
        te.mlp = nn.ModuleDict({"0": Linear(cfg.timestep_dim, D, True, dtype, device), "2": Linear(D, D, True, dtype, device)})
        self.time_embedder = te
        self.latent_pos_embed = _PosEmbed(cfg.max_latent_frames * cfg.max_latent_size ** 2, D, dtype, device)

    @torch.no_grad()
    def forward(self, inp: LanceInput, x_t: torch.Tensor, t: torch.Tensor, max_layers: int = 0, renorm_gen: bool = True):
        cfg, m = self.cfg, self.language_model.model
        dev, dt = x_t.device, self.vae2llm.weight.dtype
        S, g0, g1 = len(inp.full_ids), inp.gen_start, inp.gen_start + inp.gen_len
        hidden = m.embed_tokens(torch.tensor(inp.full_ids, dtype=torch.long, device=dev))[None]
        te = self.time_embedder.mlp
        temb = te["2"](te["0"](timestep_embedding(t.reshape(1).to(dev), cfg.timestep_dim, time_factor=1.0).to(dt), act="silu"))
        pos = self.latent_pos_embed.pos_embed[torch.tensor(inp.latent_pos_ids, dtype=torch.long, device=dev)]
        vae = self.vae2llm(x_t.to(dt).reshape(1, inp.gen_len, -1)) + temb[:, None] + pos[None]
        hidden = torch.cat((hidden[:, :g0], vae, hidden[:, g1:]), 1)
        cos, sin = lance_rope_table(inp, cfg.head_dim, cfg.rope_theta, cfg.mrope, dev)
        mask = lance_mask(S, inp.text_split_len, dt, dev)
        n = cfg.num_layers if max_layers <= 0 else min(max_layers, cfg.num_layers)
        for layer in m.layers[:n]:
            hidden = layer(hidden, g0, g1, cos, sin, mask, renorm_gen)
        return self.llm2vae(m.norm_moe_gen(hidden[:, g0:g1]))[0]

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
