"""Qwen3 decoder stack used as a text encoder: RMSNorm, grouped-query causal attention with per-head QK-RMSNorm and
half-split RoPE, SwiGLU MLP; ``forward`` returns the hidden states of a chosen layer (diffusion models condition on a late
layer, not on logits). Parameter names are those of ``Qwen3Model`` checkpoints
(serenitymojo/models/text_encoder/qwen3_encoder.mojo)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
from torch import nn

from ... import ops


@dataclass
class Qwen3Config:
    vocab_size: int = 151936
    hidden_size: int = 2560
    intermediate_size: int = 9728
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: int = 128
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1_000_000.0


class _W(nn.Module):
    def __init__(self, i, o, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype, device=device).normal_(0, 0.02))

    def forward(self, x):
        return ops.linear(x, self.weight)


class _Norm(nn.Module):
    def __init__(self, d, eps, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        v = x.float().pow(2).mean(-1, keepdim=True)
        return (x.float() * torch.rsqrt(v + self.eps)).to(x.dtype) * self.weight


def _rope(x, cos, sin):
    d = x.shape[-1] // 2
    rot = torch.cat((-x[..., d:], x[..., :d]), dim=-1)
    return x * cos + rot * sin


class _Attn(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.c = c
        self.q_proj = _W(c.hidden_size, c.num_attention_heads * c.head_dim, dtype, device)
        self.k_proj = _W(c.hidden_size, c.num_key_value_heads * c.head_dim, dtype, device)
        self.v_proj = _W(c.hidden_size, c.num_key_value_heads * c.head_dim, dtype, device)
        self.o_proj = _W(c.num_attention_heads * c.head_dim, c.hidden_size, dtype, device)
        self.q_norm, self.k_norm = _Norm(c.head_dim, c.rms_norm_eps, dtype, device), _Norm(c.head_dim, c.rms_norm_eps, dtype, device)

    def forward(self, x, cos, sin, mask):
        B, S, _ = x.shape
        c = self.c
        q = self.q_norm(self.q_proj(x).view(B, S, c.num_attention_heads, c.head_dim)).transpose(1, 2)
        k = self.k_norm(self.k_proj(x).view(B, S, c.num_key_value_heads, c.head_dim)).transpose(1, 2)
        v = self.v_proj(x).view(B, S, c.num_key_value_heads, c.head_dim).transpose(1, 2)
        q, k = _rope(q, cos, sin), _rope(k, cos, sin)
        rep = c.num_attention_heads // c.num_key_value_heads
        k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
        o = torch.nn.functional.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        return self.o_proj(o.transpose(1, 2).reshape(B, S, -1))


class _MLP(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.gate_proj, self.up_proj = _W(c.hidden_size, c.intermediate_size, dtype, device), _W(c.hidden_size, c.intermediate_size, dtype, device)
        self.down_proj = _W(c.intermediate_size, c.hidden_size, dtype, device)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


class _Layer(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.self_attn, self.mlp = _Attn(c, dtype, device), _MLP(c, dtype, device)
        self.input_layernorm = _Norm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.post_attention_layernorm = _Norm(c.hidden_size, c.rms_norm_eps, dtype, device)


class _Model(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([_Layer(c, dtype, device) for _ in range(c.num_hidden_layers)])
        self.norm = _Norm(c.hidden_size, c.rms_norm_eps, dtype, device)


class Qwen3Encoder(nn.Module):
    def __init__(self, cfg: Qwen3Config, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        self.model = _Model(cfg, dtype, device)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None, layer: int = -1, final_norm: bool = True):
        """ids [B, S], mask [B, S] (1 = token). ``layer``: index of the hidden state to return (-1 = last; -2 is what the
        image models condition on, taken before the final norm with ``final_norm=False``)."""
        c = self.cfg
        B, S = ids.shape
        x = self.model.embed_tokens(ids)
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=ids.device).float() / c.head_dim))
        ang = torch.arange(S, device=ids.device).float()[:, None] * inv[None]
        emb = torch.cat((ang, ang), dim=-1)
        cos, sin = emb.cos().to(x.dtype)[None, None], emb.sin().to(x.dtype)[None, None]
        m = torch.full((S, S), float("-inf"), device=ids.device, dtype=x.dtype).triu(1)[None, None]
        if mask is not None:
            m = m + (1.0 - mask[:, None, None, :].to(x.dtype)) * torch.finfo(x.dtype).min
        n = len(self.model.layers)
        stop = n if layer == -1 else (n + 1 + layer if layer < 0 else layer)
        for l in self.model.layers[:stop]:
            x = x + l.self_attn(l.input_layernorm(x), cos, sin, m)
            x = x + l.mlp(l.post_attention_layernorm(x))
        return self.model.norm(x) if final_norm else x
