"""GPT-OSS decoder as a frozen text encoder (Lens conditions on the hidden states after layers 5, 11, 17 and 23 of the 24-layer
20 B model): width 2880, 64 query / 8 key-value heads of 64, biased q / k / v / o projections, a learned per-head "sink" logit
appended to every softmax row (its probability mass is dropped), sliding-window causal attention (128) on even layers and full
causal attention on odd ones, YaRN-scaled half-split rotary embedding (base 150 000, factor 32, cos / sin multiplied by
``0.1 ln(factor) + 1``), and a 32-expert top-4 mixture in place of the feed-forward:

    router logits -> top-4 -> softmax over the four -> per expert ``gate_up = x W + b`` with INTERLEAVED columns (even: gate,
    odd: up), ``gate = min(gate, 7)``, ``up = clamp(up, -7, 7)``, ``(up + 1) * gate * sigmoid(1.702 gate)``, ``W_down`` + bias,
    weighted sum over the chosen experts.

Expert matrices are stored [experts, in, out]. The checkpoint keeps them as MXFP4 (``*_blocks`` uint8 with two e2m1 values per
byte, low nibble first, and ``*_scales`` e8m0 per 32 values): ``dequant_mxfp4`` and ``remap_gpt_oss_keys`` turn them into dense
tensors. Behaviour: serenitymojo/models/text_encoder/gpt_oss_encoder.mojo:14-44 (layer, mixture, configuration), :66-70 (e2m1
table); parameter names are those of ``transformers``' GptOssModel, which the test uses as the oracle.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops

LENS_CAPTURE_LAYERS = (5, 11, 17, 23)
_FP4 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


@dataclass
class GptOssConfig:
    vocab_size: int = 201088
    hidden_size: int = 2880
    num_hidden_layers: int = 24
    num_attention_heads: int = 64
    num_key_value_heads: int = 8
    head_dim: int = 64
    intermediate_size: int = 2880
    num_local_experts: int = 32
    num_experts_per_tok: int = 4
    sliding_window: int = 128
    rms_norm_eps: float = 1e-5
    rope_theta: float = 150000.0
    rope_factor: float = 32.0
    rope_beta_fast: float = 32.0
    rope_beta_slow: float = 1.0
    rope_original_max_pos: int = 4096
    swiglu_limit: float = 7.0
    swiglu_alpha: float = 1.702


def yarn_inv_freq(c: GptOssConfig):
    """(inverse frequencies [head_dim / 2] fp32, cos / sin multiplier)."""
    dim, base = c.head_dim, c.rope_theta
    pos_freqs = base ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim)
    corr = lambda rot: dim * math.log(c.rope_original_max_pos / (rot * 2 * math.pi)) / (2 * math.log(base))
    low, high = max(corr(c.rope_beta_fast), 0.0), min(corr(c.rope_beta_slow), dim - 1.0)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(dim // 2, dtype=torch.float64) - low) / (high - low)).clamp(0, 1)
    extrap = 1.0 - ramp
    inv = (1.0 / (c.rope_factor * pos_freqs)) * (1 - extrap) + (1.0 / pos_freqs) * extrap
    return inv.float(), 0.1 * math.log(c.rope_factor) + 1.0


class _Lin(nn.Module):
    def __init__(self, i, o, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype, device=device).normal_(0, 0.02))
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype, device=device))

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class _Norm(nn.Module):
    def __init__(self, d, eps, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.eps = eps

    def forward(self, x):
        v = x.float().pow(2).mean(-1, keepdim=True)
        return (self.weight * (x.float() * torch.rsqrt(v + self.eps))).to(x.dtype)


class _Attn(nn.Module):
    def __init__(self, c: GptOssConfig, layer: int, dtype, device):
        super().__init__()
        self.c = c
        self.window = c.sliding_window if layer % 2 == 0 else 0
        H, KV, Dh, D = c.num_attention_heads, c.num_key_value_heads, c.head_dim, c.hidden_size
        self.q_proj, self.k_proj, self.v_proj = _Lin(D, H * Dh, dtype, device), _Lin(D, KV * Dh, dtype, device), _Lin(D, KV * Dh, dtype, device)
        self.o_proj = _Lin(H * Dh, D, dtype, device)
        self.sinks = nn.Parameter(torch.zeros(H, dtype=dtype, device=device))

    def forward(self, x, cos, sin, key_mask):
        c = self.c
        B, S, _ = x.shape
        H, KV, Dh = c.num_attention_heads, c.num_key_value_heads, c.head_dim
        q = self.q_proj(x).view(B, S, H, Dh).transpose(1, 2)
        k = self.k_proj(x).view(B, S, KV, Dh).transpose(1, 2)
        v = self.v_proj(x).view(B, S, KV, Dh).transpose(1, 2)

        def rot(t):
            a, b = t.chunk(2, -1)
            return torch.cat((a * cos - b * sin, b * cos + a * sin), -1)

        q, k = rot(q), rot(k)
        rep = H // KV
        k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        i = torch.arange(S, device=x.device)
        allow = i[None, :] <= i[:, None]
        if self.window:
            allow = allow & (i[:, None] - i[None, :] < self.window)
        allow = allow[None, None]
        if key_mask is not None:
            allow = allow & key_mask[:, None, None, :].bool()
        logits = (q.float() @ k.float().transpose(-1, -2)) * (Dh ** -0.5)
        logits = logits.masked_fill(~allow, torch.finfo(torch.float32).min)
        logits = torch.cat((logits, self.sinks.float().reshape(1, H, 1, 1).expand(B, H, S, 1)), -1)
        probs = torch.softmax(logits, -1)[..., :-1].to(v.dtype)
        return self.o_proj((probs @ v).transpose(1, 2).reshape(B, S, H * Dh))


class _Router(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(c.num_local_experts, c.hidden_size, dtype=dtype, device=device).normal_(0, 0.02))
        self.bias = nn.Parameter(torch.zeros(c.num_local_experts, dtype=dtype, device=device))


class _Experts(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        E, D, I = c.num_local_experts, c.hidden_size, c.intermediate_size
        self.gate_up_proj = nn.Parameter(torch.empty(E, D, 2 * I, dtype=dtype, device=device).normal_(0, 0.02))
        self.gate_up_proj_bias = nn.Parameter(torch.zeros(E, 2 * I, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(E, I, D, dtype=dtype, device=device).normal_(0, 0.02))
        self.down_proj_bias = nn.Parameter(torch.zeros(E, D, dtype=dtype, device=device))


class _Moe(nn.Module):
    def __init__(self, c: GptOssConfig, dtype, device):
        super().__init__()
        self.c = c
        self.router, self.experts = _Router(c, dtype, device), _Experts(c, dtype, device)

    def forward(self, x):
        c, e = self.c, self.experts
        shape = x.shape
        t = x.reshape(-1, shape[-1])
        logits = F.linear(t, self.router.weight, self.router.bias)
        top, idx = torch.topk(logits, c.num_experts_per_tok, -1)
        w = torch.softmax(top, -1, dtype=top.dtype)
        out = torch.zeros_like(t)
        for ex in idx.unique().tolist():
            tok, slot = torch.where(idx == ex)
            gu = t[tok] @ e.gate_up_proj[ex] + e.gate_up_proj_bias[ex]
            gate, up = gu[..., 0::2].clamp(max=c.swiglu_limit), gu[..., 1::2].clamp(-c.swiglu_limit, c.swiglu_limit)
            y = ((up + 1) * gate * torch.sigmoid(gate * c.swiglu_alpha)) @ e.down_proj[ex] + e.down_proj_bias[ex]
            out.index_add_(0, tok, (y * w[tok, slot, None]).to(out.dtype))
        return out.reshape(shape)


class _Layer(nn.Module):
    def __init__(self, c, i, dtype, device):
        super().__init__()
        self.self_attn, self.mlp = _Attn(c, i, dtype, device), _Moe(c, dtype, device)
        self.input_layernorm = _Norm(c.hidden_size, c.rms_norm_eps, dtype, device)
        self.post_attention_layernorm = _Norm(c.hidden_size, c.rms_norm_eps, dtype, device)


class GptOssEncoder(nn.Module):
    def __init__(self, cfg: GptOssConfig, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([_Layer(cfg, i, dtype, device) for i in range(cfg.num_hidden_layers)])
        self.norm = _Norm(cfg.hidden_size, cfg.rms_norm_eps, dtype, device)

    @torch.no_grad()
    def layer_states(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None) -> List[torch.Tensor]:
        """Output of every layer (before the final norm); ``mask`` [B, S] marks real tokens."""
        c = self.cfg
        x = self.embed_tokens(ids)
        inv, mult = yarn_inv_freq(c)
        ang = torch.arange(ids.shape[1], device=ids.device).float()[:, None] * inv.to(ids.device)[None]
        cos, sin = (ang.cos() * mult).to(x.dtype)[None, None], (ang.sin() * mult).to(x.dtype)[None, None]
        out = []
        for l in self.layers:
            x = x + l.self_attn(l.input_layernorm(x), cos, sin, mask)
            x = x + l.mlp(l.post_attention_layernorm(x))
            out.append(x)
        return out

    def forward(self, ids, mask=None):
        return self.norm(self.layer_states(ids, mask)[-1])

    def lens_features(self, ids, mask=None, layers: Sequence[int] = LENS_CAPTURE_LAYERS) -> torch.Tensor:
        """[B, S, len(layers), hidden]: the captured layer outputs side by side (the Lens DiT normalises each one itself)."""
        st = self.layer_states(ids, mask)
        return torch.stack([st[i] for i in layers], 2)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """blocks [..., G, 16] uint8 (two e2m1 values per byte, low nibble first), scales [..., G] uint8 (e8m0, bias 127) ->
    [..., G * 32]."""
    lut = torch.tensor(_FP4, dtype=torch.float32, device=blocks.device)
    lo, hi = lut[(blocks & 0x0F).long()], lut[(blocks >> 4).long()]
    vals = torch.stack((lo, hi), -1).flatten(-2)                                        # [..., G, 32]
    vals = torch.ldexp(vals, (scales.to(torch.int32) - 127)[..., None])
    return vals.flatten(-2).to(dtype)


def remap_gpt_oss_keys(sd: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """``model.X`` -> ``X``; ``experts.<name>_blocks`` + ``_scales`` ([experts, out, G, 16] / [experts, out, G]) -> dense
    ``experts.<name>`` [experts, in, out]."""
    out = {}
    for k, v in sd.items():
        n = k[len("model."):] if k.startswith("model.") else k
        if n.startswith("lm_head") or n.endswith("_scales"):
            continue
        if n.endswith("_blocks"):
            base = n[:-len("_blocks")]
            out[base] = dequant_mxfp4(v, sd[k[:-len("_blocks")] + "_scales"], dtype).transpose(1, 2).contiguous()
        else:
            out[n] = v
    return out
