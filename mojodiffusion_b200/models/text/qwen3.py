"""Qwen3 decoder stack used as a text encoder: RMSNorm, grouped-query causal attention with per-head QK-RMSNorm and
half-split RoPE, SwiGLU MLP; ``forward`` returns the hidden states of a chosen layer (diffusion models condition on a late
layer, not on logits). Parameter names are those of ``Qwen3Model`` checkpoints
(serenitymojo/models/text_encoder/qwen3_encoder.mojo)."""
from __future__ import annotations

from dataclasses import dataclass
import math
from typing import Optional, Sequence, Tuple

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
    qk_norm: bool = True                       # per-head RMSNorm of q and k (Qwen3); Mistral-family stacks have none
    rope_scaling: Optional[Tuple[float, int, float, float]] = None   # (factor, original positions, beta_fast, beta_slow)
    qkv_bias: bool = False                     # biases on the q / k / v projections (the Qwen2 family)


def qwen25vl_text_config() -> Qwen3Config:
    """Language stack of Qwen2.5-VL-7B, Qwen-Image's text encoder: 28 layers, width 3584, 28 query / 4 key-value heads, biased
    q / k / v projections, no QK norms (serenitymojo/models/text_encoder/qwen25vl_encoder.mojo:10-19)."""
    return Qwen3Config(vocab_size=152064, hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
                       num_key_value_heads=4, head_dim=128, rms_norm_eps=1e-6, rope_theta=1.0e6, qk_norm=False, qkv_bias=True)


def mistral3b_config() -> Qwen3Config:
    """The 26-layer Mistral-3B stack ERNIE-Image conditions on (hidden state after layer 24, 512 tokens padded with id 0;
    serenitymojo/models/text_encoder/mistral3b_encoder.mojo:44-80)."""
    return Qwen3Config(vocab_size=131072, hidden_size=3072, intermediate_size=9216, num_hidden_layers=26, num_attention_heads=32,
                       num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-5, rope_theta=1.0e6, qk_norm=False,
                       rope_scaling=(16.0, 16384, 32.0, 1.0))


MISTRAL3B_EXTRACT_LAYER, MISTRAL3B_MAX_LEN = 24, 512


def scaled_inv_freq(head_dim: int, theta: float, scaling: Optional[Tuple[float, int, float, float]]) -> torch.Tensor:
    """Rotary inverse frequencies [head_dim / 2] (fp32). With ``scaling`` = (factor, original positions, beta_fast, beta_slow):
    wavelengths shorter than ``orig / round(orig beta_slow / 2 pi)`` keep their frequency, those longer than
    ``orig / round(orig beta_fast / 2 pi)`` are divided by ``factor``, the band between is interpolated linearly in
    ``orig / wavelength`` (serenitymojo/models/text_encoder/mistral3b_encoder.mojo:108-150)."""
    base = 1.0 / (float(theta) ** (torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim))
    if scaling is None:
        return base.float()
    factor, orig, beta_fast, beta_slow = scaling
    two_pi = 2.0 * math.pi
    low = max(float(int(orig / (two_pi / beta_fast) + 0.5)), 1.0)
    high = max(float(int(orig / (two_pi / beta_slow) + 0.5)), 1.0)
    wavelength = two_pi / base
    smooth = (orig / wavelength - low) / (high - low) if high != low else torch.zeros_like(base)
    mixed = (1.0 - smooth) * (base / factor) + smooth * base
    out = torch.where(wavelength < orig / high, base, torch.where(wavelength > orig / low, base / factor, mixed))
    return out.float()


def pad_or_trim_ids(ids: Sequence[int], max_len: int, pad_id: int = 0):
    """(ids padded with ``pad_id`` or cut to ``max_len``, number of real tokens)."""
    ids = list(ids)[:max_len]
    return ids + [pad_id] * (max_len - len(ids)), len(ids)


class _W(nn.Module):
    def __init__(self, i, o, dtype, device, bias: bool = False):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype, device=device).normal_(0, 0.02))
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


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
        self.q_proj = _W(c.hidden_size, c.num_attention_heads * c.head_dim, dtype, device, c.qkv_bias)
        self.k_proj = _W(c.hidden_size, c.num_key_value_heads * c.head_dim, dtype, device, c.qkv_bias)
        self.v_proj = _W(c.hidden_size, c.num_key_value_heads * c.head_dim, dtype, device, c.qkv_bias)
        self.o_proj = _W(c.num_attention_heads * c.head_dim, c.hidden_size, dtype, device)
        if c.qk_norm:
            self.q_norm, self.k_norm = _Norm(c.head_dim, c.rms_norm_eps, dtype, device), _Norm(c.head_dim, c.rms_norm_eps, dtype, device)

    def forward(self, x, cos, sin, mask):
        B, S, _ = x.shape
        c = self.c
        q, k = self.q_proj(x).view(B, S, c.num_attention_heads, c.head_dim), self.k_proj(x).view(B, S, c.num_key_value_heads, c.head_dim)
        if c.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k = q.transpose(1, 2), k.transpose(1, 2)
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
        inv = scaled_inv_freq(c.head_dim, c.rope_theta, c.rope_scaling).to(ids.device)
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

    @torch.no_grad()
    def layer_states(self, ids: torch.Tensor, mask: Optional[torch.Tensor] = None):
        """Outputs of every decoder layer (before the final norm): a list of [B, S, hidden]; entry i is what
        ``transformers`` reports as ``hidden_states[i + 1]``."""
        c = self.cfg
        B, S = ids.shape
        x = self.model.embed_tokens(ids)
        inv = scaled_inv_freq(c.head_dim, c.rope_theta, c.rope_scaling).to(ids.device)
        ang = torch.arange(S, device=ids.device).float()[:, None] * inv[None]
        emb = torch.cat((ang, ang), dim=-1)
        cos, sin = emb.cos().to(x.dtype)[None, None], emb.sin().to(x.dtype)[None, None]
        m = torch.full((S, S), float("-inf"), device=ids.device, dtype=x.dtype).triu(1)[None, None]
        if mask is not None:
            m = m + (1.0 - mask[:, None, None, :].to(x.dtype)) * torch.finfo(x.dtype).min
        out = []
        for l in self.model.layers:
            x = x + l.self_attn(l.input_layernorm(x), cos, sin, m)
            x = x + l.mlp(l.post_attention_layernorm(x))
            out.append(x)
        return out


def remap_mistral3b_keys(sd):
    """Keep the language stack of a vision-language checkpoint: ``language_model.model.X`` -> ``model.X``."""
    pre = "language_model.model."
    return {"model." + k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)}


# ---- Qwen3-VL language models used as text encoders (the vision tower is dropped; for text-only input the interleaved
# three-section rotary embedding reduces to the plain one) -----------------------------------------------------------------
KREA2_SELECT_LAYERS = (2, 5, 8, 11, 14, 17, 20, 23, 26, 29, 32, 35)     # indices into transformers' hidden_states
KREA2_PREFIX_DROP = 34                                                   # rows of the system prompt template
IDEOGRAM_TAPS = (0, 3, 6, 9, 12, 15, 18, 21, 24, 27, 30, 33, 35)         # decoder layer outputs (0-based)


def qwen3vl_text_config(size: str = "8b") -> Qwen3Config:
    """Language stack of Qwen3-VL-4B (Krea-2) or -8B (Boogu-Image, Ideogram-4): rotary base 5e6."""
    if size == "4b":
        return Qwen3Config(hidden_size=2560, intermediate_size=9728, rope_theta=5.0e6)
    return Qwen3Config(hidden_size=4096, intermediate_size=12288, rope_theta=5.0e6)


def remap_qwen3vl_text_keys(sd, dtype=torch.bfloat16):
    """``model.language_model.X`` (Boogu, Krea-2) or ``language_model.X`` (Ideogram-4) -> ``model.X``; fp8 projection
    weights with a per-row ``weight_scale`` are dequantised (serenitymojo/models/text_encoder/ideogram_qwen3vl.mojo:20-58,
    boogu_qwen3vl.mojo:5-12, krea2_qwen3vl_4b.mojo:17-22)."""
    out = {}
    for k, v in sd.items():
        for pre in ("model.language_model.", "language_model."):
            if k.startswith(pre):
                n = "model." + k[len(pre):]
                if n.endswith(".weight_scale"):
                    break
                if v.dtype == torch.float8_e4m3fn:
                    scale = sd.get(k + "_scale", sd.get(k[:-len("weight")] + "weight_scale"))
                    v = (v.float() * scale.float().reshape(-1, 1)).to(dtype)
                out[n] = v
                break
    return out


def krea2_text_features(enc: "Qwen3Encoder", ids: torch.Tensor) -> torch.Tensor:
    """[1, S] token ids of (system prefix + prompt + suffix) -> [1, S - 34, 12, hidden]: twelve layer outputs stacked on a
    new axis, the system-prefix rows dropped (serenitymojo/models/text_encoder/krea2_qwen3vl_4b.mojo:4-12,36-46)."""
    if ids.shape[1] <= KREA2_PREFIX_DROP:
        raise ValueError("krea2_text_features: the prompt leaves no rows after the system prefix")
    states = enc.layer_states(ids)
    return torch.stack([states[i - 1] for i in KREA2_SELECT_LAYERS], 2)[:, KREA2_PREFIX_DROP:]


def ideogram_text_features(enc: "Qwen3Encoder", ids: torch.Tensor) -> torch.Tensor:
    """[1, S] -> [1, S, 13 * hidden] with feature f of tap t at column ``f * 13 + t``
    (serenitymojo/models/text_encoder/ideogram_qwen3vl.mojo:60-79)."""
    states = enc.layer_states(ids)
    return torch.stack([states[i] for i in IDEOGRAM_TAPS], -1).flatten(-2)


def boogu_text_features(enc: "Qwen3Encoder", ids: torch.Tensor, final_norm: bool = True) -> torch.Tensor:
    """The last layer's output, with or without the final norm (serenitymojo/models/text_encoder/boogu_qwen3vl.mojo:10-13)."""
    return enc(ids, layer=-1, final_norm=final_norm)
