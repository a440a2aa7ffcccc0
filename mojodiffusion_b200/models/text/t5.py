"""T5 v1.1 encoder: RMSNorm (no bias), self-attention with a learned bucketed relative position bias shared from the first
block, gated-GELU feed-forward, no attention scaling. Parameter names are those of ``T5EncoderModel`` checkpoints
(serenitymojo/models/text_encoder/t5_encoder.mojo, umt5_encoder.mojo for the per-layer-bias variant)."""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch import nn

from ... import ops


@dataclass
class T5Config:
    vocab_size: int = 32128
    d_model: int = 4096
    d_kv: int = 64
    d_ff: int = 10240
    num_layers: int = 24
    num_heads: int = 64
    relative_attention_num_buckets: int = 32
    relative_attention_max_distance: int = 128
    layer_norm_epsilon: float = 1e-6
    per_layer_bias: bool = False          # UMT5: every block owns a relative_attention_bias


def t5_xxl_config():
    return T5Config()


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


def relative_bucket(rel: torch.Tensor, num_buckets: int, max_distance: int) -> torch.Tensor:
    """Bidirectional bucketing: half the buckets per sign, exact up to num_buckets/4, logarithmic beyond."""
    nb = num_buckets // 2
    out = (rel > 0).long() * nb
    n = rel.abs()
    max_exact = nb // 2
    large = max_exact + (torch.log(n.float().clamp(min=1) / max_exact) / math.log(max_distance / max_exact) * (nb - max_exact)).long()
    large = torch.minimum(large, torch.full_like(large, nb - 1))
    return out + torch.where(n < max_exact, n, large)


class _SelfAttention(nn.Module):
    def __init__(self, c, has_bias, dtype, device):
        super().__init__()
        inner = c.num_heads * c.d_kv
        self.q, self.k, self.v = (_W(c.d_model, inner, dtype, device) for _ in range(3))
        self.o = _W(inner, c.d_model, dtype, device)
        self.c = c
        if has_bias:
            self.relative_attention_bias = nn.Embedding(c.relative_attention_num_buckets, c.num_heads, dtype=dtype, device=device)

    def bias(self, S, device):
        pos = torch.arange(S, device=device)
        b = relative_bucket(pos[None, :] - pos[:, None], self.c.relative_attention_num_buckets, self.c.relative_attention_max_distance)
        return self.relative_attention_bias(b).permute(2, 0, 1)[None]           # [1, H, S, S]

    def forward(self, x, bias):
        B, S, _ = x.shape
        H, dk = self.c.num_heads, self.c.d_kv
        sh = lambda t: t.view(B, S, H, dk).transpose(1, 2)
        o = torch.nn.functional.scaled_dot_product_attention(sh(self.q(x)), sh(self.k(x)), sh(self.v(x)), attn_mask=bias, scale=1.0)
        return self.o(o.transpose(1, 2).reshape(B, S, H * dk))


class _FF(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.wi_0, self.wi_1 = _W(c.d_model, c.d_ff, dtype, device), _W(c.d_model, c.d_ff, dtype, device)
        self.wo = _W(c.d_ff, c.d_model, dtype, device)

    def forward(self, x):
        return self.wo(torch.nn.functional.gelu(self.wi_0(x), approximate="tanh") * self.wi_1(x))


class _SubLayer(nn.Module):
    def __init__(self, inner_name, inner, c, dtype, device):
        super().__init__()
        setattr(self, inner_name, inner)
        self.layer_norm = _Norm(c.d_model, c.layer_norm_epsilon, dtype, device)


class _Block(nn.Module):
    def __init__(self, c, has_bias, dtype, device):
        super().__init__()
        self.layer = nn.ModuleList([_SubLayer("SelfAttention", _SelfAttention(c, has_bias, dtype, device), c, dtype, device),
                                    _SubLayer("DenseReluDense", _FF(c, dtype, device), c, dtype, device)])


class _Stack(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.block = nn.ModuleList([_Block(c, i == 0 or c.per_layer_bias, dtype, device) for i in range(c.num_layers)])
        self.final_layer_norm = _Norm(c.d_model, c.layer_norm_epsilon, dtype, device)


class T5Encoder(nn.Module):
    def __init__(self, cfg: T5Config, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        self.shared = nn.Embedding(cfg.vocab_size, cfg.d_model, dtype=dtype, device=device)
        self.encoder = _Stack(cfg, dtype, device)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, mask: torch.Tensor = None) -> torch.Tensor:
        """ids [B, S], mask [B, S] (1 = token) -> hidden [B, S, d_model]."""
        x = self.shared(ids)
        B, S = ids.shape
        bias = None
        for blk in self.encoder.block:
            att = blk.layer[0].SelfAttention
            if hasattr(att, "relative_attention_bias"):
                bias = att.bias(S, ids.device).to(x.dtype)
                if mask is not None:
                    bias = bias + (1.0 - mask[:, None, None, :].to(x.dtype)) * torch.finfo(x.dtype).min
            x = x + att(blk.layer[0].layer_norm(x), bias)
            x = x + blk.layer[1].DenseReluDense(blk.layer[1].layer_norm(x))
        return self.encoder.final_layer_norm(x)
