"""CLIP text transformer (pre-LN, causal self-attention, quick-GELU or GELU MLP, final LayerNorm; pooled output = hidden
state at the end-of-text position). Parameter names are those of ``CLIPTextModel`` checkpoints
(serenitymojo/models/text_encoder/clip_encoder.mojo)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ... import ops


@dataclass
class CLIPTextConfig:
    vocab_size: int = 49408
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    max_position_embeddings: int = 77
    hidden_act: str = "quick_gelu"
    layer_norm_eps: float = 1e-5
    eos_token_id: int = 49407


def clip_l_config():
    return CLIPTextConfig()


def clip_g_config():
    return CLIPTextConfig(hidden_size=1280, intermediate_size=5120, num_hidden_layers=32, num_attention_heads=20, hidden_act="gelu")


class _Lin(nn.Module):
    def __init__(self, i, o, dtype, device, bias=True):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(o, i, dtype=dtype, device=device).normal_(0, 0.02))
        self.bias = nn.Parameter(torch.zeros(o, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias)


class _Attn(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        D = c.hidden_size
        self.heads = c.num_attention_heads
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (_Lin(D, D, dtype, device) for _ in range(4))

    def forward(self, x, mask):
        B, S, D = x.shape
        sh = lambda t: t.view(B, S, self.heads, D // self.heads).transpose(1, 2)
        o = torch.nn.functional.scaled_dot_product_attention(sh(self.q_proj(x)), sh(self.k_proj(x)), sh(self.v_proj(x)), attn_mask=mask)
        return self.out_proj(o.transpose(1, 2).reshape(B, S, D))


class _MLP(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.fc1, self.fc2 = _Lin(c.hidden_size, c.intermediate_size, dtype, device), _Lin(c.intermediate_size, c.hidden_size, dtype, device)
        self.act = c.hidden_act

    def forward(self, x):
        h = self.fc1(x)
        h = h * torch.sigmoid(1.702 * h) if self.act == "quick_gelu" else torch.nn.functional.gelu(h)
        return self.fc2(h)


class _Layer(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.self_attn, self.mlp = _Attn(c, dtype, device), _MLP(c, dtype, device)
        self.layer_norm1 = nn.LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype, device=device)
        self.layer_norm2 = nn.LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype, device=device)

    def forward(self, x, mask):
        x = x + self.self_attn(self.layer_norm1(x), mask)
        return x + self.mlp(self.layer_norm2(x))


class _Embeddings(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.token_embedding = nn.Embedding(c.vocab_size, c.hidden_size, dtype=dtype, device=device)
        self.position_embedding = nn.Embedding(c.max_position_embeddings, c.hidden_size, dtype=dtype, device=device)


class _Encoder(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.layers = nn.ModuleList([_Layer(c, dtype, device) for _ in range(c.num_hidden_layers)])


class _TextModel(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.embeddings, self.encoder = _Embeddings(c, dtype, device), _Encoder(c, dtype, device)
        self.final_layer_norm = nn.LayerNorm(c.hidden_size, c.layer_norm_eps, dtype=dtype, device=device)


class CLIPTextEncoder(nn.Module):
    def __init__(self, cfg: CLIPTextConfig, dtype=torch.float32, device=None):
        super().__init__()
        self.cfg = cfg
        self.text_model = _TextModel(cfg, dtype, device)

    @torch.no_grad()
    def forward(self, ids: torch.Tensor, clip_skip: int = 0):
        """ids [B, S] -> (hidden [B, S, D] after the final LayerNorm (``clip_skip`` = number of last layers to drop, the
        penultimate-layer convention of SDXL is clip_skip=1 without final norm handled by the caller), pooled [B, D])."""
        tm = self.text_model
        B, S = ids.shape
        x = tm.embeddings.token_embedding(ids) + tm.embeddings.position_embedding(torch.arange(S, device=ids.device))[None]
        mask = torch.full((S, S), float("-inf"), device=ids.device, dtype=x.dtype).triu(1)
        layers = tm.encoder.layers[: len(tm.encoder.layers) - clip_skip]
        hidden_pen = None
        for i, l in enumerate(tm.encoder.layers):
            x = l(x, mask)
            if i == len(layers) - 1:
                hidden_pen = x
        last = tm.final_layer_norm(x)
        eos = (ids == self.cfg.eos_token_id).int().argmax(dim=-1) if self.cfg.eos_token_id in ids else ids.argmax(dim=-1)
        pooled = last[torch.arange(B, device=ids.device), eos]
        return (last if clip_skip == 0 else hidden_pen), pooled
