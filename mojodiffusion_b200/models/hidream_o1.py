"""HiDream-O1-Image: a Qwen3-VL language-model spine with three small heads, denoising RGB patches directly.

No separate text encoder and no VAE: the prompt is tokenised into the spine's own embedding table, the noisy image is a
sequence of 32 x 32 x 3 pixel patches (3072 values each) embedded by a bottleneck projection (``x_embedder.proj1`` without
bias, ``proj2`` with bias), and the timestep embedding (cos-first sinusoid of 1000 t -> Linear -> SiLU -> Linear) replaces
the embedding of one reserved token in the text. One forward of the 36-layer spine (grouped-query attention, QK-RMSNorm,
SwiGLU) per denoise step; the text prefix attends causally, image rows attend to everything; rotary positions are the
interleaved three-axis table of Qwen3-VL (text tokens count up on all axes, image patches sit at ``fix_point`` + (0, h, w)).
The output head is one linear back to 3072 values per position; the caller keeps the image rows.

Behaviour and checkpoint keys: serenitymojo/models/dit/hidream_o1.mojo:8-690 (mask: 288-311, positions: 213-285).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence, Tuple

import torch
import torch.nn as nn

from .ideogram4 import mrope_table
from .layers import Linear, init_module_weights, timestep_embedding
from .text.qwen3 import Qwen3Config, _Layer, _Norm


@dataclass
class HiDreamO1Config:
    spine: Qwen3Config = field(default_factory=lambda: Qwen3Config(vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                                                                     num_hidden_layers=36, num_attention_heads=32,
                                                                     num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                                                                     rope_theta=5.0e6))
    patch_dim: int = 3072                    # 32 x 32 x 3
    bottleneck: int = 1024
    timestep_freq_dim: int = 256
    mrope_section: Tuple[int, int, int] = (24, 20, 20)
    tms_token_id: int = 151665               # the reserved token whose embedding is replaced by the timestep embedding
    image_token_id: int = 151655
    vision_start_token_id: int = 151652
    name: str = "hidream-o1-image-8b"


def tiny_hidream_o1_config() -> HiDreamO1Config:
    return HiDreamO1Config(spine=Qwen3Config(vocab_size=64, hidden_size=128, intermediate_size=256, num_hidden_layers=2,
                                             num_attention_heads=4, num_key_value_heads=2, head_dim=32, rope_theta=5.0e6),
                           patch_dim=48, bottleneck=32, timestep_freq_dim=32, mrope_section=(6, 5, 5), tms_token_id=60,
                           image_token_id=61, vision_start_token_id=62, name="tiny-hidream-o1")


def build_mrope_positions(full_ids: Sequence[int], image_token_id: int, ph: int, pw: int, fix_point: int) -> torch.Tensor:
    """[S, 3] (t, h, w) positions: text tokens before the image count 0, 1, 2, ... on all three axes (the token right
    before the first image token keeps 0), image patch (h, w) gets (fix_point, fix_point + h, fix_point + w), anything
    after stays 0. Without image tokens every position is its index."""
    total = len(full_ids)
    pos = torch.zeros(total, 3)
    first = next((i for i, t in enumerate(full_ids) if t == image_token_id), -1)
    if first < 0:
        pos[:] = torch.arange(total, dtype=torch.float32)[:, None]
        return pos
    text_len = max(first - 1, 0)
    pos[:text_len] = torch.arange(text_len, dtype=torch.float32)[:, None]
    k = 0
    for h in range(ph):
        for w in range(pw):
            if text_len + k >= total:
                break
            pos[text_len + k] = torch.tensor([fix_point, fix_point + h, fix_point + w], dtype=torch.float32)
            k += 1
    return pos


def prefix_causal_mask(S: int, ar_len: int, key_valid: torch.Tensor = None, dtype=torch.float32, device=None) -> torch.Tensor:
    """Additive [1, 1, S, S] mask: rows below ``ar_len`` are causal, the others see every key; -1e4 blocks.
    ``key_valid`` [S] additionally blocks padded key columns for every row."""
    i = torch.arange(S, device=device)
    allow = (i[None, :] <= i[:, None]) | (i[:, None] >= ar_len)
    if key_valid is not None:
        allow = allow & key_valid.to(device).bool()[None, :]
    return torch.where(allow, 0.0, -1.0e4).to(dtype)[None, None]


class _XEmbedder(nn.Module):
    def __init__(self, cfg: HiDreamO1Config, dtype, device):
        super().__init__()
        self.proj1 = Linear(cfg.patch_dim, cfg.bottleneck, False, dtype, device)
        self.proj2 = Linear(cfg.bottleneck, cfg.spine.hidden_size, True, dtype, device)


class _TEmbedder(nn.Module):
    def __init__(self, cfg: HiDreamO1Config, dtype, device):
        super().__init__()
        H = cfg.spine.hidden_size
        self.mlp = nn.ModuleDict({"0": Linear(cfg.timestep_freq_dim, H, True, dtype, device), "2": Linear(H, H, True, dtype, device)})


class _Final(nn.Module):
    def __init__(self, cfg: HiDreamO1Config, dtype, device):
        super().__init__()
        self.linear = Linear(cfg.spine.hidden_size, cfg.patch_dim, True, dtype, device)


class _Spine(nn.Module):
    def __init__(self, c: Qwen3Config, dtype, device):
        super().__init__()
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size, dtype=dtype, device=device)
        self.layers = nn.ModuleList([_Layer(c, dtype, device) for _ in range(c.num_hidden_layers)])
        self.norm = _Norm(c.hidden_size, c.rms_norm_eps, dtype, device)


class _Model(nn.Module):
    def __init__(self, cfg: HiDreamO1Config, dtype, device):
        super().__init__()
        self.language_model = _Spine(cfg.spine, dtype, device)
        self.x_embedder = _XEmbedder(cfg, dtype, device)
        self.t_embedder1 = _TEmbedder(cfg, dtype, device)
        self.final_layer2 = _Final(cfg, dtype, device)


class HiDreamO1(nn.Module):
    """forward(input_ids [S_text], noise_patches [1, L, patch_dim], positions [S_text + L, 3], ar_len, t in [0, 1]) ->
    [1, S_text + L, patch_dim]; rows S_text.. are the image prediction."""

    def __init__(self, cfg: HiDreamO1Config, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        self.model = _Model(cfg, dtype, device)

    @torch.no_grad()
    def forward(self, input_ids: Sequence[int], noise_patches: torch.Tensor, positions: torch.Tensor, ar_len: int, timestep: float,
                key_valid: torch.Tensor = None) -> torch.Tensor:
        cfg, m = self.cfg, self.model
        c = cfg.spine
        dev = noise_patches.device
        dt = m.x_embedder.proj1.weight.dtype
        ids = torch.tensor(list(input_ids), dtype=torch.long, device=dev)
        text = m.language_model.embed_tokens(ids)[None]
        te = m.t_embedder1.mlp
        t = torch.tensor([float(timestep)], device=dev)
        t_emb = te["2"](te["0"](timestep_embedding(t, cfg.timestep_freq_dim).to(dt), act="silu"))
        slot = [i for i, tok in enumerate(input_ids) if tok == cfg.tms_token_id]
        if slot:
            text = text.clone()
            text[0, slot[-1]] = t_emb[0]
        x = torch.cat((text, m.x_embedder.proj2(m.x_embedder.proj1(noise_patches.to(dt)))), 1)
        S = x.shape[1]
        cos, sin = mrope_table(positions.to(dev), c.head_dim, cfg.mrope_section, c.rope_theta)
        cos, sin = torch.cat((cos, cos), -1).to(dt)[None, None], torch.cat((sin, sin), -1).to(dt)[None, None]
        mask = prefix_causal_mask(S, ar_len, key_valid, dt, dev)
        for l in m.language_model.layers:
            x = x + l.self_attn(l.input_layernorm(x), cos, sin, mask)
            x = x + l.mlp(l.post_attention_layernorm(x))
        return m.final_layer2.linear(m.language_model.norm(x))

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
