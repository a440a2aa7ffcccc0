"""KV-cached incremental decode for the Qwen3 stack (prompt expansion / "magic prompt").

``prefill`` runs the prompt once and fills a per-layer cache with the normalised, rotated keys and the values;
``decode_step`` then processes ONE token: one-row q / k / v projections, append k and v at the current position, and a
single-query grouped-query attention over the cache (each query head reads the cache of its key/value group, no
``repeat`` of the cache), followed by the MLP; ``logits`` applies the final norm and the (tied or separate) output
head to the last position. ``generate`` loops decode + host sampling until EOS or ``max_new_tokens``
(serenitymojo/llm/decoder.mojo:1-150, serenitymojo/llm/sqa.mojo:1-116)."""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..models.text.qwen3 import Qwen3Config, Qwen3Encoder, _rope
from .sampler import Rng, SamplerConfig, sample


def single_query_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, length: int,
                           scale: Optional[float] = None) -> torch.Tensor:
    """q [B, H, Dh] (one position), caches [B, Hkv, T, Dh] valid up to ``length`` -> [B, H, Dh]. Query head h reads
    key/value head h // (H / Hkv); scores and the weighted sum are accumulated in fp32."""
    B, H, Dh = q.shape
    Hkv = k_cache.shape[1]
    rep = H // Hkv
    scale = scale if scale is not None else Dh ** -0.5
    qg = q.view(B, Hkv, rep, Dh).float()
    k = k_cache[:, :, :length].float()
    v = v_cache[:, :, :length].float()
    s = torch.einsum("bgrd,bgtd->bgrt", qg, k) * scale
    p = torch.softmax(s, dim=-1)
    return torch.einsum("bgrt,bgtd->bgrd", p, v).reshape(B, H, Dh).to(q.dtype)


class KVCache:
    def __init__(self, cfg: Qwen3Config, batch: int, max_len: int, dtype, device):
        shape = (cfg.num_hidden_layers, batch, cfg.num_key_value_heads, max_len, cfg.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.length = 0
        self.max_len = max_len


class Qwen3Decoder:
    """Wraps a :class:`Qwen3Encoder` (same weights, same parameter names) with an output head for generation."""

    def __init__(self, encoder: Qwen3Encoder, lm_head: Optional[torch.Tensor] = None):
        self.enc = encoder
        self.cfg = encoder.cfg
        self.lm_head = lm_head          # [vocab, hidden]; None: tied to the embedding table

    def _angles(self, pos: torch.Tensor, dtype):
        c = self.cfg
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.head_dim, 2, device=pos.device).float() / c.head_dim))
        ang = pos.float()[:, None] * inv[None]
        emb = torch.cat((ang, ang), dim=-1)
        return emb.cos().to(dtype), emb.sin().to(dtype)

    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, max_len: int) -> "tuple[torch.Tensor, KVCache]":
        """ids [B, S] -> (hidden of the last position [B, hidden], cache holding positions 0..S-1)."""
        c, m = self.cfg, self.enc.model
        B, S = ids.shape
        x = m.embed_tokens(ids)
        cache = KVCache(c, B, max_len, x.dtype, ids.device)
        cos, sin = self._angles(torch.arange(S, device=ids.device), x.dtype)
        cos, sin = cos[None, None], sin[None, None]
        mask = torch.full((S, S), float("-inf"), device=ids.device, dtype=x.dtype).triu(1)[None, None]
        rep = c.num_attention_heads // c.num_key_value_heads
        for li, l in enumerate(m.layers):
            a = l.self_attn
            h = l.input_layernorm(x)
            q = a.q_norm(a.q_proj(h).view(B, S, c.num_attention_heads, c.head_dim)).transpose(1, 2)
            k = a.k_norm(a.k_proj(h).view(B, S, c.num_key_value_heads, c.head_dim)).transpose(1, 2)
            v = a.v_proj(h).view(B, S, c.num_key_value_heads, c.head_dim).transpose(1, 2)
            q, k = _rope(q, cos, sin), _rope(k, cos, sin)
            cache.k[li, :, :, :S] = k
            cache.v[li, :, :, :S] = v
            o = torch.nn.functional.scaled_dot_product_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1),
                                                                 attn_mask=mask)
            x = x + a.o_proj(o.transpose(1, 2).reshape(B, S, -1))
            x = x + l.mlp(l.post_attention_layernorm(x))
        cache.length = S
        return x[:, -1], cache

    @torch.no_grad()
    def decode_step(self, token: torch.Tensor, cache: KVCache) -> torch.Tensor:
        """token [B] at position ``cache.length`` -> hidden [B, hidden]; the cache grows by one."""
        c, m = self.cfg, self.enc.model
        B = token.shape[0]
        pos = cache.length
        if pos >= cache.max_len:
            raise RuntimeError("KV cache is full")
        x = m.embed_tokens(token)                                         # [B, hidden]
        cos, sin = self._angles(torch.tensor([pos], device=token.device), x.dtype)
        for li, l in enumerate(m.layers):
            a = l.self_attn
            h = l.input_layernorm(x)
            q = _rope(a.q_norm(a.q_proj(h).view(B, c.num_attention_heads, c.head_dim)), cos, sin)
            k = _rope(a.k_norm(a.k_proj(h).view(B, c.num_key_value_heads, c.head_dim)), cos, sin)
            cache.k[li, :, :, pos] = k
            cache.v[li, :, :, pos] = a.v_proj(h).view(B, c.num_key_value_heads, c.head_dim)
            o = single_query_attention(q, cache.k[li], cache.v[li], pos + 1)
            x = x + a.o_proj(o.reshape(B, -1))
            x = x + l.mlp(l.post_attention_layernorm(x))
        cache.length = pos + 1
        return x

    @torch.no_grad()
    def logits(self, hidden: torch.Tensor) -> torch.Tensor:
        h = self.enc.model.norm(hidden)
        w = self.lm_head if self.lm_head is not None else self.enc.model.embed_tokens.weight
        return h.float() @ w.float().t()

    @torch.no_grad()
    def generate(self, prompt_ids: Sequence[int], max_new_tokens: int, cfg: SamplerConfig = SamplerConfig(),
                 eos_ids: Sequence[int] = (), device=None) -> List[int]:
        dev = device or next(self.enc.parameters()).device
        ids = torch.tensor([list(prompt_ids)], dtype=torch.long, device=dev)
        hidden, cache = self.prefill(ids, ids.shape[1] + max_new_tokens)
        rng = Rng(cfg.seed)
        out: List[int] = []
        for _ in range(max_new_tokens):
            tok = sample(self.logits(hidden)[0].tolist(), cfg, rng)
            out.append(tok)
            if tok in eos_ids or cache.length >= cache.max_len:
                break
            hidden = self.decode_step(torch.tensor([tok], dtype=torch.long, device=dev), cache)
        return out
