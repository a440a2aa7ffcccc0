"""daVinci-MagiHuman DiT (15 B): one stream of video, audio and text tokens (sorted in that order) through 40 layers of
width 5120 with 40 query / 8 key-value heads of 128. No timestep input and no cross attention.

* every RMSNorm gain is ``weight + 1`` (eps 1e-6); QK norms act per head;
* one fused projection gives q (5120) | k (1024) | v (1024) | gate (40): the attention output of head h is multiplied by
  ``sigmoid(gate_h)`` before ``linear_proj``; no biases;
* rotary embedding on the first 96 of the 128 head columns (half-split) from a Fourier table: with per-token coordinates
  (t, h, w), grid sizes and reference sizes, ``c_axis = (coord - centre) * (ref - 1) / (size - 1)`` (centre = (size - 1) / 2,
  0 for time) and angle[axis * 16 + b] = c_axis * bands[b] with the checkpoint's own 16 ``adapter.rope.bands``;
* feed-forward: layers 4..39 use SwiGLU7 on an INTERLEAVED up projection (even columns gate, odd columns linear):
  ``g = min(x_even, 7); l = clamp(x_odd, -7, 7); g * sigmoid(1.702 g) * (l + 1)`` (13 652 wide); layers 0..3 use GELU7
  ``c * sigmoid(1.702 c), c = min(x, 7)`` on a plain 20 480-wide projection;
* layers 0..3 and 36..39 hold THREE weight sets (video, audio, text) stacked along the output dimension of every norm and
  linear: each token group uses its own; layers 4..35 share one set;
* adapters ``video_embedder`` (192 -> 5120), ``audio_embedder`` (64), ``text_embedder`` (3584) with bias; heads
  ``final_norm_video`` + ``final_linear_video`` (-> 192) and the audio pair (-> 64, zero-padded to 192); text rows give zeros.

The 1080p super-resolution model has the same mathematics with split projections (``linear_q / _k / _v / _g``, and per
modality ``..._video / _audio / _text``); ``remap_magihuman_sr_keys`` concatenates them into the fused layout. Its sampler is
the distilled step ``clean = x - sigma * v; x' = sigma' * noise + (1 - sigma') * clean``.

Behaviour: serenitymojo/models/dit/magihuman_dit.mojo:10-60 (architecture), :110-176 (SwiGLU7), :292-371 (shared layer),
:443-470 (GELU7), :485-620 (per-modality layer), :640-690 (Fourier table), :708-770 (heads, adapters), :773-806 (stack);
serenitymojo/models/dit/magihuman_sr_dit.mojo:10-48 (split layout, distilled step).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Sequence, Tuple

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, init_module_weights

MODALITIES = ("video", "audio", "text")


@dataclass
class MagiHumanConfig:
    hidden_size: int = 5120
    head_dim: int = 128
    num_heads_q: int = 40
    num_heads_kv: int = 8
    rope_dim: int = 96
    intermediate_swiglu: int = 13652
    intermediate_gelu: int = 20480
    num_layers: int = 40
    mm_layers: Tuple[int, ...] = (0, 1, 2, 3, 36, 37, 38, 39)
    gelu7_layers: Tuple[int, ...] = (0, 1, 2, 3)
    video_in: int = 192
    audio_in: int = 64
    text_in: int = 3584
    rope_bands: int = 16
    rms_eps: float = 1e-6
    name: str = "magihuman-15b"

    @property
    def q_size(self):
        return self.num_heads_q * self.head_dim

    @property
    def kv_size(self):
        return self.num_heads_kv * self.head_dim

    @property
    def qkv_out(self):
        return self.q_size + 2 * self.kv_size + self.num_heads_q


def tiny_magihuman_config() -> MagiHumanConfig:
    return MagiHumanConfig(hidden_size=128, head_dim=32, num_heads_q=4, num_heads_kv=2, rope_dim=24, intermediate_swiglu=84,
                           intermediate_gelu=160, num_layers=4, mm_layers=(0, 3), gelu7_layers=(0,), video_in=24, audio_in=8,
                           text_in=40, rope_bands=4, name="tiny-magihuman")


def swiglu7(x: torch.Tensor) -> torch.Tensor:
    g = x[..., 0::2].float().clamp(max=7.0)
    l = x[..., 1::2].float().clamp(-7.0, 7.0)
    return (g * torch.sigmoid(1.702 * g) * (l + 1.0)).to(x.dtype)


def gelu7(x: torch.Tensor) -> torch.Tensor:
    c = x.float().clamp(max=7.0)
    return (c * torch.sigmoid(1.702 * c)).to(x.dtype)


def fourier_rope(coords: torch.Tensor, bands: torch.Tensor):
    """coords [L, 9] = (t, h, w, T, H, W, refT, refH, refW), bands [B] -> cos / sin [L, 3 B] fp32 (float64 inside)."""
    c = coords.detach().double().cpu()
    xyz, size, ref = c[:, 0:3], c[:, 3:6], c[:, 6:9]
    scale = (ref - 1.0) / (size - 1.0 + 1e-30)
    centre = (size - 1.0) * 0.5
    centre[:, 0] = 0.0
    proj = ((xyz - centre) * scale)[:, :, None] * bands.detach().double().cpu()[None, None, :]      # [L, 3, B]
    proj = proj.flatten(1)
    return proj.cos().float().to(coords.device), proj.sin().float().to(coords.device)


def _rope_partial(x, cos, sin, rope_dim: int):
    """Half-split rotation of the first ``rope_dim`` columns of [L, H, Dh] by tables [L, rope_dim / 2]."""
    r, rest = x[..., :rope_dim], x[..., rope_dim:]
    a, b = r.chunk(2, -1)
    c, s = cos[:, None].to(x.dtype), sin[:, None].to(x.dtype)
    return torch.cat((a * c - b * s, b * c + a * s, rest), -1)


class _W(nn.Module):
    """A bias-free weight [sets * out, in] (``sets`` = 3 in per-modality layers) or a norm gain [sets * dim]."""

    def __init__(self, shape, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.zeros(*shape, dtype=dtype, device=device))


class _Attention(nn.Module):
    def __init__(self, c: MagiHumanConfig, sets: int, dtype, device):
        super().__init__()
        self.pre_norm = _W((sets * c.hidden_size,), dtype, device)
        self.linear_qkv = _W((sets * c.qkv_out, c.hidden_size), dtype, device)
        self.q_norm = _W((sets * c.head_dim,), dtype, device)
        self.k_norm = _W((sets * c.head_dim,), dtype, device)
        self.linear_proj = _W((sets * c.hidden_size, c.q_size), dtype, device)


class _Mlp(nn.Module):
    def __init__(self, c: MagiHumanConfig, sets: int, gelu: bool, dtype, device):
        super().__init__()
        up = c.intermediate_gelu if gelu else 2 * c.intermediate_swiglu
        mid = c.intermediate_gelu if gelu else c.intermediate_swiglu
        self.pre_norm = _W((sets * c.hidden_size,), dtype, device)
        self.up_gate_proj = _W((sets * up, c.hidden_size), dtype, device)
        self.down_proj = _W((sets * c.hidden_size, mid), dtype, device)


class MagiHumanLayer(nn.Module):
    def __init__(self, c: MagiHumanConfig, index: int, dtype, device):
        super().__init__()
        self.c = c
        self.sets = 3 if index in c.mm_layers else 1
        self.gelu = index in c.gelu7_layers
        self.attention = _Attention(c, self.sets, dtype, device)
        self.mlp = _Mlp(c, self.sets, self.gelu, dtype, device)

    def _groups(self, groups: Sequence[int], L: int):
        if self.sets == 1:
            return [(0, 0, L)]
        out, o = [], 0
        for i, n in enumerate(groups):
            if n:
                out.append((i, o, o + n))
            o += n
        return out

    def _norm(self, x, w: _W, groups):
        dim = x.shape[-1]
        return torch.cat([ops.norm_modulate(x[a:b], weight=(w.weight[i * dim:(i + 1) * dim].float() + 1.0).to(x.dtype),
                                            eps=self.c.rms_eps, rms=True) for i, a, b in groups], 0)

    def _linear(self, x, w: _W, groups):
        out = w.weight.shape[0] // self.sets
        return torch.cat([ops.linear(x[a:b], w.weight[i * out:(i + 1) * out]) for i, a, b in groups], 0)

    def forward(self, x, cos, sin, groups: Sequence[int]):
        """x [L, hidden] -> [L, hidden]; ``groups`` = (video, audio, text) token counts."""
        c, a, m = self.c, self.attention, self.mlp
        L = x.shape[0]
        H, KV, Dh = c.num_heads_q, c.num_heads_kv, c.head_dim
        gs = self._groups(groups, L)
        qkv = self._linear(self._norm(x, a.pre_norm, gs), a.linear_qkv, gs)
        q, k, v, g = qkv.split((c.q_size, c.kv_size, c.kv_size, H), -1)
        q = _rope_partial(self._norm(q.reshape(L, H, Dh), a.q_norm, gs), cos, sin, c.rope_dim)
        k = _rope_partial(self._norm(k.reshape(L, KV, Dh), a.k_norm, gs), cos, sin, c.rope_dim)
        rep = H // KV
        o = ops.attention(q[None], k.repeat_interleave(rep, 1)[None], v.reshape(L, KV, Dh).repeat_interleave(rep, 1)[None])[0]
        o = (o.float() * torch.sigmoid(g.float())[..., None]).to(x.dtype).reshape(L, H * Dh)
        x = x + self._linear(o, a.linear_proj, gs)
        up = self._linear(self._norm(x, m.pre_norm, gs), m.up_gate_proj, gs)
        return x + self._linear(gelu7(up) if self.gelu else swiglu7(up), m.down_proj, gs)


class _Rope(nn.Module):
    def __init__(self, n, dtype, device):
        super().__init__()
        self.bands = nn.Parameter(torch.zeros(n, dtype=dtype, device=device))


class _Adapter(nn.Module):
    def __init__(self, c: MagiHumanConfig, dtype, device):
        super().__init__()
        self.rope = _Rope(c.rope_bands, dtype, device)
        self.video_embedder = Linear(c.video_in, c.hidden_size, True, dtype, device)
        self.audio_embedder = Linear(c.audio_in, c.hidden_size, True, dtype, device)
        self.text_embedder = Linear(c.text_in, c.hidden_size, True, dtype, device)


class _Block(nn.Module):
    def __init__(self, c, dtype, device):
        super().__init__()
        self.layers = nn.ModuleList([MagiHumanLayer(c, i, dtype, device) for i in range(c.num_layers)])


class MagiHumanDiT(nn.Module):
    """forward(video [V, 192], audio [A, 64], text [T, 3584], coords [V + A + T, 9]) -> [V + A + T, 192] fp32: video rows carry
    the video prediction, audio rows the audio prediction in their first 64 columns, text rows zeros."""

    def __init__(self, cfg: MagiHumanConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        assert cfg.rope_dim == 6 * cfg.rope_bands and cfg.rope_dim <= cfg.head_dim
        self.adapter = _Adapter(cfg, dtype, device)
        self.block = _Block(cfg, dtype, device)
        self.final_norm_video = _W((cfg.hidden_size,), dtype, device)
        self.final_linear_video = _W((cfg.video_in, cfg.hidden_size), dtype, device)
        self.final_norm_audio = _W((cfg.hidden_size,), dtype, device)
        self.final_linear_audio = _W((cfg.audio_in, cfg.hidden_size), dtype, device)

    @torch.no_grad()
    def forward(self, video, audio, text, coords):
        c, ad = self.cfg, self.adapter
        dt = ad.video_embedder.weight.dtype
        groups = (video.shape[0], audio.shape[0], text.shape[0])
        parts = [emb(t.to(dt)) for emb, t in ((ad.video_embedder, video), (ad.audio_embedder, audio), (ad.text_embedder, text)) if t.shape[0]]
        x = torch.cat(parts, 0)
        cos, sin = fourier_rope(coords, ad.rope.bands)
        for layer in self.block.layers:
            x = layer(x, cos, sin, groups)
        V, A, T = groups
        out = torch.zeros(V + A + T, max(c.video_in, c.audio_in), dtype=torch.float32, device=x.device)
        norm = lambda h, w: ops.norm_modulate(h, weight=(w.weight.float() + 1.0).to(h.dtype), eps=c.rms_eps, rms=True)
        if V:
            out[:V, :c.video_in] = ops.linear(norm(x[:V], self.final_norm_video), self.final_linear_video.weight).float()
        if A:
            out[V:V + A, :c.audio_in] = ops.linear(norm(x[V:V + A], self.final_norm_audio), self.final_linear_audio.weight).float()
        return out

    def init_weights(self, seed: int = 0, std: float = 0.02):
        init_module_weights(self, seed, std)
        with torch.no_grad():
            for n, p in self.named_parameters():
                if p.dim() == 1 and "norm" in n:
                    p.zero_()                                                          # gains are weight + 1
            half = self.cfg.rope_bands
            self.adapter.rope.bands.copy_((1.0 / 10000.0 ** (torch.arange(half).float() / half)).to(self.adapter.rope.bands.dtype))
        return self


def remap_magihuman_sr_keys(sd: Dict[str, torch.Tensor], cfg: MagiHumanConfig) -> Dict[str, torch.Tensor]:
    """Split super-resolution layout -> fused: ``linear_{q,k,v,g}[_modality]`` become ``linear_qkv`` rows ordered
    (modality, [q; k; v; g]); ``linear_proj_*`` and ``mlp.{up_gate_proj,down_proj}_*`` are stacked in modality order."""
    out = {k: v for k, v in sd.items() if not any(s in k for s in (".linear_q", ".linear_k", ".linear_v", ".linear_g")) and
           not any(k.endswith(f"_{m}.weight") and (".linear_proj_" in k or ".mlp." in k) for m in MODALITIES)}
    for i in range(cfg.num_layers):
        p = f"block.layers.{i}."
        if p + "attention.linear_q.weight" in sd:
            out[p + "attention.linear_qkv.weight"] = torch.cat([sd[p + f"attention.linear_{w}.weight"] for w in "qkvg"], 0)
        elif p + "attention.linear_q_video.weight" in sd:
            out[p + "attention.linear_qkv.weight"] = torch.cat([sd[p + f"attention.linear_{w}_{m}.weight"] for m in MODALITIES for w in "qkvg"], 0)
            out[p + "attention.linear_proj.weight"] = torch.cat([sd[p + f"attention.linear_proj_{m}.weight"] for m in MODALITIES], 0)
            for w in ("up_gate_proj", "down_proj"):
                out[p + f"mlp.{w}.weight"] = torch.cat([sd[p + f"mlp.{w}_{m}.weight"] for m in MODALITIES], 0)
    return out


def distilled_step(x: torch.Tensor, velocity: torch.Tensor, noise: torch.Tensor, sigma: float, sigma_next: float) -> torch.Tensor:
    """``clean = x - sigma * v``; ``x' = sigma_next * noise + (1 - sigma_next) * clean``."""
    clean = x.float() - sigma * velocity.float()
    return sigma_next * noise.float() + (1.0 - sigma_next) * clean
