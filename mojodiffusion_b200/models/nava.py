"""NAVA audio + video DiT: the Wan2.2 5 B transformer (width 3072, 24 heads of 128, feed-forward 14 336, text cross attention,
six-chunk timestep modulation) run over ONE sequence [video tokens, audio tokens]. The first 10 blocks are double-stream
(separate video / audio weights for the self- and cross-attention projections, QK norms and modulation tables; the affine
``norm3`` and the feed-forward are shared), the next 20 are plain Wan blocks over the joint sequence.

* video tokens: 1 x 2 x 2 patches of a 48-channel latent; rotary axes (44, 42, 42) over (frame, row, column);
* audio tokens: 128-channel latent frames through Conv1d(k = 7) -> SiLU -> a gated Conv1d MLP ``w2(silu(w1 x) * w3 x)``;
  rotary embedding only on the first 44 head columns, from the single position 0.24 * index (the rest passes through);
* QK-RMSNorm acts on the full 3072-wide projection before the head split; attention is joint over video + audio rows (or
  per modality with ``masking_modality``); cross attention reads the text (zero-padded to 512 rows) without a gate;
* both heads: ``Linear(LayerNorm(x) * (1 + m1 + e) + m0 + e)`` with their own two-row modulation; video rows are unpatchified.

Behaviour: serenitymojo/models/dit/nava_block.mojo:92-137 (rotary tables), :258-440 (double block), :505-626 (single block);
serenitymojo/models/dit/nava_embed.mojo:111-157 (video patches), :210-288 (audio embedder), :291-331 (text), :334-366 (time);
serenitymojo/models/dit/nava_dit.mojo:78-150 (heads, output layout), :150-250 (wiring). The checkpoint stores its block
linears as fp8 rows with a per-row scale under the prefix ``backbone.``: ``remap_nava_keys`` strips the prefix and dequantises.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import audio as A
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding
from .wan import LayerNormAffine, WanBlock, WanConfig, WanDiT, _Attn, _Head, _Patch, patchify_3d


@dataclass
class NavaConfig(WanConfig):
    in_dim: int = 48
    out_dim: int = 48
    dim: int = 3072
    heads: int = 24
    ffn_dim: int = 14336
    depth: int = 20                 # single (joint) blocks
    double_depth: int = 10
    audio_dim: int = 128
    audio_mlp_dim: int = 8192
    audio_rope_dim: int = 44
    audio_pos_step: float = 0.24
    text_len: int = 512
    name: str = "nava"


def tiny_nava_config() -> NavaConfig:
    return NavaConfig(in_dim=8, out_dim=8, dim=128, heads=2, ffn_dim=256, depth=2, double_depth=2, text_dim=96, freq_dim=64, audio_dim=16,
                      audio_mlp_dim=64, audio_rope_dim=22, text_len=12, name="tiny-nava")


def nava_rope_table(f: int, h: int, w: int, n_audio: int, cfg: NavaConfig, device=None):
    """cos / sin [f h w + n_audio, head_dim / 2]: video rows from three axes, audio rows from one position on the first
    ``audio_rope_dim / 2`` pairs and the identity rotation on the rest."""
    vc, vs = ops.rope_table(WanDiT.make_ids(f, h, w, device), cfg.axes_dim, cfg.theta)
    pos = (torch.arange(n_audio, dtype=torch.float32, device=device) * cfg.audio_pos_step)[:, None]
    ac, as_ = ops.rope_table(pos, (cfg.audio_rope_dim,), cfg.theta)
    half = cfg.head_dim // 2
    ac = torch.cat((ac, torch.ones(n_audio, half - ac.shape[1], device=ac.device)), 1)
    as_ = torch.cat((as_, torch.zeros(n_audio, half - as_.shape[1], device=as_.device)), 1)
    return torch.cat((vc, ac), 0).contiguous(), torch.cat((vs, as_), 0).contiguous()


class _DualAttn(nn.Module):
    """Video projections under the plain names, audio ones with the ``_audio`` suffix."""

    def __init__(self, dim, dtype, device):
        super().__init__()
        for s in ("", "_audio"):
            for n in "qkvo":
                setattr(self, n + s, Linear(dim, dim, True, dtype, device))
            setattr(self, "norm_q" + s, RMSNorm(dim, 1e-6, dtype, device))
            setattr(self, "norm_k" + s, RMSNorm(dim, 1e-6, dtype, device))


class _Mod(nn.Module):
    def __init__(self, dim, dtype, device):
        super().__init__()
        self.modulation = nn.Parameter(torch.zeros(1, 6, dim, dtype=dtype, device=device))


class NavaDoubleBlock(nn.Module):
    def __init__(self, cfg: NavaConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        D = cfg.dim
        self.self_attn, self.cross_attn = _DualAttn(D, dtype, device), _DualAttn(D, dtype, device)
        self.norm3 = LayerNormAffine(D, 1e-6, dtype, device)
        self.ffn = nn.ModuleDict({"0": Linear(D, cfg.ffn_dim, True, dtype, device), "2": Linear(cfg.ffn_dim, D, True, dtype, device)})
        self.modulation, self.modulation_audio = _Mod(D, dtype, device), _Mod(D, dtype, device)

    def forward(self, x, ctx, e0, cos, sin, n_video: int, masking_modality: bool = False):
        cfg = self.cfg
        B, S, D = x.shape
        H, Dh, V = cfg.heads, cfg.head_dim, n_video
        sa, ca = self.self_attn, self.cross_attn
        streams = (("", slice(0, V), (self.modulation.modulation.float() + e0.float()).to(x.dtype)),
                   ("_audio", slice(V, S), (self.modulation_audio.modulation.float() + e0.float()).to(x.dtype)))
        q, k, v = [], [], []
        for sfx, rows, e in streams:
            xn = ops.norm_modulate(x[:, rows], scale=e[:, 1], shift=e[:, 0], eps=1e-6)
            q.append(getattr(sa, "norm_q" + sfx)(getattr(sa, "q" + sfx)(xn)))
            k.append(getattr(sa, "norm_k" + sfx)(getattr(sa, "k" + sfx)(xn)))
            v.append(getattr(sa, "v" + sfx)(xn))
        qk = ops.qk_norm_rope(torch.cat((torch.cat(q, 1), torch.cat(k, 1)), -1), H, Dh, None, None, cos, sin, interleaved=True, do_norm=False)
        qh, kh, vh = qk[..., :D].unflatten(-1, (H, Dh)), qk[..., D:].unflatten(-1, (H, Dh)), torch.cat(v, 1).unflatten(-1, (H, Dh))
        if masking_modality:
            a = torch.cat([ops.attention(qh[:, r], kh[:, r], vh[:, r]) for _, r, _ in streams], 1)
        else:
            a = ops.attention(qh, kh, vh)
        a = a.reshape(B, S, D)
        parts = []
        for sfx, rows, e in streams:
            n = rows.stop - rows.start
            xs = getattr(sa, "o" + sfx)(a[:, rows], residual=x[:, rows], gate=e[:, 2], rows_per_group=n)
            qc = getattr(ca, "norm_q" + sfx)(getattr(ca, "q" + sfx)(self.norm3(xs))).unflatten(-1, (H, Dh))
            kc = getattr(ca, "norm_k" + sfx)(getattr(ca, "k" + sfx)(ctx)).unflatten(-1, (H, Dh))
            vc = getattr(ca, "v" + sfx)(ctx).unflatten(-1, (H, Dh))
            xs = getattr(ca, "o" + sfx)(ops.attention(qc, kc, vc).reshape(B, n, D), residual=xs)
            h = self.ffn["0"](ops.norm_modulate(xs, scale=e[:, 4], shift=e[:, 3], eps=1e-6), act="gelu_tanh")
            parts.append(self.ffn["2"](h, residual=xs, gate=e[:, 5], rows_per_group=n))
        return torch.cat(parts, 1)


class _Conv1dParams(nn.Module):
    def __init__(self, cin, cout, k, bias, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cout, cin, k, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device)) if bias else None

    def forward(self, x_nlc):
        return A.conv1d(x_nlc.transpose(1, 2), self.weight, self.bias, padding=self.weight.shape[-1] // 2).transpose(1, 2)


class _ConvMlp(nn.Module):
    def __init__(self, dim, hidden, dtype, device):
        super().__init__()
        self.w1 = _Conv1dParams(dim, hidden, 7, False, dtype, device)
        self.w2 = _Conv1dParams(hidden, dim, 7, False, dtype, device)
        self.w3 = _Conv1dParams(dim, hidden, 7, False, dtype, device)

    def forward(self, x):
        return self.w2(ops.activation(self.w1(x).contiguous(), "silu") * self.w3(x))


class NavaDiT(nn.Module):
    """forward(video [B, 48, F, H, W], audio [B, N, 128], text [B, T <= 512, 4096], t [B] in [0, 1]) ->
    (video velocity [B, 48, F, H, W], audio velocity [B, N, 128])."""

    def __init__(self, cfg: NavaConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.dim
        self.patch_embedding = _Patch(cfg, dtype, device)
        self.patch_embedding_audio = nn.ModuleDict({"0": _Conv1dParams(cfg.audio_dim, D, 7, True, dtype, device),
                                                    "2": _ConvMlp(D, cfg.audio_mlp_dim, dtype, device)})
        self.text_embedding = nn.ModuleDict({"0": Linear(cfg.text_dim, D, True, dtype, device), "2": Linear(D, D, True, dtype, device)})
        self.time_embedding = nn.ModuleDict({"0": Linear(cfg.freq_dim, D, True, dtype, device), "2": Linear(D, D, True, dtype, device)})
        self.time_projection = nn.ModuleDict({"1": Linear(D, 6 * D, True, dtype, device)})
        self.double_blocks = nn.ModuleList([NavaDoubleBlock(cfg, dtype, device) for _ in range(cfg.double_depth)])
        self.single_blocks = nn.ModuleList([WanBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        self.head = _Head(cfg, dtype, device)
        ha = nn.Module()
        ha.head = Linear(D, cfg.audio_dim, True, dtype, device)
        ha.modulation = nn.Parameter(torch.zeros(1, 2, D, dtype=dtype, device=device))
        self.head_audio = ha

    @torch.no_grad()
    def forward(self, video, audio, text, timesteps, masking_modality: bool = False):
        cfg = self.cfg
        B, C, F_, Hh, Ww = video.shape
        pt, ph, pw = cfg.patch
        f, h, w = F_ // pt, Hh // ph, Ww // pw
        D, V, Na = cfg.dim, f * h * w, audio.shape[1]
        dt = self.patch_embedding.weight.dtype
        xv = ops.linear(patchify_3d(video, pt, ph, pw).to(dt), self.patch_embedding.weight.flatten(1), self.patch_embedding.bias)
        pa = self.patch_embedding_audio
        xa = pa["2"](ops.activation(pa["0"](audio.to(dt)).contiguous(), "silu"))
        x = torch.cat((xv, xa), 1)
        if text.shape[1] < cfg.text_len:
            text = torch.cat((text, text.new_zeros(B, cfg.text_len - text.shape[1], text.shape[2])), 1)
        tx = self.text_embedding
        ctx = tx["2"](tx["0"](text.to(dt), act="gelu_tanh"))
        te = self.time_embedding
        e = te["2"](te["0"](timestep_embedding(timesteps, cfg.freq_dim).to(dt), act="silu"))
        e0 = self.time_projection["1"](ops.activation(e, "silu")).reshape(B, 6, D)
        cos, sin = nava_rope_table(f, h, w, Na, cfg, video.device)
        for blk in self.double_blocks:
            x = blk(x, ctx, e0, cos, sin, V, masking_modality)
        for blk in self.single_blocks:
            if masking_modality:
                raise NotImplementedError("per-modality attention in the joint blocks")
            x = blk(x, ctx, e0, cos, sin)
        outs = []
        for head, rows in ((self.head, slice(0, V)), (self.head_audio, slice(V, V + Na))):
            m = (head.modulation.float() + e[:, None].float()).to(x.dtype)
            outs.append(head.head(ops.norm_modulate(x[:, rows], scale=m[:, 1], shift=m[:, 0], eps=1e-6)))
        vid = outs[0].reshape(B, f, h, w, pt, ph, pw, cfg.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6).reshape(B, cfg.out_dim, F_, Hh, Ww)
        return vid, outs[1]

    def init_weights(self, seed: int = 0, std: float = 0.02):
        WanDiT.init_weights(self, seed, std)
        with torch.no_grad():
            for n, p in self.named_parameters():
                if n.endswith("norm_q_audio.weight") or n.endswith("norm_k_audio.weight"):
                    p.fill_(1.0)
        return self


def remap_nava_keys(sd: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Strip ``backbone.`` and turn every fp8 ``weight`` + per-row ``weight_scale`` pair into one ``dtype`` weight."""
    out = {}
    for k, v in sd.items():
        if not k.startswith("backbone.") or k.endswith(".weight_scale"):
            continue
        n = k[len("backbone."):]
        if v.dtype == torch.float8_e4m3fn:
            v = (v.float() * sd[k + "_scale"].float()[:, None]).to(dtype)
        out[n] = v
    return out
