"""LTX-2 joint audio / video transformer: the AV block (video and audio streams with their own self-attention, text
cross-attention and feed-forward, plus audio->video and video->audio cross-modal attention), the 1-D embeddings connector
that projects the cached text hidden states into the video (4096) and audio (2048) contexts, and normalised attention
guidance (NAG) on the text cross-attention.

Block order and tables (serenitymojo/models/ltx2/ltx2_av_block.mojo:1-120, serenitymojo/models/dit/ltx2_dit.mojo:1384-1585):
  1. video self-attn   : rows 0:3 of ``scale_shift_table`` [9, Dv] + timestep embedding -> RMS(no affine) -> modulate ->
                         q/k/v -> QK-RMSNorm over the inner dim -> split RoPE -> attention -> per-head 2*sigmoid gate -> out
                         -> gated residual
     audio self-attn   : the same with the ``audio_*`` weights (Da = 2048, 32 heads x 64, 1-D RoPE over time)
  2. text cross-attn   : rows 6:9 modulate the query side, ``prompt_scale_shift_table`` [2, D] modulates the text keys /
                         values, no RoPE, per-head gate, gated residual (video then audio)
  3. cross-modal       : both streams RMS-normalised once; ``scale_shift_table_a2v_ca_{video,audio}`` [5, D] give
                         (scale, shift) for the a2v and the v2a use of each stream and the output gate; a2v: Q = video,
                         K/V = audio; v2a: Q = audio, K/V = video; heads 32 x 64 (the audio head shape) with RoPE over time
  4. feed-forward      : rows 3:6 -> RMS -> modulate -> GELU MLP -> clamp(+-60000) -> gated residual (video then audio)
Connector (serenitymojo/models/dit/ltx2_connector.mojo:1-60): blocks ``x += attn(rms(x)); x += ff(rms(x))`` with gated
self-attention and 1-D split RoPE over the token index, final RMS. NAG (serenitymojo/models/dit/ltx2_nag.mojo,
serenitymojo/sampling/ltx2_guidance.mojo): the cross-attention output for the positive and for the negative context are
extrapolated, norm-clipped against the positive branch and blended.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..sampling.guidance import nag_attention_guidance
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class LTX2AVConfig:
    in_channels: int = 128            # video latent channels per token
    audio_in_channels: int = 128      # audio latent channels per token (8 channels x 16 mel bins)
    hidden: int = 4096
    heads: int = 32
    head_dim: int = 128
    audio_hidden: int = 2048
    audio_heads: int = 32
    audio_head_dim: int = 64
    depth: int = 48
    context_dim: int = 4096           # pre-connector text hidden size
    ffn_hidden: int = 16384
    audio_ffn_hidden: int = 8192
    axes_dim: Tuple[int, ...] = (32, 48, 48)
    theta: float = 10000.0
    connector_depth: int = 2
    connector_max_pos: int = 4096
    ff_clamp: float = 60000.0
    name: str = "ltx2-av"


def ltx2_av_config() -> LTX2AVConfig:
    return LTX2AVConfig()


def tiny_ltx2_av_config() -> LTX2AVConfig:
    return LTX2AVConfig(in_channels=32, audio_in_channels=16, hidden=256, heads=4, head_dim=64, audio_hidden=128, audio_heads=4,
                        audio_head_dim=32, depth=2, context_dim=96, ffn_hidden=512, audio_ffn_hidden=256, axes_dim=(16, 24, 24),
                        connector_depth=1, connector_max_pos=64, name="tiny-ltx2-av")


def _rope_1d(positions: torch.Tensor, dim: int, theta: float):
    """cos / sin [S, dim/2] for half-split rotation over one axis (audio time, connector token index)."""
    half = dim // 2
    freqs = theta ** (-torch.arange(half, dtype=torch.float32, device=positions.device) / max(half, 1))
    ang = positions.float()[:, None] * freqs[None]
    return torch.cos(ang), torch.sin(ang)


def _apply_rope_halfsplit(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [B, S, H, Dh]; rotates pairs (i, i + Dh/2) by the per-token table [S, Dh/2]."""
    Dh = x.shape[-1]
    a, b = x[..., :Dh // 2].float(), x[..., Dh // 2:].float()
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    return torch.cat((a * c - b * s, a * s + b * c), dim=-1).to(x.dtype)


class AVAttention(nn.Module):
    """One attention of the AV block. ``q_dim``: width of the query stream; ``kv_dim``: width of the key / value source;
    ``inner = heads * head_dim`` may differ from both (cross-modal attention runs in the audio head shape)."""

    def __init__(self, q_dim: int, kv_dim: int, heads: int, head_dim: int, dtype, device, gated: bool = True):
        super().__init__()
        inner = heads * head_dim
        self.heads, self.head_dim, self.inner = heads, head_dim, inner
        self.to_q = Linear(q_dim, inner, True, dtype, device)
        self.to_k = Linear(kv_dim, inner, True, dtype, device)
        self.to_v = Linear(kv_dim, inner, True, dtype, device)
        self.to_out = nn.ModuleList([Linear(inner, q_dim, True, dtype, device)])
        self.q_norm = RMSNorm(inner, 1e-6, dtype, device)
        self.k_norm = RMSNorm(inner, 1e-6, dtype, device)
        if gated:
            self.to_gate_logits = Linear(q_dim, heads, True, dtype, device)

    def heads_out(self, x, kv, q_rope=None, k_rope=None, kv_len=None) -> torch.Tensor:
        """Attention output before the output projection, [B, Sq, inner], per-head gate applied."""
        B, Sq, _ = x.shape
        H, Dh = self.heads, self.head_dim
        q = self.q_norm(self.to_q(x)).unflatten(-1, (H, Dh))
        if kv is x:
            kvp = packed_projection(kv, (self.to_k, self.to_v))
            k, v = kvp[..., :self.inner], kvp[..., self.inner:]
        else:
            k, v = self.to_k(kv), self.to_v(kv)
        k = self.k_norm(k).unflatten(-1, (H, Dh))
        v = v.unflatten(-1, (H, Dh))
        if q_rope is not None:
            q = _apply_rope_halfsplit(q, *q_rope)
        if k_rope is not None:
            k = _apply_rope_halfsplit(k, *k_rope)
        o = ops.attention(q.contiguous(), k.contiguous(), v.contiguous(), kv_len=kv_len)
        if hasattr(self, "to_gate_logits"):
            g = 2.0 * torch.sigmoid(self.to_gate_logits(x).float())
            o = (o.float() * g[..., None]).to(x.dtype)
        return o.reshape(B, Sq, self.inner)


class _FF(nn.Module):
    def __init__(self, dim, hidden, dtype, device):
        super().__init__()
        proj = nn.Module()
        proj.proj = Linear(dim, hidden, True, dtype, device)
        self.net = nn.ModuleDict({"0": proj, "2": Linear(hidden, dim, True, dtype, device)})

    def forward(self, x, clamp: float = 0.0):
        y = self.net["2"](self.net["0"].proj(x, act="gelu_tanh"))
        return y.clamp(-clamp, clamp) if clamp > 0 else y


def _rows(table: torch.Tensor, temb: torch.Tensor, lo: int, hi: int):
    """adaLN rows ``table[lo:hi] + temb[:, lo:hi]`` -> list of [B, D] (fp32 sum, model dtype out)."""
    m = (table[None, lo:hi].float() + temb[:, lo:hi].float()).to(temb.dtype)
    return [m[:, i] for i in range(hi - lo)]


def _mod(x, scale, shift):
    return ops.norm_modulate(x, scale=scale, shift=shift, eps=1e-6, rms=True)


def _gated(x, gate, y):
    return x + gate[:, None].to(x.dtype) * y


class LTX2AVBlock(nn.Module):
    def __init__(self, cfg: LTX2AVConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        Dv, Da = cfg.hidden, cfg.audio_hidden
        H, Dh, Ha, Dha = cfg.heads, cfg.head_dim, cfg.audio_heads, cfg.audio_head_dim
        self.attn1 = AVAttention(Dv, Dv, H, Dh, dtype, device)
        self.attn2 = AVAttention(Dv, Dv, H, Dh, dtype, device)
        self.ff = _FF(Dv, cfg.ffn_hidden, dtype, device)
        self.audio_attn1 = AVAttention(Da, Da, Ha, Dha, dtype, device)
        self.audio_attn2 = AVAttention(Da, Da, Ha, Dha, dtype, device)
        self.audio_ff = _FF(Da, cfg.audio_ffn_hidden, dtype, device)
        self.audio_to_video_attn = AVAttention(Dv, Da, Ha, Dha, dtype, device, gated=False)
        self.video_to_audio_attn = AVAttention(Da, Dv, Ha, Dha, dtype, device, gated=False)
        z = lambda r, d: nn.Parameter(torch.zeros(r, d, dtype=dtype, device=device))
        self.scale_shift_table, self.audio_scale_shift_table = z(9, Dv), z(9, Da)
        self.prompt_scale_shift_table, self.audio_prompt_scale_shift_table = z(2, Dv), z(2, Da)
        self.scale_shift_table_a2v_ca_video, self.scale_shift_table_a2v_ca_audio = z(5, Dv), z(5, Da)

    def _text_cross(self, att: AVAttention, x, ctx, table, temb, prompt_table, prompt_ts, ctx_len, nag):
        sh, sc, g = _rows(table, temb, 6, 9)
        xq = _mod(x, sc, sh)
        pk = (prompt_table[None].float() + prompt_ts.float()).to(ctx.dtype)            # [B, 2, D]: (shift_kv, scale_kv)
        kv = (ctx.float() * (1.0 + pk[:, 1:2].float()) + pk[:, 0:1].float()).to(ctx.dtype)
        o = att.heads_out(xq, kv, kv_len=ctx_len)
        if nag is not None:
            ctx_neg, scale, tau, alpha = nag
            kvn = (ctx_neg.float() * (1.0 + pk[:, 1:2].float()) + pk[:, 0:1].float()).to(ctx.dtype)
            o = nag_attention_guidance(o, att.heads_out(xq, kvn), scale, tau, alpha).to(o.dtype)
        return _gated(x, g, att.to_out[0](o))

    def forward(self, vx, ax, v_ctx, a_ctx, v_temb, a_temb, v_prompt_ts, a_prompt_ts, ca_v, ca_a, v_rope, a_rope, cm_v_rope,
                cm_a_rope, ctx_len=None, skip_cross_modal: bool = False, nag=None):
        """vx [B,Sv,Dv], ax [B,Sa,Da]; v_temb / a_temb [B,9,D]; ca_v / ca_a [B,5,D] (timestep part of the cross-modal
        tables); *_rope = (cos, sin) tables. ``nag`` = (negative video context, negative audio context, scale, tau, alpha)."""
        cfg = self.cfg
        # 1. self-attention, video then audio
        sh, sc, g = _rows(self.scale_shift_table, v_temb, 0, 3)
        h = _mod(vx, sc, sh)
        vx = _gated(vx, g, self.attn1.to_out[0](self.attn1.heads_out(h, h, v_rope, v_rope)))
        sh, sc, g = _rows(self.audio_scale_shift_table, a_temb, 0, 3)
        h = _mod(ax, sc, sh)
        ax = _gated(ax, g, self.audio_attn1.to_out[0](self.audio_attn1.heads_out(h, h, a_rope, a_rope)))
        # 2. text cross-attention
        nv = (nag[0], nag[2], nag[3], nag[4]) if nag is not None else None
        na = (nag[1], nag[2], nag[3], nag[4]) if nag is not None else None
        vx = self._text_cross(self.attn2, vx, v_ctx, self.scale_shift_table, v_temb, self.prompt_scale_shift_table, v_prompt_ts,
                              ctx_len, nv)
        ax = self._text_cross(self.audio_attn2, ax, a_ctx, self.audio_scale_shift_table, a_temb, self.audio_prompt_scale_shift_table,
                              a_prompt_ts, ctx_len, na)
        # 3. cross-modal attention
        if not skip_cross_modal:
            tv = (self.scale_shift_table_a2v_ca_video[None].float() + ca_v.float()).to(vx.dtype)
            ta = (self.scale_shift_table_a2v_ca_audio[None].float() + ca_a.float()).to(ax.dtype)
            vq = _mod(vx, tv[:, 0], tv[:, 1])                       # video as the a2v query
            ak = _mod(ax, ta[:, 0], ta[:, 1])                       # audio as the a2v key / value
            aq = _mod(ax, ta[:, 2], ta[:, 3])                       # audio as the v2a query
            vk = _mod(vx, tv[:, 2], tv[:, 3])                       # video as the v2a key / value
            a2v = self.audio_to_video_attn
            v2a = self.video_to_audio_attn
            d_v = a2v.to_out[0](a2v.heads_out(vq, ak, cm_v_rope, cm_a_rope))
            d_a = v2a.to_out[0](v2a.heads_out(aq, vk, cm_a_rope, cm_v_rope))
            vx = _gated(vx, tv[:, 4], d_v)
            ax = _gated(ax, ta[:, 4], d_a)
        # 4. feed-forward
        sh, sc, g = _rows(self.scale_shift_table, v_temb, 3, 6)
        vx = _gated(vx, g, self.ff(_mod(vx, sc, sh), cfg.ff_clamp))
        sh, sc, g = _rows(self.audio_scale_shift_table, a_temb, 3, 6)
        ax = _gated(ax, g, self.audio_ff(_mod(ax, sc, sh), cfg.ff_clamp))
        return vx, ax


class ConnectorBlock(nn.Module):
    def __init__(self, dim, heads, head_dim, hidden, dtype, device):
        super().__init__()
        self.attn1 = AVAttention(dim, dim, heads, head_dim, dtype, device)
        self.ff = _FF(dim, hidden, dtype, device)

    def forward(self, x, rope):
        h = ops.norm_modulate(x, eps=1e-6, rms=True)
        x = x + self.attn1.to_out[0](self.attn1.heads_out(h, h, rope, rope))
        return x + self.ff(ops.norm_modulate(x, eps=1e-6, rms=True))


class EmbeddingsConnector(nn.Module):
    """Text hidden states [B, T, context_dim] -> context of one modality [B, T, dim] (takes the place of a caption projection)."""

    def __init__(self, context_dim, dim, heads, head_dim, depth, max_pos, theta, dtype, device):
        super().__init__()
        self.proj_in = Linear(context_dim, dim, True, dtype, device)
        self.transformer_1d_blocks = nn.ModuleList([ConnectorBlock(dim, heads, head_dim, 4 * dim, dtype, device) for _ in range(depth)])
        self.heads, self.head_dim, self.max_pos, self.theta = heads, head_dim, max_pos, theta

    def forward(self, text):
        x = self.proj_in(text.to(self.proj_in.weight.dtype))
        T = x.shape[1]
        pos = 2.0 * torch.arange(T, device=x.device, dtype=torch.float32) / self.max_pos - 1.0      # scaled to [-1, 1)
        half = self.head_dim // 2
        freqs = self.theta ** (torch.arange(half, device=x.device, dtype=torch.float32) / max(half - 1, 1)) * (math.pi / 2)
        ang = pos[:, None] * freqs[None]
        rope = (torch.cos(ang), torch.sin(ang))
        for blk in self.transformer_1d_blocks:
            x = blk(x, rope)
        return ops.norm_modulate(x, eps=1e-6, rms=True)


class _AdaLN(nn.Module):
    def __init__(self, dim, rows, dtype, device):
        super().__init__()
        emb, te = nn.Module(), nn.Module()
        te.linear_1 = Linear(256, dim, True, dtype, device)
        te.linear_2 = Linear(dim, dim, True, dtype, device)
        emb.timestep_embedder = te
        self.emb = emb
        self.linear = Linear(dim, rows * dim, True, dtype, device)
        self.rows, self.dim = rows, dim

    def forward(self, t, dt):
        te = self.emb.timestep_embedder
        e = te.linear_2(te.linear_1(timestep_embedding(t, 256).to(dt), act="silu"))
        return e, self.linear(ops.activation(e, "silu")).reshape(t.shape[0], self.rows, self.dim)


class LTX2AVDiT(nn.Module):
    """forward(video tokens [B,Sv,Cv], audio tokens [B,Sa,Ca], text hidden [B,T,context_dim], t [B], grid (frames,h,w),
    audio_t: optional separate audio timestep) -> (video velocity [B,Sv,Cv], audio velocity [B,Sa,Ca])."""

    def __init__(self, cfg: LTX2AVConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        Dv, Da = cfg.hidden, cfg.audio_hidden
        self.patchify_proj = Linear(cfg.in_channels, Dv, True, dtype, device)
        self.audio_patchify_proj = Linear(cfg.audio_in_channels, Da, True, dtype, device)
        self.adaln_single = _AdaLN(Dv, 9, dtype, device)
        self.audio_adaln_single = _AdaLN(Da, 9, dtype, device)
        self.prompt_adaln_single = _AdaLN(Dv, 2, dtype, device)
        self.audio_prompt_adaln_single = _AdaLN(Da, 2, dtype, device)
        self.av_ca_video_scale_shift_adaln_single = _AdaLN(Dv, 5, dtype, device)
        self.av_ca_audio_scale_shift_adaln_single = _AdaLN(Da, 5, dtype, device)
        self.video_embeddings_connector = EmbeddingsConnector(cfg.context_dim, Dv, cfg.heads, cfg.head_dim, cfg.connector_depth,
                                                              cfg.connector_max_pos, cfg.theta, dtype, device)
        self.audio_embeddings_connector = EmbeddingsConnector(cfg.context_dim, Da, cfg.audio_heads, cfg.audio_head_dim,
                                                              cfg.connector_depth, cfg.connector_max_pos, cfg.theta, dtype, device)
        self.transformer_blocks = nn.ModuleList([LTX2AVBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        z = lambda r, d: nn.Parameter(torch.zeros(r, d, dtype=dtype, device=device))
        self.scale_shift_table, self.audio_scale_shift_table = z(2, Dv), z(2, Da)
        self.proj_out = Linear(Dv, cfg.in_channels, True, dtype, device)
        self.audio_proj_out = Linear(Da, cfg.audio_in_channels, True, dtype, device)
        self.gradient_checkpointing = False

    def contexts(self, text):
        return self.video_embeddings_connector(text), self.audio_embeddings_connector(text)

    def forward(self, vx, ax, text, t, grid: Tuple[int, int, int], audio_t: Optional[torch.Tensor] = None, ctx_len=None,
                skip_cross_modal: bool = False, nag=None, fps: float = 24.0, audio_tokens_per_second: float = 25.0):
        """``nag`` = (negative text hidden [B,T,context_dim], scale, tau, alpha) enables normalised attention guidance."""
        from .video_dit import VideoDiT
        cfg = self.cfg
        dt = self.patchify_proj.weight.dtype
        B, Sa = vx.shape[0], ax.shape[1]
        audio_t = t if audio_t is None else audio_t
        ids = VideoDiT.make_ids(*grid, device=vx.device)
        v_rope = ops.rope_table(ids, cfg.axes_dim, cfg.theta)
        a_time = torch.arange(Sa, device=vx.device, dtype=torch.float32) / audio_tokens_per_second
        a_rope = _rope_1d(a_time * audio_tokens_per_second, cfg.audio_head_dim, cfg.theta)
        # cross-modal rotation: both streams by their time in seconds, in the audio head shape
        v_time = ids[:, 0] * (8.0 / fps)                       # a latent frame spans 8 video frames
        cm_v = _rope_1d(v_time * audio_tokens_per_second, cfg.audio_head_dim, cfg.theta)
        cm_a = a_rope
        v_rope = (v_rope[0], v_rope[1])
        e_v, v_temb = self.adaln_single(t, dt)
        e_a, a_temb = self.audio_adaln_single(audio_t, dt)
        _, v_pts = self.prompt_adaln_single(t, dt)
        _, a_pts = self.audio_prompt_adaln_single(audio_t, dt)
        _, ca_v = self.av_ca_video_scale_shift_adaln_single(t, dt)
        _, ca_a = self.av_ca_audio_scale_shift_adaln_single(audio_t, dt)
        v_ctx, a_ctx = self.contexts(text)
        nag_blk = None
        if nag is not None:
            nv, na = self.contexts(nag[0])
            nag_blk = (nv, na, nag[1], nag[2], nag[3])
        hv = self.patchify_proj(vx.to(dt))
        ha = self.audio_patchify_proj(ax.to(dt))
        vr = self._video_rope(v_rope, hv)
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.transformer_blocks:
            args = (hv, ha, v_ctx, a_ctx, v_temb, a_temb, v_pts, a_pts, ca_v, ca_a, vr, a_rope, cm_v, cm_a, ctx_len, skip_cross_modal, nag_blk)
            if ckpt:
                hv, ha = torch.utils.checkpoint.checkpoint(blk, *args, use_reentrant=False, preserve_rng_state=False)
            else:
                hv, ha = blk(*args)
        mv = (self.scale_shift_table[None].float() + e_v[:, None].float()).to(hv.dtype)
        ma = (self.audio_scale_shift_table[None].float() + e_a[:, None].float()).to(ha.dtype)
        out_v = self.proj_out(ops.norm_modulate(hv, scale=mv[:, 1], shift=mv[:, 0], eps=1e-6))
        out_a = self.audio_proj_out(ops.norm_modulate(ha, scale=ma[:, 1], shift=ma[:, 0], eps=1e-6))
        return out_v, out_a

    def _video_rope(self, tables, hv):
        """The table builder returns [S, Dh/2] cos / sin over the three axes concatenated: used as a half-split rotation."""
        cos, sin = tables
        return cos.float(), sin.float()

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)


def ltx2_av_lora_prefixes(depth: int):
    """Adapter prefixes of the AV model as the reference's LoRA surface names them
    (serenitymojo/training/ltx2/lora_surface.mojo:25-90)."""
    out = []
    for i in range(depth):
        base = f"diffusion_model.transformer_blocks.{i}."
        for att in ("attn1", "attn2", "audio_attn1", "audio_attn2", "audio_to_video_attn", "video_to_audio_attn"):
            out += [base + f"{att}.{p}" for p in ("to_q", "to_k", "to_v", "to_out.0")]
            if att in ("attn1", "attn2", "audio_attn1", "audio_attn2"):
                out.append(base + f"{att}.to_gate_logits")
        out += [base + "ff.net.0.proj", base + "ff.net.2", base + "audio_ff.net.0.proj", base + "audio_ff.net.2"]
    return out
