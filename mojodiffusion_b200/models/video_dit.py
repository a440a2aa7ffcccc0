"""LTX-2-shaped video DiT: 48 layers, D=4096, 32 heads x 128, FFN 16384 (GELU-tanh), text cross-attention to a
[256, 4096] context, 3-D split RoPE, QK-RMSNorm over the full inner dim, per-head 2*sigmoid output gates, adaLN from a
learned scale_shift_table plus the timestep embedding. Weights can be served as fp8 (e4m3, per-channel scales).

Facts: serenitymojo/models/dit/ltx2_dit.mojo:135-152 (shape), :518-652 (block op order), ltx2_rope.mojo:1-40 (3-axis
positions), key names :198-291 (`transformer_blocks.{i}.attn1.to_q`, `ff.net.0.proj`, `scale_shift_table` ...), fp8
serving of blocks 4-46 (serenitymojo/offload/ltx2_block_stream.mojo:77-374).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from .layers import Linear, RMSNorm, init_module_weights, packed_projection, timestep_embedding


@dataclass
class VideoDiTConfig:
    in_channels: int = 128
    hidden: int = 4096
    heads: int = 32
    head_dim: int = 128
    depth: int = 48
    context_dim: int = 4096
    ffn_hidden: int = 16384
    axes_dim: Tuple[int, ...] = (32, 48, 48)     # (t, h, w) split of the head dim
    theta: float = 10000.0
    gated_heads: bool = True
    name: str = "ltx2-video"


def ltx2_config() -> VideoDiTConfig:
    return VideoDiTConfig()


def tiny_video_dit_config() -> VideoDiTConfig:
    return VideoDiTConfig(in_channels=32, hidden=256, heads=4, head_dim=64, depth=2, context_dim=128, ffn_hidden=512,
                          axes_dim=(16, 24, 24), name="tiny-video-dit")


class FP8Linear(nn.Module):
    """Linear whose weight is stored as float8_e4m3fn with one fp32 scale per output channel; activations are
    quantised per token on the fly and both scales are applied in the tcgen05 GEMM epilogue."""

    def __init__(self, lin: Linear):
        super().__init__()
        q, s = ops.fp8_quant_rows(lin.weight.detach())
        self.in_features, self.out_features = lin.in_features, lin.out_features
        self.register_buffer("weight", q)
        self.register_buffer("weight_scale", s)
        self.bias = lin.bias
        self.slots = nn.ModuleList()

    def forward(self, x, act=None, residual=None, gate=None, rows_per_group: int = 1, out=None):
        y = ops.fp8_linear(x, self.weight, self.weight_scale, self.bias, act, residual, gate, rows_per_group)
        if out is not None:
            out.copy_(y)
            return out
        return y


class MXFP8Linear(nn.Module):
    """Linear with the weight held in MXFP8 (E4M3 + one E8M0 scale per 32 input features); activations are quantised the
    same way per call and the tensor core applies both block scales (``ops.gemm_mxfp8``). Activation, residual and gate
    run as the usual separate kernels after the GEMM."""

    def __init__(self, lin: Linear):
        super().__init__()
        self.in_features, self.out_features = lin.in_features, lin.out_features
        w = ops.MXFP8Weight(lin.weight.detach(), lin.bias.detach() if lin.bias is not None else None)
        self.register_buffer("weight", w.q)
        self.register_buffer("weight_scale", w.sf)
        self.bias = lin.bias
        self.slots = nn.ModuleList()

    def forward(self, x, act=None, residual=None, gate=None, rows_per_group: int = 1, out=None):
        x2 = x.reshape(-1, self.in_features).to(torch.bfloat16).contiguous()
        aq, asf = ops.mxfp8_quant_rows(x2, 128)
        b = self.bias.to(torch.bfloat16) if self.bias is not None else None
        y = ops.gemm_mxfp8(aq, asf, self.weight, self.weight_scale, b).reshape(*x.shape[:-1], self.out_features).to(x.dtype)
        if act:
            y = ops.activation(y, act)
        if residual is not None:
            y = ops.gate_residual(residual, y, gate, rows_per_group)
        if out is not None:
            out.copy_(y)
            return out
        return y


class VideoAttention(nn.Module):
    def __init__(self, cfg: VideoDiTConfig, cross: bool, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.cfg, self.cross = cfg, cross
        self.to_q = Linear(D, D, True, dtype, device)
        self.to_k = Linear(cfg.context_dim if cross else D, D, True, dtype, device)
        self.to_v = Linear(cfg.context_dim if cross else D, D, True, dtype, device)
        self.to_out = nn.ModuleList([Linear(D, D, True, dtype, device)])
        self.q_norm = RMSNorm(D, 1e-6, dtype, device)
        self.k_norm = RMSNorm(D, 1e-6, dtype, device)
        if cfg.gated_heads and not cross:
            self.to_gate_logits = Linear(D, cfg.heads, True, dtype, device)

    def forward(self, x, context=None, cos=None, sin=None, kv_len=None):
        cfg = self.cfg
        B, S, D = x.shape
        H, Dh = cfg.heads, cfg.head_dim
        if not self.cross:
            qkv = packed_projection(x, (self.to_q, self.to_k, self.to_v))
            q = self.q_norm(qkv[..., 0:D])
            k = self.k_norm(qkv[..., D:2 * D])
            qk = torch.cat((q, k), dim=-1) if (torch.is_grad_enabled() or not x.is_cuda) else None
            if qk is None:
                qkv[..., 0:D] = q
                qkv[..., D:2 * D] = k
                qk = qkv
            qk = ops.qk_norm_rope(qk, H, Dh, None, None, cos, sin, interleaved=False, do_norm=False)
            q = qk[..., 0:D].unflatten(-1, (H, Dh))
            k = qk[..., D:2 * D].unflatten(-1, (H, Dh))
            v = qkv[..., 2 * D:3 * D].unflatten(-1, (H, Dh))
        else:
            q = self.q_norm(self.to_q(x)).unflatten(-1, (H, Dh))
            kv = packed_projection(context, (self.to_k, self.to_v))
            k = self.k_norm(kv[..., 0:D]).unflatten(-1, (H, Dh))
            v = kv[..., D:2 * D].unflatten(-1, (H, Dh))
        o = ops.attention(q, k, v, kv_len=kv_len)
        if hasattr(self, "to_gate_logits"):
            g = 2.0 * torch.sigmoid(self.to_gate_logits(x).float())
            o = (o.float() * g[..., None]).to(x.dtype)
        return o.reshape(B, S, D)


class VideoFF(nn.Module):
    def __init__(self, cfg: VideoDiTConfig, dtype, device):
        super().__init__()
        proj = nn.Module()
        proj.proj = Linear(cfg.hidden, cfg.ffn_hidden, True, dtype, device)
        self.net = nn.ModuleDict({"0": proj, "2": Linear(cfg.ffn_hidden, cfg.hidden, True, dtype, device)})

    def forward(self, x, residual, gate, rows):
        return self.net["2"](self.net["0"].proj(x, act="gelu_tanh"), residual=residual, gate=gate, rows_per_group=rows)


class VideoBlock(nn.Module):
    def __init__(self, cfg: VideoDiTConfig, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.attn1 = VideoAttention(cfg, False, dtype, device)
        self.attn2 = VideoAttention(cfg, True, dtype, device)
        self.ff = VideoFF(cfg, dtype, device)
        self.scale_shift_table = nn.Parameter(torch.zeros(6, D, dtype=dtype, device=device))

    def forward(self, x, context, temb6, cos, sin, ctx_len=None):
        B, S, D = x.shape
        m = (self.scale_shift_table[None].float() + temb6.float()).to(x.dtype)       # [B, 6, D]
        sh1, sc1, g1, sh2, sc2, g2 = [m[:, i] for i in range(6)]
        h = self.attn1(ops.norm_modulate(x, scale=sc1, shift=sh1, eps=1e-6, rms=True), None, cos, sin)
        x = self.attn1.to_out[0](h, residual=x, gate=g1, rows_per_group=S)
        h = self.attn2(ops.norm_modulate(x, eps=1e-6, rms=True), context, kv_len=ctx_len)
        x = self.attn2.to_out[0](h, residual=x)
        return self.ff(ops.norm_modulate(x, scale=sc2, shift=sh2, eps=1e-6, rms=True), x, g2, S)


class VideoDiT(nn.Module):
    """forward(latent tokens [B, S, 128], context [B, 256, 4096], t [B], grid (frames, h, w)) -> velocity [B, S, 128]."""

    def __init__(self, cfg: VideoDiTConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        self.patchify_proj = Linear(cfg.in_channels, D, True, dtype, device)
        emb = nn.Module()
        te = nn.Module()
        te.linear_1 = Linear(256, D, True, dtype, device)
        te.linear_2 = Linear(D, D, True, dtype, device)
        emb.timestep_embedder = te
        ad = nn.Module()
        ad.emb = emb
        ad.linear = Linear(D, 6 * D, True, dtype, device)
        self.adaln_single = ad
        cp = nn.Module()
        cp.linear_1 = Linear(cfg.context_dim, D, True, dtype, device)
        cp.linear_2 = Linear(D, cfg.context_dim, True, dtype, device)
        self.caption_projection = cp
        self.transformer_blocks = nn.ModuleList([VideoBlock(cfg, dtype, device) for _ in range(cfg.depth)])
        self.scale_shift_table = nn.Parameter(torch.zeros(2, D, dtype=dtype, device=device))
        self.proj_out = Linear(D, cfg.in_channels, True, dtype, device)
        self.gradient_checkpointing = False

    @staticmethod
    def make_ids(frames: int, h: int, w: int, device=None) -> torch.Tensor:
        t = torch.arange(frames, device=device, dtype=torch.float32)[:, None, None].expand(frames, h, w)
        y = torch.arange(h, device=device, dtype=torch.float32)[None, :, None].expand(frames, h, w)
        x = torch.arange(w, device=device, dtype=torch.float32)[None, None, :].expand(frames, h, w)
        return torch.stack((t, y, x), -1).reshape(-1, 3)

    def to_fp8(self, first: int = 0, last: Optional[int] = None, block_scaled: bool = False) -> "VideoDiT":
        """Replace the big linears of blocks [first, last) by fp8-resident weights (the reference serves blocks 4-46 so).
        ``block_scaled``: MXFP8 (one scale per 32 input features, applied by the tensor core) instead of one scale per
        output channel."""
        FP8 = MXFP8Linear if block_scaled else FP8Linear
        last = len(self.transformer_blocks) if last is None else last
        for blk in self.transformer_blocks[first:last]:
            for att in (blk.attn1, blk.attn2):
                for n in ("to_q", "to_k", "to_v"):
                    setattr(att, n, FP8(getattr(att, n)))
                att.to_out[0] = FP8(att.to_out[0])
            blk.ff.net["0"].proj = FP8(blk.ff.net["0"].proj)
            blk.ff.net["2"] = FP8(blk.ff.net["2"])
        return self

    def forward(self, x, context, t, grid: Tuple[int, int, int], ctx_len: Optional[torch.Tensor] = None):
        cfg = self.cfg
        D = cfg.hidden
        dt = self.patchify_proj.weight.dtype
        B = x.shape[0]
        cos, sin = ops.rope_table(self.make_ids(*grid, device=x.device), cfg.axes_dim, cfg.theta)
        te = self.adaln_single.emb.timestep_embedder
        emb = te.linear_2(te.linear_1(timestep_embedding(t, 256).to(dt), act="silu"))       # embedded timestep
        temb6 = self.adaln_single.linear(ops.activation(emb, "silu")).reshape(B, 6, D)
        h = self.patchify_proj(x.to(dt))
        cp = self.caption_projection
        ctx = cp.linear_2(cp.linear_1(context.to(dt), act="gelu_tanh"))
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        for blk in self.transformer_blocks:
            if ckpt:
                h = torch.utils.checkpoint.checkpoint(blk, h, ctx, temb6, cos, sin, ctx_len, use_reentrant=False, preserve_rng_state=False)
            else:
                h = blk(h, ctx, temb6, cos, sin, ctx_len)
        m = (self.scale_shift_table[None].float() + emb[:, None].float()).to(h.dtype)
        return self.proj_out(ops.norm_modulate(h, scale=m[:, 1], shift=m[:, 0], eps=1e-6))

    def init_weights(self, seed: int = 0, std: float = 0.02):
        return init_module_weights(self, seed, std)
