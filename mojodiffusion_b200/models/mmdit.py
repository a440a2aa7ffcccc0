"""FLUX.1-shaped MMDiT: double-stream + single-stream blocks with per-block adaLN modulation, 3-axis
interleaved RoPE, QK-RMSNorm, GELU-tanh MLPs and biases everywhere.

Architecture facts follow serenitymojo/models/dit/flux1_dit.mojo:7-30,82-95 (19 double + 38 single, D=3072,
24 heads x 128, in 64, ctx 4096, pooled 768, guidance embed, RoPE axes (16,56,56), theta 1e4) and :228-406
(block op order); parameter names are the BFL checkpoint keys listed at :105-128,264-406, so a real
``flux1-dev.safetensors`` loads with ``load_state_dict``.

Two execution styles share the same modules:
* inference (autograd off, CUDA): each linear is ONE tcgen05 GEMM launch with its bias / GELU / gated-residual
  epilogue; the txt and img QKV projections write straight into one joint [B, S_txt+S_img, 3D] buffer that the
  QK-norm+RoPE kernel updates in place and the attention kernel reads through strides (no concat, no permute);
  single-block ``linear2`` consumes [attn | gelu(mlp)] as two K segments of one GEMM.
* training (autograd on, or CPU): the same math as differentiable ops (``ops.functional``).
"""
from __future__ import annotations

import contextlib

import zlib
from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..utils.tracing import nvtx_enabled, nvtx_range
from ..ops import native
from .layers import Linear, MLPEmbedder, timestep_embedding


@dataclass
class MMDiTConfig:
    in_channels: int = 64
    out_channels: Optional[int] = None
    context_dim: int = 4096
    vec_dim: int = 768
    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    depth_double: int = 19
    depth_single: int = 38
    mlp_ratio: float = 4.0
    axes_dim: Tuple[int, ...] = (16, 56, 56)
    theta: float = 10000.0
    guidance_embed: bool = True
    qkv_bias: bool = True
    time_dim: int = 256
    name: str = "flux1-dev"

    @property
    def mlp_hidden(self) -> int:
        return int(self.hidden * self.mlp_ratio)


def flux1_dev_config() -> MMDiTConfig:
    return MMDiTConfig()


def tiny_mmdit_config() -> MMDiTConfig:
    """The CPU plumbing config: hidden 256, 4 heads x 64, 2 double + 2 single, RoPE (16,24,24), text dim 256."""
    return MMDiTConfig(in_channels=64, context_dim=256, vec_dim=256, hidden=256, heads=4, head_dim=64, depth_double=2,
                       depth_single=2, axes_dim=(16, 24, 24), guidance_embed=False, name="tiny-mmdit")


class RMSScale(nn.Module):
    """Holds the ``scale`` vector of a per-head RMSNorm (applied inside the fused QK-norm+RoPE kernel)."""

    def __init__(self, dim: int, dtype, device):
        super().__init__()
        self.scale = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))


class QKNorm(nn.Module):
    def __init__(self, dim: int, dtype, device):
        super().__init__()
        self.query_norm = RMSScale(dim, dtype, device)
        self.key_norm = RMSScale(dim, dtype, device)


class SelfAttentionParams(nn.Module):
    def __init__(self, cfg: MMDiTConfig, dtype, device):
        super().__init__()
        D = cfg.hidden
        self.qkv = Linear(D, 3 * D, cfg.qkv_bias, dtype, device)
        self.norm = QKNorm(cfg.head_dim, dtype, device)
        self.proj = Linear(D, D, True, dtype, device)


class Modulation(nn.Module):
    def __init__(self, dim: int, n: int, dtype, device):
        super().__init__()
        self.n = n
        self.lin = Linear(dim, n * dim, True, dtype, device)

    def forward(self, vec_silu: torch.Tensor):
        return self.lin(vec_silu)  # [B, n*D]; callers slice views (shift, scale, gate) x (n/3)


def _mlp(cfg: MMDiTConfig, dtype, device) -> nn.ModuleDict:
    return nn.ModuleDict({"0": Linear(cfg.hidden, cfg.mlp_hidden, True, dtype, device),
                          "2": Linear(cfg.mlp_hidden, cfg.hidden, True, dtype, device)})


def _fused_path(x: torch.Tensor) -> bool:
    return native.use_native(x) and not torch.is_grad_enabled()


class DoubleStreamBlock(nn.Module):
    def __init__(self, cfg: MMDiTConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        self.img_mod = Modulation(D, 6, dtype, device)
        self.img_attn = SelfAttentionParams(cfg, dtype, device)
        self.img_mlp = _mlp(cfg, dtype, device)
        self.txt_mod = Modulation(D, 6, dtype, device)
        self.txt_attn = SelfAttentionParams(cfg, dtype, device)
        self.txt_mlp = _mlp(cfg, dtype, device)

    def forward(self, img, txt, vec_silu, cos, sin, sp=None):
        cfg = self.cfg
        B, S_img, D = img.shape
        S_txt = txt.shape[1]
        S = S_txt + S_img
        H, Dh = cfg.heads, cfg.head_dim
        mi = self.img_mod(vec_silu)
        mt = self.txt_mod(vec_silu)
        i_shift1, i_scale1, i_gate1, i_shift2, i_scale2, i_gate2 = [mi[:, j * D:(j + 1) * D] for j in range(6)]
        t_shift1, t_scale1, t_gate1, t_shift2, t_scale2, t_gate2 = [mt[:, j * D:(j + 1) * D] for j in range(6)]
        img_n = ops.norm_modulate(img, scale=i_scale1, shift=i_shift1, eps=1e-6)
        txt_n = ops.norm_modulate(txt, scale=t_scale1, shift=t_shift1, eps=1e-6)
        wqi, wki = self.img_attn.norm.query_norm.scale, self.img_attn.norm.key_norm.scale
        wqt, wkt = self.txt_attn.norm.query_norm.scale, self.txt_attn.norm.key_norm.scale
        if sp is not None:
            # sequence parallel: the projections scatter heads to their owners, attention returns this rank's rows
            sp.scatter_qkv(txt_n, self.txt_attn.qkv.weight, self.txt_attn.qkv.bias, "txt")
            sp.scatter_qkv(img_n, self.img_attn.qkv.weight, self.img_attn.qkv.bias, "img")
            sp.finish_scatter()
            sp.attention(wqt, wkt, wqi, wki, cos, sin)
            attn = sp.finish_attention()
            qkv = None
        elif _fused_path(img):
            qkv = torch.empty(B, S, 3 * D, dtype=img.dtype, device=img.device)
            for b in range(B):
                self.txt_attn.qkv(txt_n[b], out=qkv[b, :S_txt])
                self.img_attn.qkv(img_n[b], out=qkv[b, S_txt:])
            ops.qk_norm_rope(qkv[:, :S_txt], H, Dh, wqt, wkt, cos, sin, pos_offset=0)
            ops.qk_norm_rope(qkv[:, S_txt:], H, Dh, wqi, wki, cos, sin, pos_offset=S_txt)
        else:
            # training path: one packed projection buffer, norm/rope + attention as a single autograd node
            qkv = torch.cat((self.txt_attn.qkv(txt_n), self.img_attn.qkv(img_n)), dim=1)
            attn = ops.qkv_attention(qkv, H, Dh, wqi, wki, cos, sin, split=S_txt, wq_first=wqt, wk_first=wkt)
            qkv = None
        if qkv is not None:
            q = qkv[..., 0:D].unflatten(-1, (H, Dh))
            k = qkv[..., D:2 * D].unflatten(-1, (H, Dh))
            v = qkv[..., 2 * D:3 * D].unflatten(-1, (H, Dh))
            attn = ops.attention(q, k, v).reshape(B, S, D)
        txt_a, img_a = attn[:, :S_txt], attn[:, S_txt:]
        img = self.img_attn.proj(img_a, residual=img, gate=i_gate1, rows_per_group=S_img)
        txt = self.txt_attn.proj(txt_a, residual=txt, gate=t_gate1, rows_per_group=S_txt)
        h = self.img_mlp["0"](ops.norm_modulate(img, scale=i_scale2, shift=i_shift2, eps=1e-6), act="gelu_tanh")
        img = self.img_mlp["2"](h, residual=img, gate=i_gate2, rows_per_group=S_img)
        h = self.txt_mlp["0"](ops.norm_modulate(txt, scale=t_scale2, shift=t_shift2, eps=1e-6), act="gelu_tanh")
        txt = self.txt_mlp["2"](h, residual=txt, gate=t_gate2, rows_per_group=S_txt)
        return img, txt


class SingleStreamBlock(nn.Module):
    def __init__(self, cfg: MMDiTConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        D, F_ = cfg.hidden, cfg.mlp_hidden
        self.linear1 = Linear(D, 3 * D + F_, True, dtype, device)
        self.linear2 = Linear(D + F_, D, True, dtype, device)
        self.norm = QKNorm(cfg.head_dim, dtype, device)
        self.modulation = Modulation(D, 3, dtype, device)

    def forward(self, x, vec_silu, cos, sin, sp=None):
        cfg = self.cfg
        B, S, D = x.shape
        H, Dh, F_ = cfg.heads, cfg.head_dim, cfg.mlp_hidden
        m = self.modulation(vec_silu)
        shift, scale, gate = m[:, 0:D], m[:, D:2 * D], m[:, 2 * D:3 * D]
        xn = ops.norm_modulate(x, scale=scale, shift=shift, eps=1e-6)
        wq, wk = self.norm.query_norm.scale, self.norm.key_norm.scale
        fused = _fused_path(x) and len(self.linear1.slots) == 0 and len(self.linear2.slots) == 0
        if sp is not None:
            w1, b1, w2 = self.linear1.weight, self.linear1.bias, self.linear2.weight
            bq = b1[:3 * D] if b1 is not None else None
            sp.scatter_qkv_joint(xn, w1[:3 * D], bq)
            mlp = ops.linear(xn, w1[3 * D:], b1[3 * D:] if b1 is not None else None, act="gelu_tanh")
            sp.finish_scatter()
            sp.attention(wq, wk, wq, wk, cos, sin)
            attn = sp.finish_attention()
            return ops.linear(attn, w2[:, :D], self.linear2.bias, residual=x, gate=gate, rows_per_group=S,
                              extra=[(mlp, w2[:, D:])])
        if fused:
            w1, b1 = self.linear1.weight, self.linear1.bias
            qkv = ops.linear(xn, w1[:3 * D], b1[:3 * D] if b1 is not None else None)
            mlp = ops.linear(xn, w1[3 * D:], b1[3 * D:] if b1 is not None else None, act="gelu_tanh")
            ops.qk_norm_rope(qkv, H, Dh, wq, wk, cos, sin)
        else:
            # training path: attention and the activated MLP half land in one buffer, as one autograd node
            mid = ops.packed_attention_mlp(self.linear1(xn), H, Dh, wq, wk, cos, sin, act="gelu_tanh")
            return self.linear2(mid, residual=x, gate=gate, rows_per_group=S)
        q = qkv[..., 0:D].unflatten(-1, (H, Dh))
        k = qkv[..., D:2 * D].unflatten(-1, (H, Dh))
        v = qkv[..., 2 * D:3 * D].unflatten(-1, (H, Dh))
        attn = ops.attention(q, k, v).reshape(B, S, D)
        if fused:
            w2 = self.linear2.weight
            return ops.linear(attn, w2[:, :D], self.linear2.bias, residual=x, gate=gate, rows_per_group=S,
                              extra=[(mlp, w2[:, D:])])
        return self.linear2(torch.cat((attn, mlp), dim=-1), residual=x, gate=gate, rows_per_group=S)


class LastLayer(nn.Module):
    def __init__(self, hidden: int, out_channels: int, dtype, device):
        super().__init__()
        self.linear = Linear(hidden, out_channels, True, dtype, device)
        self.adaLN_modulation = nn.ModuleDict({"1": Linear(hidden, 2 * hidden, True, dtype, device)})

    def forward(self, x, vec_silu):
        D = x.shape[-1]
        m = self.adaLN_modulation["1"](vec_silu)
        shift, scale = m[:, :D], m[:, D:]
        return self.linear(ops.norm_modulate(x, scale=scale, shift=shift, eps=1e-6))


_NULL = contextlib.nullcontext()


class MMDiT(nn.Module):
    """FLUX-style double + single stream diffusion transformer predicting the rectified-flow velocity."""

    def __init__(self, cfg: MMDiTConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D = cfg.hidden
        assert cfg.heads * cfg.head_dim == D and sum(cfg.axes_dim) == cfg.head_dim
        self.img_in = Linear(cfg.in_channels, D, True, dtype, device)
        self.time_in = MLPEmbedder(cfg.time_dim, D, dtype, device)
        self.vector_in = MLPEmbedder(cfg.vec_dim, D, dtype, device)
        if cfg.guidance_embed:
            self.guidance_in = MLPEmbedder(cfg.time_dim, D, dtype, device)
        self.txt_in = Linear(cfg.context_dim, D, True, dtype, device)
        self.double_blocks = nn.ModuleList([DoubleStreamBlock(cfg, dtype, device) for _ in range(cfg.depth_double)])
        self.single_blocks = nn.ModuleList([SingleStreamBlock(cfg, dtype, device) for _ in range(cfg.depth_single)])
        self.final_layer = LastLayer(D, cfg.out_channels or cfg.in_channels, dtype, device)
        self.gradient_checkpointing = False
        self.streamer = None          # offload.StreamedStack over double + single blocks (block-swap weights)
        self._rope_cache = {}

    # ---- positions ---------------------------------------------------------------------------
    @staticmethod
    def make_ids(h: int, w: int, n_txt: int, device=None) -> torch.Tensor:
        """Joint position ids [n_txt + h*w, 3]: text tokens (0,0,0), image token (0,row,col)
        (serenitymojo/models/dit/flux1_dit.mojo:480-550)."""
        ids = torch.zeros(n_txt + h * w, 3, dtype=torch.float32, device=device)
        rows = torch.arange(h, device=device, dtype=torch.float32)[:, None].expand(h, w).reshape(-1)
        cols = torch.arange(w, device=device, dtype=torch.float32)[None, :].expand(h, w).reshape(-1)
        ids[n_txt:, 1] = rows
        ids[n_txt:, 2] = cols
        return ids

    def rope(self, ids: torch.Tensor):
        key = (ids.data_ptr(), tuple(ids.shape), str(ids.device))
        hit = self._rope_cache.get(key)
        if hit is None:
            hit = ops.rope_table(ids, self.cfg.axes_dim, self.cfg.theta)
            self._rope_cache = {key: hit}
        return hit

    # ---- conditioning vector ---------------------------------------------------------------------
    def embed_vec(self, timesteps, y, guidance=None):
        dt = self.img_in.weight.dtype
        vec = self.time_in(timestep_embedding(timesteps, self.cfg.time_dim).to(dt))
        if self.cfg.guidance_embed:
            g = guidance if guidance is not None else torch.ones_like(timesteps)
            vec = vec + self.guidance_in(timestep_embedding(g, self.cfg.time_dim).to(dt))
        vec = vec + self.vector_in(y.to(dt))
        return vec

    def forward(self, img, txt, timesteps, y, guidance=None, ids: Optional[torch.Tensor] = None,
                hw: Optional[Tuple[int, int]] = None, sp=None):
        """img: [B, S_img, in_channels] packed latents, txt: [B, S_txt, context_dim], timesteps/guidance: [B] in
        [0, 1] (scaled by 1000 inside), y: [B, vec_dim]. ``ids`` [S_txt+S_img, 3] or ``hw`` latent grid."""
        cfg = self.cfg
        S_txt, S_img = txt.shape[1], img.shape[1]
        if sp is not None:
            # sequence parallel (inference): img / txt are this rank's token shards, ids cover the global sequence
            assert not torch.is_grad_enabled() and ids is not None and ids.shape[0] == sp.S
        if ids is None:
            if hw is None:
                side = int(round(S_img ** 0.5))
                hw = (side, S_img // side)
            ids = self.make_ids(hw[0], hw[1], S_txt, img.device)
        cos, sin = self.rope(ids)
        dt = self.img_in.weight.dtype
        img = self.img_in(img.to(dt))
        txt = self.txt_in(txt.to(dt))
        vec = self.embed_vec(timesteps, y, guidance)
        vec_silu = ops.activation(vec, "silu")
        ckpt = self.gradient_checkpointing and torch.is_grad_enabled()
        st = self.streamer
        if st is not None:
            # streamed weights: block i's parameters are views of a device slot while it runs; under autograd each
            # block is a recompute boundary (serenitymojo/models/flux/flux_stack_lora.mojo:1619-2019)
            nd = len(self.double_blocks)
            for i in range(nd):
                img, txt = st.step(i, lambda b, im, tx, v: b(im, tx, v, cos, sin, sp), img, txt, vec_silu)
            x = torch.cat((txt, img), dim=1)
            for i in range(len(self.single_blocks)):
                x = st.step(nd + i, lambda b, h, v: b(h, v, cos, sin, sp), x, vec_silu)
            return self.final_layer(x[:, S_txt:], vec_silu)
        trace = nvtx_enabled()
        for i, blk in enumerate(self.double_blocks):
            with nvtx_range(f"block/double/{i}") if trace else _NULL:
                if ckpt:
                    img, txt = torch.utils.checkpoint.checkpoint(blk, img, txt, vec_silu, cos, sin, use_reentrant=False, preserve_rng_state=False)
                else:
                    img, txt = blk(img, txt, vec_silu, cos, sin, sp)
        x = torch.cat((txt, img), dim=1)
        for i, blk in enumerate(self.single_blocks):
            with nvtx_range(f"block/single/{i}") if trace else _NULL:
                if ckpt:
                    x = torch.utils.checkpoint.checkpoint(blk, x, vec_silu, cos, sin, use_reentrant=False, preserve_rng_state=False)
                else:
                    x = blk(x, vec_silu, cos, sin, sp)
        x = x[:, S_txt:]
        return self.final_layer(x, vec_silu)

    def enable_block_swap(self, device, resident_budget_bytes: int = 0, slot_count: int = 2, pin: bool = True):
        """Moves the transformer blocks' weights into a pinned host store and streams them through ``slot_count``
        device slots; the first blocks that fit ``resident_budget_bytes`` stay on the device. Adapter parameters
        (the ``slots`` of a linear) stay with the module. Returns the loader (telemetry lives there)."""
        from ..offload import BlockSwapLoader, OffloadConfig, PinnedBlockStore, StreamedStack
        from ..offload.plan import flux_plan
        plan = flux_plan(len(self.double_blocks), len(self.single_blocks), OffloadConfig(slot_count, min(1, slot_count - 1)))
        blocks = list(self.double_blocks) + list(self.single_blocks)
        tensors = {}
        for spec, blk in zip(plan.blocks, blocks):
            for n, p in blk.named_parameters():
                if ".slots." not in n:
                    tensors[spec.prefix + n] = p.detach()
        loader = BlockSwapLoader(PinnedBlockStore(plan, tensors, pin=pin), device)
        if resident_budget_bytes > 0:
            loader.pin_residents(resident_budget_bytes)
        self.streamer = StreamedStack(blocks, loader)
        self.streamer.detach_weights()
        return loader

    # ---- initialisation ------------------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: int = 0, std: float = 0.02):
        """Deterministic random init (normal, std 0.02; biases zero; norm scales one) from a CPU generator."""
        g = torch.Generator().manual_seed(seed)
        for name, p in self.named_parameters():
            if name.endswith(".scale"):
                p.fill_(1.0)
            elif name.endswith(".bias"):
                p.zero_()
            elif p.dim() >= 2:
                if p.device.type == "cuda" and p.numel() > (1 << 22):
                    p.copy_(ops.randn(tuple(p.shape), seed=seed + zlib.crc32(name.encode()) % 100003, dtype=torch.float32,
                                      device=p.device) * std)
                else:
                    p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
        return self


def pack_latents(z: torch.Tensor, p: int = 2) -> torch.Tensor:
    """[B, C, H, W] -> [B, (H/p)(W/p), C*p*p] with per-token order (c, ph, pw)
    (serenitymojo/pipeline/flux_sample_cli.mojo:134-181)."""
    B, C, H, W = z.shape
    z = z.reshape(B, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5)
    return z.reshape(B, (H // p) * (W // p), C * p * p)


def unpack_latents(x: torch.Tensor, h: int, w: int, p: int = 2) -> torch.Tensor:
    """Inverse of :func:`pack_latents`; h, w are the packed grid (H/p, W/p)."""
    B, _, CPP = x.shape
    C = CPP // (p * p)
    x = x.reshape(B, h, w, C, p, p).permute(0, 3, 1, 4, 2, 5)
    return x.reshape(B, C, h * p, w * p)
