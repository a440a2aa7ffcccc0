"""Building blocks shared by the backbones: a Linear that runs the tcgen05 GEMM with fused epilogues and can
carry LoRA adapters (whole-weight or per-row-range for fused projections), embedders and small helpers."""
from __future__ import annotations

import math
import zlib
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from .. import ops
from ..ops import native


class LoRASlot(nn.Module):
    """One low-rank adapter ``delta = (alpha / rank) * up @ down`` for rows [row0, row1) of a host weight.

    ``down`` [rank, in] is initialised kaiming-uniform(a=sqrt(5)), ``up`` [rows, rank] with zeros, as in
    serenitymojo/models/flux/flux_stack_lora.mojo:104-121. ``key`` is the checkpoint prefix of the adapter.
    """

    def __init__(self, key: str, in_features: int, rows: Tuple[int, int], rank: int, alpha: float, dtype, device,
                 seed: int = 0):
        super().__init__()
        self.key = key
        self.row0, self.row1 = rows
        self.rank = rank
        self.alpha = float(alpha)
        # kaiming-uniform(a=sqrt(5)) == U(-1/sqrt(in), 1/sqrt(in)); drawn from a generator keyed by (seed, key) so
        # every rank of a data-parallel job builds identical adapters without a broadcast
        gen = torch.Generator().manual_seed((int(seed) * 1000003 + zlib.crc32(key.encode())) & 0x7FFFFFFFFFFF)
        bound = 1.0 / math.sqrt(in_features)
        down = (torch.rand(rank, in_features, generator=gen, dtype=torch.float32) * 2.0 - 1.0) * bound
        self.down = nn.Parameter(down.to(dtype=dtype, device=device))
        self.up = nn.Parameter(torch.zeros(self.row1 - self.row0, rank, dtype=dtype, device=device))

    @property
    def scale(self) -> float:
        return self.alpha / self.rank


class _BlockUp(torch.autograd.Function):
    """[N, R] matrix holding each adapter's scaled up-projection in its (row range, rank column range) block and zeros
    elsewhere: one fill plus one multiply-into-place per adapter, and one multiply per adapter in backward."""

    @staticmethod
    def forward(ctx, n, r, places, *ups):
        ctx.places = places
        out = ups[0].new_zeros(n, r)
        for (r0, r1, c0, c1, sc), u in zip(places, ups):
            torch.mul(u, sc, out=out[r0:r1, c0:c1])
        return out

    @staticmethod
    def backward(ctx, g):
        return (None, None, None) + tuple(g[r0:r1, c0:c1] * sc for (r0, r1, c0, c1, sc) in ctx.places)


class Linear(nn.Module):
    """``y = x W^T + b`` on the tcgen05 GEMM, with optional fused activation / gated residual and LoRA slots."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None
        self.slots = nn.ModuleList()
        self.lora_multiplier = 1.0
        self.reset_parameters()

    def reset_parameters(self, std: Optional[float] = None):
        std = std if std is not None else 1.0 / math.sqrt(self.in_features)
        with torch.no_grad():
            self.weight.normal_(0.0, std)
            if self.bias is not None:
                self.bias.zero_()

    # ---- LoRA -------------------------------------------------------------------------------
    def add_lora(self, key: str, rank: int, alpha: float, rows: Optional[Tuple[int, int]] = None,
                 seed: int = 0) -> LoRASlot:
        rows = rows or (0, self.out_features)
        slot = LoRASlot(key, self.in_features, rows, rank, alpha, self.weight.dtype, self.weight.device, seed)
        self.slots.append(slot)
        return slot

    def _lora_operands(self):
        """(down_cat [sum r, K], up_blk [N, sum r]) with each slot's scale folded into its up block."""
        slots: List[LoRASlot] = list(self.slots)
        if len(slots) == 1 and slots[0].row0 == 0 and slots[0].row1 == self.out_features:
            s = slots[0]
            return s.down, s.up * (s.scale * self.lora_multiplier)
        down = torch.cat([s.down for s in slots], 0)
        R = down.shape[0]
        places, c0 = [], 0
        for s in slots:
            places.append((s.row0, s.row1, c0, c0 + s.rank, s.scale * self.lora_multiplier))
            c0 += s.rank
        up = _BlockUp.apply(self.out_features, R, tuple(places), *[s.up for s in slots])
        return down, up

    # ---- forward ------------------------------------------------------------------------------
    def forward(self, x, act=None, residual=None, gate=None, rows_per_group: int = 1, out=None):
        if len(self.slots) == 0:
            return ops.linear(x, self.weight, self.bias, act, residual, gate, rows_per_group, out=out)
        down, up = self._lora_operands()
        return ops.lora_linear(x, self.weight, self.bias, down, up, 1.0, act, residual, gate, rows_per_group, out)


class MLPEmbedder(nn.Module):
    """Linear -> SiLU -> Linear (timestep / guidance / pooled-vector embedders; serenitymojo/ops/embeddings.mojo:245-297)."""

    def __init__(self, in_dim: int, hidden: int, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.in_layer = Linear(in_dim, hidden, True, dtype, device)
        self.out_layer = Linear(hidden, hidden, True, dtype, device)

    def forward(self, x):
        return self.out_layer(self.in_layer(x, act="silu"))


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0, time_factor: float = 1000.0,
                       cos_first: bool = True) -> torch.Tensor:
    """Sinusoidal embedding [B, dim] (fp32). FLUX uses cos-first with t scaled by 1000
    (serenitymojo/ops/embeddings.mojo:55-111; serenitymojo/models/dit/flux1_dit.mojo:412-457)."""
    t = t.float() * time_factor
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t[:, None] * freqs[None]
    emb = torch.cat([torch.cos(args), torch.sin(args)] if cos_first else [torch.sin(args), torch.cos(args)], dim=-1)
    if dim % 2:
        emb = torch.cat([emb, torch.zeros_like(emb[:, :1])], dim=-1)
    return emb


def model_dtype(m: nn.Module):
    return next(m.parameters()).dtype


def iter_linears(module: nn.Module, prefix: str = ""):
    for name, sub in module.named_modules():
        if isinstance(sub, Linear):
            yield name, sub


class RMSNorm(nn.Module):
    """RMSNorm with a learned weight over the last dim (serenitymojo/ops/norm.mojo:47-230)."""

    def __init__(self, dim: int, eps: float = 1e-6, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device))

    def forward(self, x, scale=None, shift=None, rows_per_group=None):
        return ops.norm_modulate(x, weight=self.weight, scale=scale, shift=shift, rows_per_group=rows_per_group,
                                 eps=self.eps, rms=True)


class LayerNorm(nn.Module):
    """LayerNorm, affine optional (serenitymojo/ops/norm.mojo:318-460,652-782)."""

    def __init__(self, dim: int, eps: float = 1e-6, affine: bool = True, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, dtype=dtype, device=device)) if affine else None
        self.bias = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device)) if affine else None

    def forward(self, x, scale=None, shift=None, rows_per_group=None):
        return ops.norm_modulate(x, weight=self.weight, bias=self.bias, scale=scale, shift=shift,
                                 rows_per_group=rows_per_group, eps=self.eps, rms=False)


def packed_projection(x: torch.Tensor, linears) -> torch.Tensor:
    """Run several Linear modules on the same input and return their outputs side by side in ONE buffer
    ([..., sum(out_features)]): on the GPU inference path each GEMM stores straight into its column slice, so
    separate to_q / to_k / to_v weights (diffusers layout) still give the packed qkv the attention kernels read."""
    widths = [l.out_features for l in linears]
    if native.use_native(x) and not torch.is_grad_enabled():
        lead = x.shape[:-1]
        out = torch.empty(*lead, sum(widths), dtype=x.dtype, device=x.device)
        c = 0
        for l, w in zip(linears, widths):
            l(x, out=out[..., c:c + w])
            c += w
        return out
    return torch.cat([l(x) for l in linears], dim=-1)


@torch.no_grad()
def init_module_weights(module: nn.Module, seed: int = 0, std: float = 0.02) -> nn.Module:
    """Deterministic random init shared by all backbones: normal(0, std) matrices, zero biases, unit norm weights.
    Large tensors are drawn on the device by the Philox kernel, small ones from a CPU generator."""
    g = torch.Generator().manual_seed(seed)
    for name, p in module.named_parameters():
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("scale",) or (leaf == "weight" and p.dim() == 1):
            p.fill_(1.0)
        elif leaf == "bias" or p.dim() == 1:
            p.zero_()
        else:
            if p.device.type == "cuda" and p.numel() > (1 << 22) and p.dtype in (torch.bfloat16, torch.float32):
                p.copy_(ops.randn(tuple(p.shape), seed=seed + zlib.crc32(name.encode()) % 100003, dtype=torch.float32,
                                  device=p.device) * std)
            else:
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
    return module
