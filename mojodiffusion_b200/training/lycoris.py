"""LyCORIS adapter family on top of a frozen linear / conv weight: LoHa, LoKr, LoCon (conv LoRA), Tucker conv,
Diag-OFT, BOFT, DoRA and Full. Every adapter is the identity at initialisation (one zero leaf) and every factor
receives gradient once that leaf has left zero.

Design: each adapter builds the effective weight ``W_eff`` (fp32 factor math under autograd, cast once to the
compute dtype) and the layer runs ONE tcgen05 GEMM with it, so forward and dgrad cost the same as the frozen layer and
the factor gradients come from the dW GEMM of that same layer followed by tiny factor-sized products.

Save keys follow the upstream LyCORIS conventions (no ``.weight`` suffix on hada_*/lokr_*/oft_blocks; ``.alpha`` per
module; ``dora_scale`` fp32) (serenitymojo/training/loha_adapter.mojo:10-45, loha_save.mojo:6, lokr_adapter.mojo:10-60,
lokr_save.mojo:2-30, oft_adapter.mojo:14-60, boft_adapter.mojo:8-60, dora_adapter.mojo:10-70, dora_save.mojo:107-113,
locon_conv_adapter.mojo, tucker_conv_adapter.mojo / tucker_save.mojo:160-166, full_adapter.mojo:6-20)."""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch
from torch import nn

from .. import ops


def factorization(dim: int, factor: int = -1) -> Tuple[int, int]:
    """Split ``dim`` into (m, n), m <= n, m * n == dim; with factor > 0 prefer m == factor when it divides, otherwise the
    most balanced split whose small side does not exceed ``factor``; factor == -1: most balanced split."""
    if factor > 0 and dim % factor == 0:
        m, n = factor, dim // factor
        return (m, n) if m <= n else (n, m)
    if factor < 0:
        factor = dim
    m, n = 1, dim
    length = m + n
    while m < n:
        new_m = m + 1
        while dim % new_m:
            new_m += 1
        new_n = dim // new_m
        if new_m + new_n > length or new_m > factor:
            break
        m, n = new_m, new_n
        length = m + n
    return (m, n) if m <= n else (n, m)


class _Adapter(nn.Module):
    algo = "base"

    def __init__(self, out_f: int, in_f: int, rank: int, alpha: float):
        super().__init__()
        self.out_f, self.in_f, self.rank = out_f, in_f, rank
        self.register_buffer("alpha", torch.tensor(float(alpha)))
        self.scale = float(alpha) / max(1, rank)

    def delta_weight(self) -> torch.Tensor:          # [out, in] fp32
        raise NotImplementedError

    def effective_weight(self, W: torch.Tensor) -> torch.Tensor:
        return (W.float() + self.delta_weight()).to(W.dtype)

    def state_tensors(self, prefix: str) -> Dict[str, torch.Tensor]:
        raise NotImplementedError


class LoHa(_Adapter):
    algo = "loha"

    def __init__(self, out_f, in_f, rank=8, alpha=8.0, gen: Optional[torch.Generator] = None):
        super().__init__(out_f, in_f, rank, alpha)
        r = lambda *s, std: nn.Parameter(torch.randn(*s, generator=gen) * std)
        self.hada_w1_a, self.hada_w1_b = r(out_f, rank, std=0.1), r(rank, in_f, std=1.0)
        self.hada_w2_a, self.hada_w2_b = nn.Parameter(torch.zeros(out_f, rank)), r(rank, in_f, std=1.0)

    def delta_weight(self):
        return (self.hada_w1_a.float() @ self.hada_w1_b.float()) * (self.hada_w2_a.float() @ self.hada_w2_b.float()) * self.scale

    def state_tensors(self, prefix):
        return {f"{prefix}.hada_w1_a": self.hada_w1_a, f"{prefix}.hada_w1_b": self.hada_w1_b,
                f"{prefix}.hada_w2_a": self.hada_w2_a, f"{prefix}.hada_w2_b": self.hada_w2_b,
                f"{prefix}.alpha": self.alpha.reshape(1)}


class LoKr(_Adapter):
    """dW = kron(W1, W2) * scale with W1 [out_l, in_m], W2 [out_k, in_n]. W2 is factored iff
    rank < max(out_k, in_n) / 2; W1 is factored only with decompose_both and rank < max(out_l, in_m) / 2. With a full
    W2 the scale is forced to 1 (the saved alpha still round-trips)."""
    algo = "lokr"

    def __init__(self, out_f, in_f, rank=8, alpha=8.0, factor=-1, decompose_both=False, gen=None):
        super().__init__(out_f, in_f, rank, alpha)
        self.out_l, self.out_k = factorization(out_f, factor)
        self.in_m, self.in_n = factorization(in_f, factor)
        ku = lambda *s: nn.Parameter((torch.rand(*s, generator=gen) * 2 - 1) / math.sqrt(s[-1]))
        self.w1_factored = decompose_both and rank < max(self.out_l, self.in_m) / 2
        self.w2_factored = rank < max(self.out_k, self.in_n) / 2
        if self.w1_factored:
            self.lokr_w1_a, self.lokr_w1_b = ku(self.out_l, rank), ku(rank, self.in_m)
        else:
            self.lokr_w1 = ku(self.out_l, self.in_m)
        if self.w2_factored:
            self.lokr_w2_a, self.lokr_w2_b = ku(self.out_k, rank), nn.Parameter(torch.zeros(rank, self.in_n))
        else:
            self.lokr_w2 = nn.Parameter(torch.zeros(self.out_k, self.in_n))
            self.scale = 1.0

    def delta_weight(self):
        w1 = self.lokr_w1_a.float() @ self.lokr_w1_b.float() if self.w1_factored else self.lokr_w1.float()
        w2 = self.lokr_w2_a.float() @ self.lokr_w2_b.float() if self.w2_factored else self.lokr_w2.float()
        return torch.kron(w1, w2) * self.scale

    def state_tensors(self, prefix):
        d = {f"{prefix}.alpha": self.alpha.reshape(1)}
        if self.w1_factored:
            d[f"{prefix}.lokr_w1_a"], d[f"{prefix}.lokr_w1_b"] = self.lokr_w1_a, self.lokr_w1_b
        else:
            d[f"{prefix}.lokr_w1"] = self.lokr_w1
        if self.w2_factored:
            d[f"{prefix}.lokr_w2_a"], d[f"{prefix}.lokr_w2_b"] = self.lokr_w2_a, self.lokr_w2_b
        else:
            d[f"{prefix}.lokr_w2"] = self.lokr_w2
        return d


class Full(_Adapter):
    algo = "full"

    def __init__(self, out_f, in_f, bias: bool = False, **_):
        super().__init__(out_f, in_f, 1, 1.0)
        self.diff = nn.Parameter(torch.zeros(out_f, in_f))
        self.diff_b = nn.Parameter(torch.zeros(out_f)) if bias else None

    def delta_weight(self):
        return self.diff.float()

    def state_tensors(self, prefix):
        d = {f"{prefix}.diff.weight": self.diff}
        if self.diff_b is not None:
            d[f"{prefix}.diff_b"] = self.diff_b
        return d


class DoRA(_Adapter):
    """W_eff = m * (W + dW) / (||W + dW||_row.detach() + eps); m starts at ||W||_row (fp32), so W_eff == W at init."""
    algo = "dora"

    def __init__(self, out_f, in_f, rank=8, alpha=8.0, base_weight: Optional[torch.Tensor] = None, eps=1e-12, gen=None):
        super().__init__(out_f, in_f, rank, alpha)
        self.lora_down = nn.Parameter(torch.randn(rank, in_f, generator=gen) / math.sqrt(in_f))
        self.lora_up = nn.Parameter(torch.zeros(out_f, rank))
        mag = base_weight.detach().float().norm(dim=1) if base_weight is not None else torch.ones(out_f)
        self.dora_scale = nn.Parameter(mag.clone())
        self.eps = eps

    def delta_weight(self):
        return (self.lora_up.float() @ self.lora_down.float()) * self.scale

    def effective_weight(self, W):
        wp = W.float() + self.delta_weight()
        den = wp.norm(dim=1, keepdim=True).detach() + self.eps
        return (self.dora_scale.float().unsqueeze(1) * wp / den).to(W.dtype)

    def state_tensors(self, prefix):
        return {f"{prefix}.lora_down.weight": self.lora_down, f"{prefix}.lora_up.weight": self.lora_up,
                f"{prefix}.dora_scale": self.dora_scale, f"{prefix}.alpha": self.alpha.reshape(1)}


def cayley(S: torch.Tensor) -> torch.Tensor:
    """Exact Cayley rotation of the skew part of S [..., b, b]: Q = (S - S^T) / 2, R = (I + Q)^-1 (I - Q)."""
    Q = 0.5 * (S - S.transpose(-1, -2))
    I = torch.eye(S.shape[-1], dtype=S.dtype, device=S.device).expand_as(Q)
    return torch.linalg.solve(I + Q, I - Q)


class OFT(_Adapter):
    """W_eff = R W with R block-diagonal over groups of ``block`` output rows."""
    algo = "oft"

    def __init__(self, out_f, in_f, block: int = 4, alpha=1.0, **_):
        assert out_f % block == 0
        super().__init__(out_f, in_f, block, alpha)
        self.block, self.num_blocks = block, out_f // block
        self.oft_blocks = nn.Parameter(torch.zeros(self.num_blocks, block, block))

    def rotation_blocks(self):
        return cayley(self.oft_blocks.float())

    def effective_weight(self, W):
        R = self.rotation_blocks()                                        # [nb, b, b]
        Wg = W.float().view(self.num_blocks, self.block, self.in_f)
        return torch.bmm(R, Wg).view(self.out_f, self.in_f).to(W.dtype)

    def delta_weight(self):
        raise RuntimeError("OFT rotates the base weight; use effective_weight")

    def state_tensors(self, prefix):
        return {f"{prefix}.oft_blocks": self.oft_blocks, f"{prefix}.alpha": self.alpha.reshape(1)}


def butterfly_permutation(n: int, b: int, stage: int) -> torch.Tensor:
    """Index permutation of stage ``stage``: view the n features as (c, 2, k) with k = 2^stage * b / 2, swap the last
    two axes and flatten."""
    k = max(1, (2 ** stage) * b // 2)
    if n % (2 * k):
        return torch.arange(n)
    return torch.arange(n).view(n // (2 * k), 2, k).transpose(1, 2).reshape(n)


class BOFT(_Adapter):
    """W_eff = B_{m-1} ... B_0 W with B_i = P_i^T R_i P_i, R_i block-diagonal Cayley rotations and P_i the butterfly
    permutation of stage i; m = popcount(num_blocks - 1) + 1."""
    algo = "boft"

    def __init__(self, out_f, in_f, block: int = 4, alpha=1.0, **_):
        assert out_f % block == 0
        super().__init__(out_f, in_f, block, alpha)
        self.block, self.num_blocks = block, out_f // block
        self.boft_m = bin(self.num_blocks - 1).count("1") + 1
        self.oft_blocks = nn.Parameter(torch.zeros(self.boft_m, self.num_blocks, block, block))
        for i in range(self.boft_m):
            self.register_buffer(f"perm{i}", butterfly_permutation(out_f, block, i), persistent=False)

    def effective_weight(self, W):
        R = cayley(self.oft_blocks.float())                               # [m, nb, b, b]
        Wf = W.float()
        for i in range(self.boft_m):
            perm = getattr(self, f"perm{i}")
            inv = torch.argsort(perm)
            x = Wf[perm]                                                  # P_i W
            x = torch.bmm(R[i], x.view(self.num_blocks, self.block, self.in_f)).view(self.out_f, self.in_f)
            Wf = x[inv]                                                   # P_i^T (...)
        return Wf.to(W.dtype)

    def delta_weight(self):
        raise RuntimeError("BOFT rotates the base weight; use effective_weight")

    def state_tensors(self, prefix):
        return {f"{prefix}.oft_blocks": self.oft_blocks, f"{prefix}.alpha": self.alpha.reshape(1)}


class LoConConv(_Adapter):
    """Conv LoRA: down = k x k conv to ``rank`` channels (the base conv's stride / padding), up = 1 x 1 conv.
    Weights are kept OIHW for the file format; dW [out, in, kh, kw] = up @ down."""
    algo = "locon"

    def __init__(self, out_c, in_c, k: int = 3, rank=8, alpha=8.0, gen=None):
        super().__init__(out_c, in_c * k * k, rank, alpha)
        self.k, self.in_c = k, in_c
        self.lora_down = nn.Parameter(torch.randn(rank, in_c, k, k, generator=gen) / math.sqrt(in_c * k * k))
        self.lora_up = nn.Parameter(torch.zeros(out_c, rank, 1, 1))

    def delta_weight(self):
        d = self.lora_up.float().view(self.out_f, self.rank) @ self.lora_down.float().view(self.rank, -1)
        return d.view(self.out_f, self.in_c, self.k, self.k) * self.scale

    def effective_weight(self, W):
        return (W.float() + self.delta_weight()).to(W.dtype)

    def state_tensors(self, prefix):
        return {f"{prefix}.lora_down.weight": self.lora_down, f"{prefix}.lora_up.weight": self.lora_up,
                f"{prefix}.alpha": self.alpha.reshape(1)}


class TuckerConv(_Adapter):
    """Tucker-2 conv LoRA: down 1x1 [r, in], core k x k [r, r, k, k], up 1x1 [out, r];
    dW[o, i, h, w] = sum_{a, b} up[o, a] core[a, b, h, w] down[b, i]."""
    algo = "tucker"

    def __init__(self, out_c, in_c, k: int = 3, rank=8, alpha=8.0, gen=None):
        super().__init__(out_c, in_c * k * k, rank, alpha)
        self.k, self.in_c = k, in_c
        self.lora_down = nn.Parameter(torch.randn(rank, in_c, 1, 1, generator=gen) / math.sqrt(in_c))
        self.lora_mid = nn.Parameter(torch.randn(rank, rank, k, k, generator=gen) / math.sqrt(rank * k * k))
        self.lora_up = nn.Parameter(torch.zeros(out_c, rank, 1, 1))

    def delta_weight(self):
        up = self.lora_up.float().view(self.out_f, self.rank)
        down = self.lora_down.float().view(self.rank, self.in_c)
        return torch.einsum("oa,abhw,bi->oihw", up, self.lora_mid.float(), down) * self.scale

    def effective_weight(self, W):
        return (W.float() + self.delta_weight()).to(W.dtype)

    def state_tensors(self, prefix):
        return {f"{prefix}.lora_down.weight": self.lora_down, f"{prefix}.lora_mid.weight": self.lora_mid,
                f"{prefix}.lora_up.weight": self.lora_up, f"{prefix}.alpha": self.alpha.reshape(1)}


ALGOS = {"loha": LoHa, "lokr": LoKr, "full": Full, "dora": DoRA, "oft": OFT, "boft": BOFT, "locon": LoConConv,
         "tucker": TuckerConv}


class LycorisLinear(nn.Module):
    """A frozen linear plus one adapter. The forward is one GEMM with the effective weight."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor], adapter: _Adapter):
        super().__init__()
        self.register_buffer("weight", weight.detach())
        self.register_buffer("bias", None if bias is None else bias.detach())
        self.adapter = adapter

    def forward(self, x):
        W = self.adapter.effective_weight(self.weight)
        b = self.bias
        if getattr(self.adapter, "diff_b", None) is not None:
            b = self.adapter.diff_b.to(x.dtype) if b is None else b + self.adapter.diff_b.to(b.dtype)
        return ops.linear(x, W, b)

    @torch.no_grad()
    def merged_weight(self, strength: float = 1.0) -> torch.Tensor:
        W = self.adapter.effective_weight(self.weight).float()
        return (self.weight.float() + strength * (W - self.weight.float())).to(self.weight.dtype)


def inject_lycoris(model: nn.Module, algo: str, targets=("Linear",), match=None, **kw) -> Dict[str, _Adapter]:
    """Replace the forward of every targeted linear in ``model`` (framework ``Linear`` or ``nn.Linear``) by a GEMM with
    the adapter's effective weight. Returns {module path: adapter}; base weights are frozen."""
    cls = ALGOS[algo]
    out = {}
    for name, mod in list(model.named_modules()):
        if type(mod).__name__ not in targets or not hasattr(mod, "weight") or mod.weight.dim() != 2:
            continue
        if match is not None and not match(name):
            continue
        W = mod.weight
        extra = dict(kw)
        if algo == "dora":
            extra["base_weight"] = W
        ad = cls(W.shape[0], W.shape[1], **extra).to(W.device)
        mod.weight.requires_grad_(False)
        if getattr(mod, "bias", None) is not None:
            mod.bias.requires_grad_(False)
        mod.add_module("lycoris", ad)

        def fwd(x, _m=mod, _a=ad):
            return ops.linear(x, _a.effective_weight(_m.weight), _m.bias)

        mod.forward = fwd
        out[name] = ad
    return out


def lycoris_state_dict(adapters: Dict[str, _Adapter], prefix: str = "lycoris") -> Dict[str, torch.Tensor]:
    sd = {}
    for path, ad in adapters.items():
        key = f"{prefix}_{path.replace('.', '_')}"
        for k, v in ad.state_tensors(key).items():
            t = v.detach()
            keep32 = k.endswith(".alpha") or k.endswith(".dora_scale")
            sd[k] = t.float().contiguous() if keep32 else t.to(torch.bfloat16).contiguous()
    return sd


def load_lycoris_state_dict(adapters: Dict[str, _Adapter], sd: Dict[str, torch.Tensor], prefix: str = "lycoris") -> None:
    for path, ad in adapters.items():
        key = f"{prefix}_{path.replace('.', '_')}"
        for k, v in ad.state_tensors(key).items():
            if k.endswith(".alpha"):
                continue
            src = sd.get(k)
            if src is None and k.endswith(".dora_scale"):
                src = sd.get(k.replace(".dora_scale", ".magnitude_vector"))
            if src is None:
                raise KeyError(k)
            with torch.no_grad():
                v.copy_(src.to(v.device, v.dtype).view_as(v))
