"""Parity harness: cosine similarity, max-abs and relative L2 error of a result against a reference, accumulated in
float64, with named gates (default cos >= 0.999; 0.99 for bf16 end-to-end; 0.99999999 for training blocks against an
fp32 twin) and a report that tests print on failure (serenitymojo/parity.mojo:21-107)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Mapping, Optional

import torch

GATE_DEFAULT, GATE_BF16, GATE_TRAINING_BLOCK = 0.999, 0.99, 0.99999999


@dataclass
class ParityResult:
    name: str
    cos: float
    max_abs: float
    rel_l2: float
    ref_max: float
    n: int
    finite: bool

    def ok(self, cos_min: float = GATE_DEFAULT, max_abs: Optional[float] = None, rel_l2: Optional[float] = None) -> bool:
        if not self.finite or self.cos < cos_min:
            return False
        if max_abs is not None and self.max_abs > max_abs:
            return False
        return rel_l2 is None or self.rel_l2 <= rel_l2

    def line(self) -> str:
        return (f"[parity] {self.name}: cos={self.cos:.10f} max_abs={self.max_abs:.4e} rel_l2={self.rel_l2:.4e} "
                f"ref_max={self.ref_max:.4e} n={self.n}{'' if self.finite else ' NON-FINITE'}")


def compare(name: str, got: torch.Tensor, ref: torch.Tensor) -> ParityResult:
    if tuple(got.shape) != tuple(ref.shape):
        raise ValueError(f"{name}: shape {tuple(got.shape)} vs reference {tuple(ref.shape)}")
    a = got.detach().to("cpu", torch.float64).flatten()
    b = ref.detach().to("cpu", torch.float64).flatten()
    finite = bool(torch.isfinite(a).all())
    na, nb = float(a.norm()), float(b.norm())
    if na == 0.0 and nb == 0.0:
        cos = 1.0
    elif na == 0.0 or nb == 0.0:
        cos = 0.0
    else:
        cos = float(torch.dot(a, b)) / (na * nb)
    d = a - b
    return ParityResult(name, cos, float(d.abs().max()) if a.numel() else 0.0,
                        float(d.norm()) / nb if nb > 0 else float(d.norm()), float(b.abs().max()) if b.numel() else 0.0,
                        a.numel(), finite)


class ParityHarness:
    """Collects comparisons; ``assert_all`` raises with every failing line."""

    def __init__(self, cos_min: float = GATE_DEFAULT):
        self.cos_min = cos_min
        self.results: Dict[str, ParityResult] = {}
        self.failed = []

    def check(self, name: str, got: torch.Tensor, ref: torch.Tensor, cos_min: Optional[float] = None,
              max_abs: Optional[float] = None, rel_l2: Optional[float] = None) -> ParityResult:
        r = compare(name, got, ref)
        self.results[name] = r
        if not r.ok(self.cos_min if cos_min is None else cos_min, max_abs, rel_l2):
            self.failed.append(r)
        return r

    def check_dict(self, got: Mapping[str, torch.Tensor], ref: Mapping[str, torch.Tensor], **kw) -> None:
        missing = set(ref) - set(got)
        if missing:
            raise KeyError(f"parity: missing tensors {sorted(missing)[:5]}")
        for k in ref:
            self.check(k, got[k], ref[k], **kw)

    def bit_equal(self, name: str, got: torch.Tensor, ref: torch.Tensor) -> int:
        """Number of mismatching elements (fused-vs-unfused self parity where the math is identical)."""
        n = int((got != ref).sum())
        if n:
            self.failed.append(ParityResult(name + " (bit)", float("nan"), float((got.float() - ref.float()).abs().max()),
                                            float("nan"), float(ref.float().abs().max()), got.numel(), True))
        return n

    def report(self) -> str:
        return "\n".join(r.line() for r in self.results.values())

    def assert_all(self) -> None:
        if self.failed:
            raise AssertionError("parity gate failed:\n" + "\n".join(r.line() for r in self.failed))


def nondegenerate_fill(shape, seed: int = 0, dtype=torch.float32, device="cpu") -> torch.Tensor:
    """Test data whose rows / heads never repeat: sum of incommensurate sinusoids plus seeded noise. Periodic integer
    fills can alias with tensor strides and produce constant operands whose gradients are exactly zero."""
    n = math.prod(shape)
    i = torch.arange(n, dtype=torch.float64)
    g = torch.Generator().manual_seed(seed)
    x = torch.sin(i * 0.7310585786) + 0.5 * torch.cos(i * 0.2689414214 + seed) + 0.25 * torch.randn(n, generator=g, dtype=torch.float64)
    return x.view(shape).to(dtype).to(device)
