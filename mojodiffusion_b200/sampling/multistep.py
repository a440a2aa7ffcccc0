"""Multistep solvers with fp64 coefficient math and history buffers: DPM-Solver++(2M) and UniPC (bh2), written for
a data-prediction model in the (alpha, sigma) parametrisation, with adapters for flow-matching (alpha = 1 - sigma)
and for epsilon models. Behaviour reference: serenitymojo/sampling/dpmpp_2m.mojo:52-261, serenitymojo/sampling/unipc.mojo:61-931.
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional, Sequence

import torch


def _lambda(alpha: float, sigma: float) -> float:
    return math.log(max(alpha, 1e-12)) - math.log(max(sigma, 1e-12))


def flow_alpha_sigma(s: float):
    """Flow matching: x_t = (1 - s) x0 + s eps."""
    return 1.0 - s, s


def vp_alpha_sigma_from_sigma(sig: float):
    """k-diffusion sigma (VE-scaled VP): alpha = 1/sqrt(1+sig^2), sigma = sig/sqrt(1+sig^2)."""
    a = 1.0 / math.sqrt(1.0 + sig * sig)
    return a, sig * a


def x0_from_velocity(x, v, s: float):
    """Flow matching velocity v = eps - x0  ->  x0 = x - s v."""
    return x - s * v


class DPMPP2M:
    """x_{i+1} = (sigma_{i+1}/sigma_i) x_i - alpha_{i+1} (e^{-h} - 1) D, D = (1 + 1/(2r)) x0_i - 1/(2r) x0_{i-1}."""

    def __init__(self, alphas: Sequence[float], sigmas: Sequence[float]):
        self.alphas, self.sigmas = list(alphas), list(sigmas)
        self.prev_x0: Optional[torch.Tensor] = None
        self.prev_h: Optional[float] = None

    def step(self, x: torch.Tensor, x0: torch.Tensor, i: int) -> torch.Tensor:
        a0, s0, a1, s1 = self.alphas[i], self.sigmas[i], self.alphas[i + 1], self.sigmas[i + 1]
        if s1 <= 0.0:
            self.prev_x0, self.prev_h = x0, None
            return x0.to(x.dtype) * a1 if a1 != 1.0 else x0.to(x.dtype)
        h = _lambda(a1, s1) - _lambda(a0, s0)
        if self.prev_x0 is None or self.prev_h is None:
            D = x0
        else:
            r = self.prev_h / h
            D = (1.0 + 1.0 / (2.0 * r)) * x0 - (1.0 / (2.0 * r)) * self.prev_x0
        out = (s1 / s0) * x - a1 * math.expm1(-h) * D
        self.prev_x0, self.prev_h = x0, h
        return out


class UniPCMultistep:
    """UniPC predictor-corrector, bh2 variant, order <= 2 history (the common configuration)."""

    def __init__(self, alphas: Sequence[float], sigmas: Sequence[float], order: int = 2, corrector: bool = True):
        self.alphas, self.sigmas, self.order, self.use_corrector = list(alphas), list(sigmas), order, corrector
        self.hist_x0: List[torch.Tensor] = []
        self.hist_i: List[int] = []
        self.last_sample: Optional[torch.Tensor] = None

    def _lam(self, i):
        return _lambda(self.alphas[i], self.sigmas[i])

    def _update(self, x, i_from, i_to, x0_new: Optional[torch.Tensor], order: int):
        """Shared predictor (x0_new None) / corrector (x0_new = model output at i_to) formula, data prediction."""
        a_t, s_t, s_0 = self.alphas[i_to], self.sigmas[i_to], self.sigmas[i_from]
        h = self._lam(i_to) - self._lam(i_from)
        m0 = self.hist_x0[-1]
        hh = -h
        h_phi_1 = math.expm1(hh)
        B_h = math.expm1(hh)                      # bh2
        rks, D1s = [], []
        for k in range(1, order):
            if len(self.hist_x0) > k:
                rk = (self._lam(self.hist_i[-(k + 1)]) - self._lam(i_from)) / h
                rks.append(rk)
                D1s.append((self.hist_x0[-(k + 1)] - m0) / rk)
        x_t = (s_t / s_0) * x - a_t * h_phi_1 * m0
        if x0_new is None:                          # predictor
            if D1s:
                x_t = x_t - a_t * B_h * 0.5 * D1s[0]
            return x_t
        rks.append(1.0)
        # solve the small Vandermonde system R rho = b (order <= 2 -> closed form / 2x2)
        n = len(rks)
        h_phi_k = h_phi_1 / hh - 1.0
        fact = 1.0
        R = torch.zeros(n, n, dtype=torch.float64)
        b = torch.zeros(n, dtype=torch.float64)
        for k in range(1, n + 1):
            R[k - 1] = torch.tensor([rk ** (k - 1) for rk in rks], dtype=torch.float64)
            b[k - 1] = h_phi_k * fact / B_h
            fact *= (k + 1)
            h_phi_k = h_phi_k / hh - 1.0 / fact
        rho = torch.linalg.solve(R, b) if n > 1 else torch.tensor([0.5], dtype=torch.float64)
        corr = 0.0
        for k, D1 in enumerate(D1s):
            corr = corr + float(rho[k]) * D1
        D1_t = x0_new - m0
        return x_t - a_t * B_h * (corr + float(rho[-1]) * D1_t)

    def step(self, x: torch.Tensor, x0: torch.Tensor, i: int) -> torch.Tensor:
        """x0: data prediction at step i for the sample x (which is the predictor's output of the previous call)."""
        if self.use_corrector and self.last_sample is not None and self.hist_x0:
            order_c = min(self.order, len(self.hist_x0))
            x = self._update(self.last_sample, self.hist_i[-1], i, x0, order_c)
        self.hist_x0.append(x0)
        self.hist_i.append(i)
        if len(self.hist_x0) > self.order:
            self.hist_x0.pop(0)
            self.hist_i.pop(0)
        if self.sigmas[i + 1] <= 0.0:
            self.last_sample = None
            return x0.to(x.dtype)
        order_p = min(self.order, len(self.hist_x0), len(self.sigmas) - 1 - i)
        self.last_sample = x
        return self._update(x, i, i + 1, None, order_p)


@torch.no_grad()
def sample_multistep(x0_fn: Callable[[torch.Tensor, int], torch.Tensor], x: torch.Tensor, solver, n_steps: int):
    """Drive a solver: x0_fn(x, i) returns the data prediction at schedule index i."""
    x = x.float()
    for i in range(n_steps):
        x = solver.step(x, x0_fn(x, i).float(), i)
    return x
