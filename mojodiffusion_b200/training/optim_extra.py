"""Optimizer family beyond fused AdamW, selected by the config's optimizer identifier: Lion, StableAdamW, Adafactor,
Prodigy, schedule-free AdamW, SGD with momentum, and 8-bit AdamW with block-wise (256) dynamic-map quantised moments.
All run on whatever device the parameters live on (serenitymojo/training/opt_lion.mojo, opt_stableadamw.mojo, adafactor.mojo,
adamw_schedulefree.mojo, adamw8bit.mojo (bitsandbytes block-256 dynamic map parity), optimizer_dispatch.mojo)."""
from __future__ import annotations

import math
from typing import Iterable, Optional

import torch

from .optim import FusedAdamW


def _device_step(opt, kind: str, grad_scale: float, lr: float, b1: float, b2: float) -> bool:
    """Lion / StableAdamW on the GPU: every tensor in one (Lion) or two (StableAdamW: moments + per-tensor update RMS,
    then the clipped update) multi-tensor launches over the same device table the fused AdamW uses. Returns False when the
    parameters are not on a GPU with the native extension (the torch statements below then run)."""
    from ..ops import native
    from .optim import CHUNK
    ps = [p for p in opt.params if p.grad is not None]
    if not ps or not ps[0].is_cuda or not native.use_native(ps[0]):
        return False
    p0, g0 = ps[0], ps[0].grad
    if any(p.dtype != p0.dtype or p.grad.dtype != g0.dtype or not p.is_contiguous() or not p.grad.is_contiguous() for p in ps):
        return False
    if p0.dtype not in (torch.float32, torch.bfloat16) or g0.dtype not in (torch.float32, torch.bfloat16):
        return False
    key = tuple((p.data_ptr(), p.grad.data_ptr()) for p in ps)
    if getattr(opt, "_table_key", None) != key:
        rows, chunks = [], []
        for i, p in enumerate(ps):
            v = opt.v[id(p)].data_ptr() if hasattr(opt, "v") else 0
            rows.append([p.data_ptr(), p.grad.data_ptr(), opt.m[id(p)].data_ptr(), v, 0, p.numel()])
            chunks += [[i, c] for c in range((p.numel() + CHUNK - 1) // CHUNK)]
        opt._table = (torch.tensor(rows, dtype=torch.int64).to(p0.device), torch.tensor(chunks, dtype=torch.int32).to(p0.device))
        opt._table_key = key
    table, ch = opt._table
    o = native.ops()
    pb, gb = p0.dtype == torch.bfloat16, g0.dtype == torch.bfloat16
    if kind == "lion":
        o.lion_multi(table, ch, CHUNK, pb, gb, lr, b1, b2, opt.wd, grad_scale)
    else:
        opt.last_update_rms = o.stable_adamw_multi(table, ch, CHUNK, pb, gb, lr, b1, b2, opt.eps, opt.wd, grad_scale)
    return True


class _Base:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float):
        self.params = [p for p in params]
        self.lr = lr
        self.step_count = 0

    def zero_grad(self, set_to_none: bool = True):
        for p in self.params:
            p.grad = None if set_to_none else (p.grad.zero_() if p.grad is not None else None)

    def _grads(self, grad_scale):
        return [(p, p.grad.float() * grad_scale) for p in self.params if p.grad is not None]


class Lion(_Base):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, lr)
        self.betas, self.wd = betas, weight_decay
        self.m = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.params}

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        lr = self.lr if lr is None else lr
        self.step_count += 1
        b1, b2 = self.betas
        if _device_step(self, "lion", grad_scale, lr, b1, b2):
            return
        for p, g in self._grads(grad_scale):
            m = self.m[id(p)]
            upd = torch.sign(b1 * m + (1 - b1) * g)
            p.copy_((p.float() * (1 - lr * self.wd) - lr * upd).to(p.dtype))
            m.mul_(b2).add_(g, alpha=1 - b2)


class SGD(_Base):
    def __init__(self, params, lr=1e-3, momentum=0.9, weight_decay=0.0):
        super().__init__(params, lr)
        self.mu, self.wd = momentum, weight_decay
        self.buf = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.params}

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        lr = self.lr if lr is None else lr
        self.step_count += 1
        for p, g in self._grads(grad_scale):
            if self.wd:
                g = g + self.wd * p.float()
            b = self.buf[id(p)]
            b.mul_(self.mu).add_(g)
            p.copy_((p.float() - lr * b).to(p.dtype))


class StableAdamW(_Base):
    """AdamW whose per-tensor learning rate is divided by max(1, RMS(g / sqrt(v))) (update clipping)."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.01):
        super().__init__(params, lr)
        self.betas, self.eps, self.wd = betas, eps, weight_decay
        self.m = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.params}
        self.v = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.params}

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        lr = self.lr if lr is None else lr
        self.step_count += 1
        t = self.step_count
        b1, b2 = self.betas
        b1h = b1 * (1 - b1 ** (t - 1)) / (1 - b1 ** t)
        b2h = b2 * (1 - b2 ** (t - 1)) / (1 - b2 ** t)
        if _device_step(self, "stable_adamw", grad_scale, lr, b1h, b2h):
            return
        for p, g in self._grads(grad_scale):
            m, v = self.m[id(p)], self.v[id(p)]
            m.mul_(b1h).add_(g, alpha=1 - b1h)
            v.mul_(b2h).addcmul_(g, g, value=1 - b2h)
            rms = float(torch.sqrt((g * g / v.clamp_min(self.eps ** 2)).mean()))
            eta = lr / max(1.0, rms)
            p.copy_((p.float() * (1 - eta * self.wd) - eta * m / (v.sqrt() + self.eps)).to(p.dtype))


class Automagic3(_Base):
    """Self-tuning optimizer: a magnitude-normalised update from a factored second moment, and ONE learning rate for the
    whole parameter group that a per-element vote over the last ``history`` update signs raises or lowers every step.

    Per tensor: for matrices row = b2 row + (1 - b2)(mean_cols(g^2) + eps), col likewise over rows, update =
    rsqrt(row / mean(row)) x rsqrt(col) * g; for vectors v = b2 v + (1 - b2) g^2, update = rsqrt(v + eps) g. The update is
    divided by max(RMS(update) / clip, 1) and clamped to +-clip. Vote: an element whose last H update signs all agree adds
    +|update| ("step too small"), one whose signs alternate perfectly adds -|update| ("overshoot"); pooled over every
    element of every tensor, lr *= exp(clamp(sum / sum|update|, -1, 1)), once per step, and not before a tensor's window is
    full. The parameter step uses the learning rate from before the vote; weight decay is added to the update. bf16
    parameters are written back with stochastic rounding (a uniform dither in the 16 dropped mantissa bits, then
    truncation): at the small self-chosen rates round-to-nearest would leave most weights unchanged.
    The scheduler's learning rate is ignored after the first step (serenitymojo/training/automagic3.mojo:1-500)."""

    LR_MIN, LR_MAX = 1e-30, 1e3

    def __init__(self, params, lr=1e-6, beta2=0.999, eps=1e-30, clip=1.0, weight_decay=0.0, history=8, seed=0):
        super().__init__(params, lr)
        self.beta2, self.eps, self.clip, self.wd = beta2, eps, clip, weight_decay
        self.h = min(max(int(history), 2), 64)
        self.state = {}
        self.gen = {}
        self.seed = seed

    def _rng(self, device):
        key = str(device)
        if key not in self.gen:
            self.gen[key] = torch.Generator(device=device).manual_seed(0x9E3779B97F4A7C15 % (2 ** 63) + self.seed)
        return self.gen[key]

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        self.step_count += 1
        b2, H = self.beta2, self.h
        num = den = 0.0
        for p, g in self._grads(grad_scale):
            g = torch.nan_to_num(g, nan=0.0, posinf=0.0, neginf=0.0)
            st = self.state.setdefault(id(p), {"idx": 0, "fill": 0})
            sq = g * g
            if g.dim() >= 2:
                if "row" not in st:
                    st["row"] = torch.zeros(g.shape[:-1], dtype=torch.float32, device=g.device)
                    st["col"] = torch.zeros(g.shape[:-2] + g.shape[-1:], dtype=torch.float32, device=g.device)
                st["row"].mul_(b2).add_(sq.mean(-1) + self.eps, alpha=1 - b2)
                st["col"].mul_(b2).add_(sq.mean(-2) + self.eps, alpha=1 - b2)
                r = torch.rsqrt(st["row"] / st["row"].mean(-1, keepdim=True))
                upd = r.unsqueeze(-1) * torch.rsqrt(st["col"]).unsqueeze(-2) * g
            else:
                if "v" not in st:
                    st["v"] = torch.zeros_like(g)
                st["v"].mul_(b2).add_(sq, alpha=1 - b2)
                upd = torch.rsqrt(st["v"] + self.eps) * g
            upd = upd / max(float(upd.square().mean().sqrt()) / self.clip, 1.0)
            upd = upd.clamp(-self.clip, self.clip)
            flat = upd.reshape(-1)
            if "hist" not in st:
                st["hist"] = torch.zeros(H, flat.numel(), dtype=torch.bool, device=g.device)
            st["hist"][st["idx"]] = flat > 0
            st["idx"] = (st["idx"] + 1) % H
            st["fill"] = min(st["fill"] + 1, H)
            if st["fill"] == H:
                hist = torch.roll(st["hist"], -st["idx"], 0)                    # oldest plane first
                s1 = hist.sum(0)
                agree = (s1 == H) | (s1 == 0)
                alternate = ((hist[1:] != hist[:-1]).sum(0) == H - 1) & ~agree
                w = flat.abs().double()
                num += float((w * agree).sum() - (w * alternate).sum())
                den += float(w.sum())
            if self.wd:
                upd = upd + self.wd * p.float()
            new = p.float() - self.lr * upd
            if p.dtype == torch.bfloat16:
                bits = new.contiguous().view(torch.int32)
                dither = torch.randint(0, 1 << 16, bits.shape, dtype=torch.int32, device=bits.device, generator=self._rng(bits.device))
                new = ((bits + dither) & ~0xFFFF).view(torch.float32)
            p.copy_(new.to(p.dtype))
        if den > 0.0:
            signal = min(max(num / max(den, 1e-30), -1.0), 1.0)
            self.lr = min(max(self.lr * math.exp(signal), self.LR_MIN), self.LR_MAX)


class Adafactor(_Base):
    """Factored second moments for matrices (row / column statistics), relative step off, no first moment."""

    def __init__(self, params, lr=1e-4, decay_rate=-0.8, eps=(1e-30, 1e-3), clip_threshold=1.0, weight_decay=0.0):
        super().__init__(params, lr)
        self.decay_rate, self.eps, self.clip, self.wd = decay_rate, eps, clip_threshold, weight_decay
        self.state = {}

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        lr = self.lr if lr is None else lr
        self.step_count += 1
        rho = 1.0 - self.step_count ** self.decay_rate
        for p, g in self._grads(grad_scale):
            st = self.state.setdefault(id(p), {})
            g2 = g * g + self.eps[0]
            if g.dim() >= 2:
                r = st.setdefault("r", torch.zeros(g.shape[:-1], device=g.device))
                c = st.setdefault("c", torch.zeros(g.shape[:-2] + g.shape[-1:], device=g.device))
                r.mul_(rho).add_(g2.mean(-1), alpha=1 - rho)
                c.mul_(rho).add_(g2.mean(-2), alpha=1 - rho)
                vhat = (r / r.mean(-1, keepdim=True)).unsqueeze(-1) * c.unsqueeze(-2)
            else:
                v = st.setdefault("v", torch.zeros_like(g))
                v.mul_(rho).add_(g2, alpha=1 - rho)
                vhat = v
            u = g / vhat.sqrt()
            u = u / max(1.0, float(u.pow(2).mean().sqrt()) / self.clip)
            p.copy_((p.float() * (1 - lr * self.wd) - lr * u).to(p.dtype))


class Prodigy(_Base):
    """Adam with a distance estimate d that scales the step (d grows from d0 as evidence accumulates)."""

    def __init__(self, params, lr=1.0, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, d0=1e-6, d_coef=1.0):
        super().__init__(params, lr)
        self.betas, self.eps, self.wd, self.d, self.d_coef = betas, eps, weight_decay, d0, d_coef
        self.d_numerator = 0.0
        self.m = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.params}
        self.v = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.params}
        self.s = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.params}
        self.p0 = {id(p): p.detach().float().clone() for p in self.params}

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        lr = self.lr if lr is None else lr
        self.step_count += 1
        b1, b2 = self.betas
        d = self.d
        dlr = d * lr
        sb2 = math.sqrt(b2)
        self.d_numerator *= sb2
        s_norm = 0.0
        for p, g in self._grads(grad_scale):
            k = id(p)
            self.d_numerator += (d / 1.0) * dlr * float((g * (self.p0[k] - p.float())).sum())
            self.m[k].mul_(b1).add_(g, alpha=d * (1 - b1))
            self.v[k].mul_(b2).addcmul_(g, g, value=d * d * (1 - b2))
            self.s[k].mul_(sb2).add_(g, alpha=(d / 1.0) * dlr)
            s_norm += float(self.s[k].abs().sum())
        if s_norm > 0:
            self.d = max(self.d, self.d_coef * self.d_numerator / s_norm)
        for p, g in self._grads(grad_scale):
            k = id(p)
            denom = self.v[k].sqrt() + d * self.eps
            p.copy_((p.float() * (1 - self.wd * dlr) - dlr * self.m[k] / denom).to(p.dtype))


class ScheduleFreeAdamW(_Base):
    """Schedule-free AdamW: gradients are evaluated at y = (1-beta1) z + beta1 x; x is the running average of z."""

    def __init__(self, params, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, warmup_steps=0):
        super().__init__(params, lr)
        self.betas, self.eps, self.wd, self.warmup = betas, eps, weight_decay, warmup_steps
        self.z = {id(p): p.detach().float().clone() for p in self.params}
        self.v = {id(p): torch.zeros_like(p, dtype=torch.float32) for p in self.params}
        self.lr_sum = 0.0

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        lr = self.lr if lr is None else lr
        self.step_count += 1
        t = self.step_count
        b1, b2 = self.betas
        sched = min(1.0, t / self.warmup) if self.warmup > 0 else 1.0
        lr_t = lr * sched * math.sqrt(1 - b2 ** t)
        self.lr_sum += lr_t ** 2
        ck = (lr_t ** 2) / self.lr_sum
        for p, g in self._grads(grad_scale):
            k = id(p)
            self.v[k].mul_(b2).addcmul_(g, g, value=1 - b2)
            gn = g / (self.v[k].sqrt() + self.eps)
            y = p.float()
            gn = gn + self.wd * y
            y = y.lerp(self.z[k], ck)                       # x-average folded into y
            y = y + gn * (lr_t * (b1 * (1 - ck) - 1))
            self.z[k].sub_(gn, alpha=lr_t)
            p.copy_(y.to(p.dtype))


# ---- 8-bit AdamW: block-wise (256) dynamic-map quantisation of the moments ---------------------------------
def dynamic_map(signed: bool = True, max_exponent_bits: int = 7, total_bits: int = 8) -> torch.Tensor:
    """The 256-entry dynamic quantisation map (exponent + linear fraction per sign), sorted ascending."""
    data = []
    non_sign_bits = total_bits - (1 if signed else 1)
    additional = 2 ** (non_sign_bits - max_exponent_bits) - 1
    for i in range(max_exponent_bits):
        frac_items = int(2 ** (i + non_sign_bits - max_exponent_bits) + 1) if signed else int(2 ** (i + non_sign_bits - max_exponent_bits + 1) + 1)
        bounds = torch.linspace(0.1, 1, frac_items)
        means = (bounds[:-1] + bounds[1:]) / 2.0
        data += ((10 ** (-(max_exponent_bits - 1) + i)) * means).tolist()
        if signed:
            data += (-(10 ** (-(max_exponent_bits - 1) + i)) * means).tolist()
    if additional > 0:
        bounds = torch.linspace(0.1, 1, additional + 1)
        means = (bounds[:-1] + bounds[1:]) / 2.0
        data += ((10 ** (-(max_exponent_bits - 1) + max_exponent_bits - 1)) * means).tolist()
        if signed:
            data += (-(10 ** (-(max_exponent_bits - 1) + max_exponent_bits - 1)) * means).tolist()
    data += [0.0, 1.0]
    while len(data) < 256:
        data.append(0.0)
    return torch.tensor(sorted(data)[:256] if len(data) > 256 else sorted(data), dtype=torch.float32)


def quantize_blockwise(x: torch.Tensor, code: torch.Tensor, block: int = 256):
    """Returns (uint8 codes, fp32 absmax per block): x/absmax is mapped to the nearest code entry (binary search)."""
    flat = x.float().flatten()
    n = flat.numel()
    pad = (-n) % block
    if pad:
        flat = torch.cat((flat, flat.new_zeros(pad)))
    blocks = flat.view(-1, block)
    absmax = blocks.abs().amax(1).clamp_min(1e-30)
    normed = blocks / absmax[:, None]
    c = code.to(x.device)
    idx = torch.searchsorted(c, normed.contiguous()).clamp(1, 255)
    lo, hi = c[idx - 1], c[idx]
    idx = torch.where((normed - lo).abs() <= (hi - normed).abs(), idx - 1, idx)
    return idx.to(torch.uint8).flatten()[:n], absmax


def dequantize_blockwise(q: torch.Tensor, absmax: torch.Tensor, code: torch.Tensor, shape, block: int = 256):
    n = q.numel()
    vals = code.to(q.device)[q.long()]
    pad = (-n) % block
    if pad:
        vals = torch.cat((vals, vals.new_zeros(pad)))
    return (vals.view(-1, block) * absmax[:, None]).flatten()[:n].view(shape)


class AdamW8bit(_Base):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, block: int = 256):
        super().__init__(params, lr)
        self.betas, self.eps, self.wd, self.block = betas, eps, weight_decay, block
        self.code_s, self.code_u = dynamic_map(True), dynamic_map(False)
        self.state = {}

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        lr = self.lr if lr is None else lr
        self.step_count += 1
        t = self.step_count
        b1, b2 = self.betas
        from ..ops import native
        for p in self.params:
            if p.grad is None or not (p.is_cuda and native.use_native(p)) or p.dtype not in (torch.bfloat16, torch.float32):
                continue
            # GPU: one kernel per tensor de-quantises, updates and re-quantises block by block (csrc/optim.cu)
            st = self.state.get(id(p))
            n = p.numel()
            if st is None:
                nb = (n + self.block - 1) // self.block
                st = {"qm": torch.zeros(n, dtype=torch.uint8, device=p.device), "qv": torch.zeros(n, dtype=torch.uint8, device=p.device),
                      "am": torch.zeros(nb, device=p.device), "av": torch.zeros(nb, device=p.device), "t": 0}
                self.state[id(p)] = st
                self._codes = getattr(self, "_codes", {})
                if p.device not in self._codes:
                    self._codes[p.device] = (self.code_s.to(p.device).contiguous(), self.code_u.to(p.device).contiguous())
            cs, cu = self._codes[p.device]
            st["t"] += 1
            g = p.grad if p.grad.dtype in (torch.bfloat16, torch.float32) else p.grad.float()
            assert self.block == 256 and p.is_contiguous()
            native.ops().adamw8bit(p.data, g.contiguous(), st["qm"], st["qv"], st["am"], st["av"], cs, cu, lr, b1, b2, self.eps,
                                   self.wd, st["t"], grad_scale)
        for p in self.params:
            if p.grad is None or (p.is_cuda and native.use_native(p) and p.dtype in (torch.bfloat16, torch.float32)):
                continue
            g = p.grad.float() * grad_scale
            st = self.state.get(id(p))
            if st is None:
                m, v = torch.zeros_like(g), torch.zeros_like(g)
            else:
                m = dequantize_blockwise(st["qm"], st["am"], self.code_s, g.shape, self.block)
                v = dequantize_blockwise(st["qv"], st["av"], self.code_u, g.shape, self.block)
            m = b1 * m + (1 - b1) * g
            v = b2 * v + (1 - b2) * g * g
            pf = p.float() * (1 - lr * self.wd)
            pf = pf - (lr / (1 - b1 ** t)) * m / (v.sqrt() / math.sqrt(1 - b2 ** t) + self.eps)
            p.copy_(pf.to(p.dtype))
            qm, am = quantize_blockwise(m, self.code_s, self.block)
            qv, av = quantize_blockwise(v, self.code_u, self.block)
            self.state[id(p)] = {"qm": qm, "am": am, "qv": qv, "av": av}


def create_optimizer(name: str, params, lr: float, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                     max_grad_norm: float = 0.0, stochastic_rounding: bool = False):
    """Config identifier (OneTrainer-style, case-insensitive) -> optimizer instance."""
    n = (name or "ADAMW").upper().replace("-", "_")
    params = list(params)
    if n in ("ADAMW", "ADAMW_FUSED", "ADAM"):
        return FusedAdamW(params, lr, betas, eps, weight_decay, max_grad_norm=max_grad_norm,
                          stochastic_rounding=stochastic_rounding)
    if n in ("ADAMW_BF16", "ADAMW_OT"):
        return FusedAdamW(params, lr, betas, eps, weight_decay, moment_dtype=torch.bfloat16, stochastic_rounding=True,
                          max_grad_norm=max_grad_norm)
    if n in ("ADAMW_8BIT", "ADAMW8BIT"):
        return AdamW8bit(params, lr, betas, eps, weight_decay)
    if n == "LION":
        return Lion(params, lr, (betas[0], 0.99), weight_decay)
    if n in ("STABLEADAMW", "STABLE_ADAMW"):
        return StableAdamW(params, lr, (betas[0], 0.99), eps, weight_decay)
    if n == "ADAFACTOR":
        return Adafactor(params, lr, weight_decay=weight_decay)
    if n in ("AUTOMAGIC3", "AUTOMAGIC"):
        return Automagic3(params, lr, weight_decay=weight_decay)
    if n == "PRODIGY":
        return Prodigy(params, lr if lr >= 0.1 else 1.0, betas, eps, weight_decay)
    if n in ("SCHEDULE_FREE_ADAMW", "ADAMW_SCHEDULEFREE"):
        return ScheduleFreeAdamW(params, lr, betas, eps, weight_decay)
    if n == "SGD":
        return SGD(params, lr, 0.9, weight_decay)
    raise ValueError(f"unknown optimizer '{name}'")
