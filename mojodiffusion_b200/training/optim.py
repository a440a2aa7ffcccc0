"""Optimizers. ``FusedAdamW`` updates every tensor in ONE kernel launch on the GPU (multi-tensor table walk in
``csrc/optim.cu``) and falls back to the same fp32 math in torch on CPU. Variants selectable by flags:

* fp32 or bf16 parameters; fp32 or bf16 gradients
* fp32 moments (torch.optim.AdamW semantics) or bf16 moments (OneTrainer-style memory saving)
* stochastic-rounding bf16 write-back (``stochastic_rounding=True``) or round-to-nearest-even
* clip-by-global-norm with the norm computed on the device and consumed by the update kernel without a host sync

Reference behaviour: serenitymojo/training/optim.mojo:79-364, serenitymojo/training/fused_adamw_multitensor.mojo:45-285,
serenitymojo/training/lora_adamw_ot_fused.mojo:13-142, serenitymojo/training/lora_adamw_plain_fused.mojo,
serenitymojo/training/on_device_global_norm.mojo.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional, Tuple

import torch

from ..ops import native, reference as ref

CHUNK = 4096 * 4


class FusedAdamW:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-4, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, moment_dtype=torch.float32, stochastic_rounding: bool = False,
                 max_grad_norm: float = 0.0, seed: int = 0, master_weights: bool = False):
        self.params: List[torch.nn.Parameter] = [p for p in params]
        assert self.params, "no parameters"
        # full fine-tune: fp32 masters are what the kernel updates; the bf16 model tensors are rewritten from them
        # in the same pass (the table's shadow slot)
        self.masters = [p.detach().float().clone() for p in self.params] if master_weights else None
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.moment_dtype = moment_dtype
        self.stochastic_rounding = stochastic_rounding
        self.max_grad_norm = max_grad_norm
        self.seed = seed
        self.step_count = 0
        self.m = [torch.zeros_like(p, dtype=moment_dtype) for p in self.params]
        self.v = [torch.zeros_like(p, dtype=moment_dtype) for p in self.params]
        self._index = {id(p): i for i, p in enumerate(self.params)}
        self._table = None
        self._table_key = None
        self.last_grad_norm: Optional[torch.Tensor] = None

    # ---- state access (checkpoint sidecars) -------------------------------------------------------
    def moments(self, p) -> Tuple[torch.Tensor, torch.Tensor]:
        i = self._index[id(p)]
        return self.m[i], self.v[i]

    def set_moments(self, p, m, v) -> None:
        i = self._index[id(p)]
        with torch.no_grad():
            self.m[i].copy_(m.to(self.m[i].dtype))
            self.v[i].copy_(v.to(self.v[i].dtype))

    def zero_grad(self, set_to_none: bool = False):
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    # ---- device tables -------------------------------------------------------------------------------
    def _build_table(self, grads: List[torch.Tensor]):
        key = tuple((p.data_ptr(), g.data_ptr()) for p, g in zip(self.params, grads))
        if self._table_key == key:
            return self._table
        dev = self.params[0].device
        rows, chunks = [], []
        for i, (p, g) in enumerate(zip(self.params, grads)):
            assert p.is_contiguous() and g.is_contiguous()
            if self.masters is not None:
                rows.append([self.masters[i].data_ptr(), g.data_ptr(), self.m[i].data_ptr(), self.v[i].data_ptr(),
                             p.data_ptr() if p.dtype == torch.bfloat16 else 0, p.numel()])
            else:
                rows.append([p.data_ptr(), g.data_ptr(), self.m[i].data_ptr(), self.v[i].data_ptr(), 0, p.numel()])
            for c in range((p.numel() + CHUNK - 1) // CHUNK):
                chunks.append([i, c])
        table = torch.tensor(rows, dtype=torch.int64).to(dev)
        ch = torch.tensor(chunks, dtype=torch.int32).to(dev)
        self._table, self._table_key = (table, ch), key
        return self._table

    # ---- step ---------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None) -> None:
        lr = self.lr if lr is None else lr
        self.step_count += 1
        grads = [p.grad if p.grad is not None else torch.zeros_like(p) for p in self.params]
        p0 = self.params[0]
        b1, b2 = self.betas
        if p0.is_cuda and native.use_native(p0):
            o = native.ops()
            g0 = grads[0]
            assert all(g.dtype == g0.dtype for g in grads) and all(p.dtype == p0.dtype for p in self.params)
            table, chunks = self._build_table(grads)
            norm_sq = None
            g_bf16 = g0.dtype == torch.bfloat16
            if self.max_grad_norm > 0:
                norm_sq = o.sumsq_multi(table, chunks, CHUNK, g_bf16)
                self.last_grad_norm = norm_sq
            o.adamw_multi(table, chunks, CHUNK, p0.dtype == torch.bfloat16 and self.masters is None, g_bf16,
                          self.moment_dtype == torch.bfloat16, lr, b1, b2, self.eps, self.weight_decay,
                          self.step_count, grad_scale, norm_sq, self.max_grad_norm,
                          (self.seed * 1000003 + self.step_count) & 0x7FFFFFFF, self.stochastic_rounding)
            return
        # CPU / reference path
        clip = 1.0
        if self.max_grad_norm > 0:
            total = math.sqrt(sum(float((g.float() * grad_scale).pow(2).sum()) for g in grads))
            self.last_grad_norm = torch.tensor(total * total / (grad_scale * grad_scale) if grad_scale else 0.0)
            clip = min(1.0, self.max_grad_norm / (total + 1e-6))
        for i, (p, g) in enumerate(zip(self.params, grads)):
            src = p if self.masters is None else self.masters[i]
            pn, mn, vn = ref.adamw_step(src, g, self.m[i], self.v[i], lr, b1, b2, self.eps, self.weight_decay,
                                        self.step_count, grad_scale * clip)
            if self.masters is not None:
                self.masters[i].copy_(pn)
            p.copy_(pn.to(p.dtype))
            self.m[i].copy_(mn.to(self.m[i].dtype))
            self.v[i].copy_(vn.to(self.v[i].dtype))

    def grad_norm(self) -> float:
        """Global L2 norm of the (unscaled) gradients seen by the last clipped step (device sync)."""
        if self.last_grad_norm is None:
            return float("nan")
        return float(self.last_grad_norm.float().sqrt())

    def state_dict(self):
        return {"step": self.step_count, "m": self.m, "v": self.v}


def build_tensor_table(shadows, params):
    """Device table for the multi-tensor EMA kernel: one row [param, 0, shadow, 0, 0, numel] per tensor plus the
    (tensor, chunk) work list."""
    rows, chunks = [], []
    for i, (s_, p_) in enumerate(zip(shadows, params)):
        assert s_.is_contiguous() and p_.is_contiguous()
        rows.append([p_.data_ptr(), 0, s_.data_ptr(), 0, 0, p_.numel()])
        for c in range((p_.numel() + CHUNK - 1) // CHUNK):
            chunks.append([i, c])
    dev = params[0].device
    return torch.tensor(rows, dtype=torch.int64).to(dev), torch.tensor(chunks, dtype=torch.int32).to(dev)
