"""Data-parallel adapter training with the gradient all-reduce, the 1/world scale, the global-norm clip and the
AdamW update fused into peer-memory kernels (``csrc/comm_kernels.cu``).

All trainable parameters live in one flat bf16 buffer and all gradients in another, both in symmetric memory.
Per step and rank: reduce-scatter by direct peer loads (or ``multimem.ld_reduce`` through NVSwitch) of this rank's
1/N shard -> partial sum of squares to every peer -> AdamW on the shard with fp32 moments that exist only for the
shard -> the new bf16 parameters are stored into every rank's parameter buffer (``multimem.st`` or peer stores).
Everything is ordered on the caller's stream by epoch flags; nothing returns to the host.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..ops import native
from ..utils.tracing import nvtx_range
from .symm import SymmetricBuffer, emulated_group

SLOT_READY, SLOT_NORM, SLOT_DONE = 0, 1, 2
_FLAG_BYTES = 4 * 8 * 8          # 8 slots x 8 ranks int32
_SCALAR_BYTES = 4 * 8


def _layout(params: Sequence[torch.Tensor], world: int):
    offs, n = [], 0
    for p in params:
        offs.append(n)
        n += (p.numel() + 7) // 8 * 8
    unit = 8 * world
    total = (n + unit - 1) // unit * unit
    return offs, total


class FusedDPAdamW:
    """One instance per rank. ``step()`` replaces all-reduce + clip + optimizer.step()."""

    def __init__(self, params: Sequence[torch.nn.Parameter], lr=1e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01,
                 max_grad_norm: float = 0.0, group=None, symm: Optional[SymmetricBuffer] = None,
                 use_multicast: bool = True, check_every: int = 16):
        """``check_every``: every that many steps ``step()`` reads the device status word (one small synchronising copy)
        and raises if a bounded wait of the fused kernels ran out; a step after such a time-out leaves the parameters
        untouched on the device. ``check()`` does the same on demand (call it before every save or backup)."""
        self.params = list(params)
        p0 = self.params[0]
        assert p0.is_cuda and all(p.dtype == torch.bfloat16 for p in self.params), "bf16 CUDA parameters"
        native.load(True)
        self.lr, self.betas, self.eps, self.wd, self.max_norm = lr, betas, eps, weight_decay, max_grad_norm
        world = symm.world if symm is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.offsets, self.total = _layout(self.params, world)
        pbytes = self.total * 2
        need = _FLAG_BYTES + _SCALAR_BYTES + 2 * pbytes + 512
        self.symm = symm if symm is not None else SymmetricBuffer.create(need, group, p0.device, use_multicast)
        assert self.symm.local.numel() >= need
        self.rank, self.world = self.symm.rank, self.symm.world
        self.off_flags, self.off_scalars = 0, _FLAG_BYTES
        self.off_params = 512
        self.off_grads = 512 + pbytes
        self.flags = self.symm.view(self.off_flags, 64, torch.int32)
        self.scalars = self.symm.view(self.off_scalars, 8, torch.float32)
        self.flat_params = self.symm.view(self.off_params, self.total, torch.bfloat16)
        self.flat_grads = self.symm.view(self.off_grads, self.total, torch.bfloat16)
        with torch.no_grad():
            for p, o in zip(self.params, self.offsets):
                self.flat_params[o:o + p.numel()].copy_(p.detach().reshape(-1))
                p.data = self.flat_params[o:o + p.numel()].view_as(p)
        self.attach_grads()
        shard = self.total // self.world
        self.lo, self.hi = self.rank * shard, (self.rank + 1) * shard
        dev = p0.device
        self.red = torch.zeros(shard, dtype=torch.float32, device=dev)
        self.m = torch.zeros(shard, dtype=torch.float32, device=dev)
        self.v = torch.zeros(shard, dtype=torch.float32, device=dev)
        self.sumsq = torch.zeros((), dtype=torch.float32, device=dev)
        self.norm_out = torch.zeros((), dtype=torch.float32, device=dev)
        self.done_counter = torch.zeros((), dtype=torch.int32, device=dev)
        self.epoch = 0
        self.step_count = 0
        self.check_every = max(1, int(check_every))
        self.group = group
        self._state_cache = None          # (step_count, m_full, v_full) from the last gather_state()

    def attach_grads(self):
        for p, o in zip(self.params, self.offsets):
            p.grad = self.flat_grads[o:o + p.numel()].view_as(p)

    def zero_grad(self, set_to_none: bool = False):
        self.flat_grads.zero_()
        self.attach_grads()

    # ---- phases (the single-GPU emulation calls them rank by rank) ----------------------------------
    def phase_ready(self):
        self.epoch += 1
        self.step_count += 1
        o = native.ops()
        self.sumsq.zero_()
        self.done_counter.zero_()
        o.flag_signal(self.symm.ptrs_at(self.off_flags), SLOT_READY, self.rank, self.epoch, self.flags, None)

    def phase_reduce(self):
        native.ops().dp_reduce_shard(self.symm.ptrs_at(self.off_grads), self.symm.mc_at(self.off_grads), self.flags,
                                     SLOT_READY, self.epoch, self.lo, self.hi, self.red, self.sumsq)

    def phase_publish(self):
        native.ops().publish_scalar(self.symm.ptrs_at(self.off_scalars), self.symm.ptrs_at(self.off_flags), self.sumsq,
                                    SLOT_NORM, self.rank, self.epoch)

    def phase_update(self, lr: Optional[float] = None):
        b1, b2 = self.betas
        native.ops().dp_adamw_shard(self.symm.ptrs_at(self.off_params), self.symm.mc_at(self.off_params),
                                    self.symm.ptrs_at(self.off_flags), self.flags, self.scalars, SLOT_NORM, SLOT_DONE,
                                    self.epoch, self.rank, self.lo, self.hi, self.red, self.m, self.v,
                                    self.lr if lr is None else lr, b1, b2, self.eps, self.wd, self.step_count,
                                    1.0 / self.world, self.max_norm, self.norm_out, self.done_counter)

    def phase_finish(self):
        native.ops().flag_wait(self.flags, SLOT_DONE, self.world, self.epoch, None)

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0, lr: Optional[float] = None):
        assert grad_scale == 1.0, "the 1/world scale is applied inside the fused kernels"
        with nvtx_range("collective/dp/reduce_scatter_adamw_all_gather"):
            self.phase_ready()
            self.phase_reduce()
            self.phase_publish()
            self.phase_update(lr)
            self.phase_finish()
        if self.step_count % self.check_every == 0:
            self.check()

    def check(self) -> None:
        """Raise if any bounded wait ran out on this device since the last check (synchronises the stream)."""
        native.check_status(self.red)

    def grad_norm(self) -> float:
        return float(self.norm_out)

    # ---- optimizer-state access for checkpoints (moments are sharded) ---------------------------------------
    def gather_state(self):
        """COLLECTIVE: every rank calls it, once, before the rank-0-only save branch. All-gathers the sharded moments
        (two collectives in total) and caches the full vectors; ``moments(p)`` then slices the cache without communicating."""
        self.check()
        if self.world == 1 or not dist.is_initialized():
            m, v = self.m.clone(), self.v.clone()
        else:
            m = torch.empty(self.total, dtype=torch.float32, device=self.m.device)
            v = torch.empty_like(m)
            dist.all_gather_into_tensor(m, self.m, group=self.group)
            dist.all_gather_into_tensor(v, self.v, group=self.group)
        self._state_cache = (self.step_count, m, v)
        return m, v

    def moments(self, p):
        """fp32 (m, v) of parameter ``p`` from the last ``gather_state()`` (which must belong to the current step when the
        group has more than one rank: this call itself never communicates, so rank 0 may call it alone)."""
        if self._state_cache is None or self._state_cache[0] != self.step_count:
            if self.world > 1:
                raise RuntimeError("FusedDPAdamW.moments: call gather_state() on every rank after the last step first")
            self.gather_state()
        _, m, v = self._state_cache
        i = [id(q) for q in self.params].index(id(p))
        o = self.offsets[i]
        return m[o:o + p.numel()].view_as(p), v[o:o + p.numel()].view_as(p)

    def set_moments(self, p, m, v) -> None:
        """Restore the moments of one parameter: the part of it that falls into this rank's shard is written."""
        i = [id(q) for q in self.params].index(id(p))
        o = self.offsets[i]
        lo, hi = max(o, self.lo), min(o + p.numel(), self.hi)
        if hi > lo:
            dev = self.m.device
            self.m[lo - self.lo:hi - self.lo].copy_(m.reshape(-1)[lo - o:hi - o].to(dev, torch.float32))
            self.v[lo - self.lo:hi - self.lo].copy_(v.reshape(-1)[lo - o:hi - o].to(dev, torch.float32))
        self._state_cache = None

    def load_state(self, m_full: torch.Tensor, v_full: torch.Tensor, step: int) -> None:
        """Restore from full-length moment vectors (as returned by ``gather_state``) and the bias-correction step."""
        dev = self.m.device
        self.m.copy_(m_full[self.lo:self.hi].to(dev, torch.float32))
        self.v.copy_(v_full[self.lo:self.hi].to(dev, torch.float32))
        self.step_count = int(step)
        self._state_cache = None


def emulate_ranks(param_sets: List[Sequence[torch.nn.Parameter]], **kw) -> List[FusedDPAdamW]:
    """Single-GPU stand-in for N ranks: N parameter replicas, N symmetric buffers on one device."""
    world = len(param_sets)
    _, total = _layout(list(param_sets[0]), world)
    bufs = emulated_group(world, _FLAG_BYTES + _SCALAR_BYTES + 4 * total + 512)
    return [FusedDPAdamW(ps, symm=bufs[r], **kw) for r, ps in enumerate(param_sets)]


def emulated_step(ranks: List[FusedDPAdamW], lr: Optional[float] = None):
    for r in ranks:
        r.phase_ready()
    for r in ranks:
        r.phase_reduce()
    for r in ranks:
        r.phase_publish()
    for r in ranks:
        r.phase_update(lr)
    for r in ranks:
        r.phase_finish()
