"""Fully-sharded data parallel linears for full finetuning, with the collectives fused into the GEMMs.

Every ``FSDPLinear`` keeps only 1/N of its weight rows: the bf16 shard lives in symmetric memory (peers read it),
the fp32 master copy and the AdamW moments exist for the shard only.

* forward  : ``y = x @ W^T`` where W is re-assembled INSIDE the consuming GEMM: warp 6 of every CTA streams its share
             of each remote weight shard over NVLink (bulk copies through shared memory) into a transient full-weight
             buffer while the tensor core already works on the output columns of the local shard (parameter
             all-gather fused into the first consumer).
* backward : ``dx = dy @ W`` from the gathered buffer (re-gathered by peer loads if another layer has reused it);
             ``dW = dy^T x`` whose bf16 tiles the GEMM epilogue stores straight into slot [rank] of the row OWNER's
             staging buffer (gradient reduce-scatter fused into the producing GEMM); a tail kernel does the all-rank
             barrier and adds the N slots into the owner's fp32 gradient shard.
* step     : after one flag barrier, a single multi-tensor AdamW launch updates every local master shard and writes
             the new bf16 shard back into symmetric memory (fp32 masters, bf16 shadows: csrc/optim.cu).

The reference has no FSDP; its closest analogue keeps fp32 masters and 8-bit moments on the host
(serenitymojo/training/full_finetune_zimage.mojo:1-36). ``mode="nccl"`` is the all_gather / reduce_scatter baseline.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import native
from ..utils.tracing import nvtx_range
from ..ops.functional import _flat2d, _gemm
from .symm import SymmetricBuffer

SLOT_BWD_DONE, SLOT_STEP_DONE, SLOT_RS = 6, 7, 5
_FLAG_BYTES = 512


class FSDPContext:
    """Owns the symmetric arena (weight shards + gradient shards of all layers), the transient gather buffer and the
    flags. Layers register themselves; ``finalize()`` allocates."""

    def __init__(self, group=None, mode: str = "fused", device=None, fuse_optimizer: bool = False,
                 offload_optimizer: bool = False):
        """``offload_optimizer``: the fp32 master shards and both AdamW moments (12 of the 14 resident bytes per sharded
        parameter) live in pinned host memory; ``step`` streams them through four device staging slots, layer by layer,
        on two copy streams (one per direction) that run ahead of / behind the per-layer AdamW launches (not combinable with ``fuse_optimizer``).

        ``fuse_optimizer``: the reduce-scatter tail of every layer's weight gradient also applies AdamW to the owner's
        shard (one launch per layer inside backward, no stored gradient shard); call ``begin_step`` with the step's
        hyper-parameters before backward, ``step`` afterwards only publishes the new shards. Each layer may be used once
        per step in this mode, and there is no gradient accumulation or clipping across layers."""
        self.group, self.mode = group, mode
        self.fuse_optimizer = fuse_optimizer
        self.offload_optimizer = offload_optimizer
        assert not (fuse_optimizer and offload_optimizer), "the fused optimizer updates device-resident state"
        self.hyper = None
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.layers: List["FSDPLinear"] = []
        self.symm: Optional[SymmetricBuffer] = None
        self.gathered_owner = None
        self.step_count = 0

    def register(self, layer: "FSDPLinear"):
        self.layers.append(layer)

    def finalize(self):
        off = _FLAG_BYTES
        for l in self.layers:
            l.off_w = off
            off += (l.rows_local * l.in_features * 2 + 255) // 256 * 256
            l.off_g = off
            off += (l.rows_local * l.in_features * 4 + 255) // 256 * 256
        big = max(l.out_features * l.in_features for l in self.layers)
        # two staging buffers for the reduce-scatter of dW (bf16 partial rows from every rank), used alternately so a rank
        # that is one layer ahead never writes into a buffer that is still being summed
        self.off_stage = []
        for _ in range(2):
            self.off_stage.append(off)
            off += (big * 2 + 255) // 256 * 256
        native.load(True)
        if self.mode == "fused" and self.world > 1:
            self.symm = SymmetricBuffer.create(off, self.group, self.device, False)
            arena = self.symm.local
        else:
            arena = torch.zeros(off, dtype=torch.uint8, device=self.device)
        self.arena = arena
        self.flags = arena[:256].view(torch.int32)
        self.counters = torch.zeros(16, dtype=torch.int32, device=self.device)
        self.ready = torch.zeros(8, dtype=torch.int32, device=self.device)
        self.rs_calls = 0
        self.wbuf = torch.empty(big, dtype=torch.bfloat16, device=self.device)
        for l in self.layers:
            n = l.rows_local * l.in_features
            l.w_shard = arena[l.off_w:l.off_w + n * 2].view(torch.bfloat16).view(l.rows_local, l.in_features)
            l.g_shard = arena[l.off_g:l.off_g + n * 4].view(torch.float32).view(l.rows_local, l.in_features)
            l.w_shard.copy_(l.master.to(torch.bfloat16))
            l.g_shard.zero_()
        torch.cuda.synchronize(self.device)
        if self.offload_optimizer:
            biggest = max(l.rows_local * l.in_features for l in self.layers)
            self._slots = [torch.empty(3, biggest, dtype=torch.float32, device=self.device) for _ in range(4)]
            self._copy_stream = torch.cuda.Stream(self.device)       # host -> device
            self._back_stream = torch.cuda.Stream(self.device)       # device -> host: both directions of the link run at once
            for l in self.layers:                                  # [master | m | v] of a layer as one pinned block = one DMA each way
                host = torch.empty(3, l.master.numel(), dtype=torch.float32).pin_memory()
                host[0].copy_(l.master.reshape(-1))
                host[1:].zero_()
                l.host_state = host
                l.master = host[0].view(l.rows_local, l.in_features)
                l.m = host[1].view(l.rows_local, l.in_features)
                l.v = host[2].view(l.rows_local, l.in_features)
            torch.cuda.empty_cache()
        if self.world > 1:
            dist.barrier(self.group)
        return self

    # ---- flag barriers (stream ordered, no host sync) ----------------------------------------------------
    def barrier(self, slot: int):
        if self.world == 1:
            return
        if self.symm is not None:
            o = native.ops()
            o.flag_signal(self.symm.ptrs_at(0), slot, self.rank, 0, self.flags, self.counters)
            o.flag_wait(self.flags, slot, self.world, 0, self.counters)
        else:
            dist.barrier(self.group)

    def full_weight(self, layer: "FSDPLinear") -> torch.Tensor:
        return self.wbuf[:layer.out_features * layer.in_features].view(layer.out_features, layer.in_features)

    def ensure_gathered(self, layer: "FSDPLinear") -> torch.Tensor:
        """Full weight in the transient buffer (plain peer-load all-gather; used by backward when needed)."""
        W = self.full_weight(layer)
        if self.gathered_owner is layer:
            return W
        if self.world == 1:
            W.copy_(layer.w_shard)
        elif self.symm is not None:
            native.ops().peer_gather(self.symm.ptrs_at(layer.off_w), W, layer.rows_local * layer.in_features * 2,
                                     self.rank, True)
        else:
            dist.all_gather_into_tensor(W, layer.w_shard.contiguous(), group=self.group)
        self.gathered_owner = layer
        return W

    # ---- optimizer ---------------------------------------------------------------------------------------------
    def begin_step(self, lr=1e-5, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, grad_scale: Optional[float] = None):
        """Fused-optimizer mode: fix this step's AdamW hyper-parameters before backward runs."""
        self.step_count += 1
        self.hyper = (float(lr), float(betas[0]), float(betas[1]), float(eps), float(weight_decay), self.step_count,
                      (1.0 / self.world) if grad_scale is None else float(grad_scale))
        for l in self.layers:
            l._updated = False

    def fused_active(self) -> bool:
        return self.fuse_optimizer and self.world > 1 and self.symm is not None

    @torch.no_grad()
    def step(self, lr=1e-5, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, grad_scale: Optional[float] = None):
        """AdamW on every local master shard (one launch), bf16 shards refreshed for the next all-gather."""
        if self.fused_active():
            if self.hyper is None:
                raise RuntimeError("fuse_optimizer: call begin_step() before backward")
            # layers that received no gradient this step (their output does not reach the loss) still decay: one AdamW
            # launch over just those, with their zero gradient shards
            idle = tuple(i for i, l in enumerate(self.layers) if not getattr(l, "_updated", False))
            if idle:
                self._adamw_over(idle, *self.hyper)
            self.hyper = None
            self.gathered_owner = None
            self.barrier(SLOT_STEP_DONE)                      # every rank's updated shards are in place before the next gather
            if self.step_count % getattr(self, "check_every", 16) == 0:
                self.check()
            return
        with nvtx_range("collective/fsdp/grad_barrier"):
            self.barrier(SLOT_BWD_DONE)                       # every rank's dW tiles have been added into my shards
        self.step_count += 1
        scale = (1.0 / self.world) if grad_scale is None else grad_scale
        from ..training.optim import CHUNK
        if self.offload_optimizer:
            self._offloaded_adamw(lr, betas, eps, weight_decay, scale)
            for l in self.layers:
                l.g_shard.zero_()
            self.gathered_owner = None
            self.barrier(SLOT_STEP_DONE)
            if self.step_count % getattr(self, "check_every", 16) == 0:
                self.check()
            return
        if getattr(self, "_table", None) is None:
            rows, chunks = [], []
            for i, l in enumerate(self.layers):
                n = l.master.numel()
                rows.append([l.master.data_ptr(), l.g_shard.data_ptr(), l.m.data_ptr(), l.v.data_ptr(), l.w_shard.data_ptr(), n])
                chunks += [[i, c] for c in range((n + CHUNK - 1) // CHUNK)]
            self._table = (torch.tensor(rows, dtype=torch.int64).to(self.device),
                           torch.tensor(chunks, dtype=torch.int32).to(self.device))
        table, chunks = self._table
        native.ops().adamw_multi(table, chunks, CHUNK, False, False, False, lr, betas[0], betas[1], eps, weight_decay,
                                 self.step_count, scale, None, 0.0, 0, False)
        for l in self.layers:
            l.g_shard.zero_()
        self.gathered_owner = None
        self.barrier(SLOT_STEP_DONE)                      # new shards visible everywhere before the next gather
        if self.step_count % getattr(self, "check_every", 16) == 0:
            self.check()

    def _offloaded_adamw(self, lr, betas, eps, wd, scale):
        """Layer i's [master | m | v] block goes host -> slot i % 4 on one copy stream, AdamW runs on it in the compute
        stream (gradient shard and bf16 weight shard stay on the device), and the block returns to the host on a second
        copy stream while the next layers' blocks are already arriving in the other slots."""
        from ..training.optim import CHUNK
        cs, bs, main = self._copy_stream, self._back_stream, torch.cuda.current_stream(self.device)
        NS = len(self._slots)
        if getattr(self, "_off_tables", None) is None:
            self._off_tables = []
            for i, l in enumerate(self.layers):
                n, slot = l.master.numel(), self._slots[i % NS]
                row = [[slot[0].data_ptr(), l.g_shard.data_ptr(), slot[1].data_ptr(), slot[2].data_ptr(), l.w_shard.data_ptr(), n]]
                self._off_tables.append((torch.tensor(row, dtype=torch.int64).to(self.device),
                                         torch.tensor([[0, c] for c in range((n + CHUNK - 1) // CHUNK)], dtype=torch.int32).to(self.device)))
        L = len(self.layers)
        loaded = [torch.cuda.Event() for _ in range(L)]
        updated = [torch.cuda.Event() for _ in range(L)]
        stored = [torch.cuda.Event() for _ in range(L)]
        cs.wait_stream(main)
        bs.wait_stream(main)

        def fetch(i):
            n = self.layers[i].master.numel()
            if i >= NS:
                cs.wait_event(stored[i - NS])                     # the slot's previous block is back on the host
            with torch.cuda.stream(cs):
                self._slots[i % NS][:, :n].copy_(self.layers[i].host_state, non_blocking=True)
                loaded[i].record(cs)

        def write_back(i):
            bs.wait_event(updated[i])
            n = self.layers[i].master.numel()
            with torch.cuda.stream(bs):
                self.layers[i].host_state.copy_(self._slots[i % NS][:, :n], non_blocking=True)
                stored[i].record(bs)
        for i in range(min(NS - 1, L)):
            fetch(i)
        for i in range(L):
            main.wait_event(loaded[i])
            table, chunks = self._off_tables[i]
            native.ops().adamw_multi(table, chunks, CHUNK, False, False, False, lr, betas[0], betas[1], eps, wd,
                                     self.step_count, scale, None, 0.0, 0, False)
            updated[i].record(main)
            write_back(i)
            if i + NS - 1 < L:
                fetch(i + NS - 1)
        main.wait_stream(cs)
        main.wait_stream(bs)
        bs.synchronize()                                          # host tensors are read by checkpointing right after step()

    def _adamw_over(self, idx, lr, b1, b2, eps, wd, t_step, scale):
        from ..training.optim import CHUNK
        cache = self.__dict__.setdefault("_idle_tables", {})
        if idx not in cache:
            rows, chunks = [], []
            for j, i in enumerate(idx):
                l = self.layers[i]
                n = l.master.numel()
                rows.append([l.master.data_ptr(), l.g_shard.data_ptr(), l.m.data_ptr(), l.v.data_ptr(), l.w_shard.data_ptr(), n])
                chunks += [[j, c] for c in range((n + CHUNK - 1) // CHUNK)]
            cache[idx] = (torch.tensor(rows, dtype=torch.int64).to(self.device), torch.tensor(chunks, dtype=torch.int32).to(self.device))
        table, chunks = cache[idx]
        native.ops().adamw_multi(table, chunks, CHUNK, False, False, False, lr, b1, b2, eps, wd, t_step, scale, None, 0.0, 0, False)

    def check(self) -> None:
        """Raise if a bounded wait of the fused kernels ran out on this device since the last check (the AdamW launch of
        such a step leaves the shards untouched). Synchronises the stream: called every ``check_every`` (16) steps by
        ``step()`` and meant to be called before every save or backup."""
        native.check_status(self.layers[0].master if self.layers else None)


class _FSDPLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, layer):
        c = layer.ctx
        W = c.full_weight(layer)
        if c.world > 1 and c.symm is not None:
            rl = layer.rows_local
            W[c.rank * rl:(c.rank + 1) * rl].copy_(layer.w_shard)
            y = _gemm([x2], [W], bias=layer.bias, gather_ptrs=c.symm.ptrs_at(layer.off_w),
                      gather_cfg=[c.rank, 1, rl, rl * layer.in_features * 2], gather_dst=W, gather_ready=c.ready)
            c.gathered_owner = layer
        else:
            W = c.ensure_gathered(layer)
            y = _gemm([x2], [W], bias=layer.bias)
        ctx.layer = layer
        ctx.save_for_backward(x2)
        return y

    @staticmethod
    def backward(ctx, dy):
        (x2,) = ctx.saved_tensors
        layer = ctx.layer
        c = layer.ctx
        dy = _flat2d(dy)
        dx = None
        if ctx.needs_input_grad[0]:
            W = c.ensure_gathered(layer)
            dx = _gemm([dy], [W], b_mn=True)
        # dW = dy^T x, reduce-scattered over ranks into the owners' fp32 gradient shards
        if c.world > 1 and c.symm is not None:
            # bf16 partial rows go into slot [rank] of the row owner's staging buffer; the tail kernel does the barrier and
            # adds the N slots into the owner's fp32 gradient shard
            c.rs_calls += 1
            off = c.off_stage[c.rs_calls % 2]
            rl, K = layer.rows_local, layer.in_features
            _gemm([dy], [x2], a_mn=True, b_mn=True, route_ptrs=c.symm.ptrs_at(off), route_cfg=[rl, K, c.rank])
            stage = c.arena[off:off + c.world * rl * K * 2].view(torch.bfloat16).view(c.world, rl, K)
            if c.fuse_optimizer:
                if c.hyper is None:
                    raise RuntimeError("fuse_optimizer: begin_step() was not called before backward")
                if getattr(layer, "_updated", False):
                    raise RuntimeError("fuse_optimizer: a layer took part in backward twice in one step")
                lr, b1, b2, eps_, wd, t_step, gs = c.hyper
                native.ops().rs_adamw(c.symm.ptrs_at(0), c.flags, SLOT_RS, c.rs_calls, c.rank, stage, layer.master, layer.m, layer.v,
                                      layer.w_shard, lr, b1, b2, eps_, wd, t_step, gs)
                layer._updated = True
            else:
                native.ops().rs_finalize(c.symm.ptrs_at(0), c.flags, SLOT_RS, c.rs_calls, c.rank, stage, None, None, None, 1,
                                         layer.g_shard)
        else:
            dw = _gemm([dy], [x2], a_mn=True, b_mn=True, out_fp32=True)
            if c.world > 1:
                part = torch.empty_like(layer.g_shard)
                dist.reduce_scatter_tensor(part, dw.contiguous(), group=c.group)
                layer.g_shard += part
            else:
                layer.g_shard += dw
        if layer.bias is not None and layer.bias.requires_grad:
            g = dy.float().sum(0)
            layer.bias.grad = g.to(layer.bias.dtype) if layer.bias.grad is None else layer.bias.grad + g.to(layer.bias.dtype)
        return dx, None


class FSDPLinear(nn.Module):
    def __init__(self, ctx: FSDPContext, in_features: int, out_features: int, bias: bool = True, full_weight=None,
                 seed: int = 0):
        super().__init__()
        assert out_features % ctx.world == 0 and in_features % 8 == 0
        self.ctx = ctx
        self.in_features, self.out_features = in_features, out_features
        self.rows_local = out_features // ctx.world
        r = ctx.rank
        if full_weight is None:
            g = torch.Generator().manual_seed(seed)
            full_weight = torch.randn(out_features, in_features, generator=g) / math.sqrt(in_features)
        shard = full_weight[r * self.rows_local:(r + 1) * self.rows_local].float().to(ctx.device)
        self.master = shard.contiguous()                                  # fp32 master (shard)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=torch.bfloat16, device=ctx.device)) if bias else None
        self.w_shard = self.g_shard = None
        self.off_w = self.off_g = 0
        ctx.register(self)

    def forward(self, x):
        lead = x.shape[:-1]
        x2 = _flat2d(x)
        if not x2.requires_grad and torch.is_grad_enabled():
            x2 = x2.detach().requires_grad_(True)            # dW must be produced even for the first layer
        y = _FSDPLinearFn.apply(x2, self)
        return y.reshape(*lead, self.out_features)

    def full_master(self) -> torch.Tensor:
        """All-gather of the fp32 master shards (checkpointing)."""
        if self.ctx.world == 1:
            return self.master.clone()
        mine = self.master.to(self.ctx.device)                  # a host-resident master (offloaded optimizer) travels by the device
        parts = [torch.empty_like(mine) for _ in range(self.ctx.world)]
        dist.all_gather(parts, mine, group=self.ctx.group)
        return torch.cat(parts, 0)


class ShardedLinear(nn.Module):
    """Drop-in for ``models.layers.Linear`` inside a fully-sharded model: the projection is an :class:`FSDPLinear` (weight
    rows sharded over the ranks, collectives inside the GEMMs), the activation / gated residual that ``Linear`` fuses into
    its epilogue run as the differentiable element-wise ops after it."""

    def __init__(self, ctx: FSDPContext, lin):
        super().__init__()
        self.in_features, self.out_features = lin.in_features, lin.out_features
        self.inner = FSDPLinear(ctx, lin.in_features, lin.out_features, bias=lin.bias is not None,
                                full_weight=lin.weight.detach())
        if lin.bias is not None:
            with torch.no_grad():
                self.inner.bias.copy_(lin.bias)
        self.slots = nn.ModuleList()

    @property
    def bias(self):
        return self.inner.bias

    @property
    def weight(self):
        """This rank's bf16 rows of the weight (callers read its dtype / device; the full matrix exists only transiently)."""
        return self.inner.w_shard

    def forward(self, x, act=None, residual=None, gate=None, rows_per_group: int = 1, out=None):
        y = self.inner(x)
        if act is not None:
            y = ops.activation(y, act)
        if residual is not None:
            y = ops.gate_residual(residual, y, gate, rows_per_group)
        elif gate is not None:
            raise ValueError("a gate needs a residual")
        if out is not None:
            out.copy_(y)
            return out
        return y


def shard_model(model: nn.Module, ctx: FSDPContext, min_params: int = 1 << 16, skip=()) -> int:
    """Replace every ``Linear`` of ``model`` whose weight has at least ``min_params`` elements and whose row count
    divides by the world size with a :class:`ShardedLinear` (the full weight is released as soon as its shard has been
    cut), then allocate the context. Returns the number of sharded layers; the remaining parameters (norm scales, biases,
    small embedders) stay replicated and are the caller's to all-reduce."""
    from ..models.layers import Linear
    todo = []
    for name, mod in model.named_modules():
        for cname, child in mod.named_children():
            full = f"{name}.{cname}" if name else cname
            if isinstance(child, Linear) and child.weight.numel() >= min_params and child.out_features % ctx.world == 0 \
                    and child.in_features % 8 == 0 and len(child.slots) == 0 and not any(full.startswith(s) for s in skip):
                todo.append((mod, cname, child))
    for mod, cname, child in todo:
        sharded = ShardedLinear(ctx, child)
        child.weight.data = torch.empty(0, dtype=child.weight.dtype, device=child.weight.device)
        if isinstance(mod, (nn.ModuleList, nn.ModuleDict)):
            mod[int(cname) if isinstance(mod, nn.ModuleList) else cname] = sharded
        else:
            setattr(mod, cname, sharded)
    ctx.finalize()
    return len(todo)
