"""Tensor-parallel MLP with the collectives fused into the GEMMs (activations stay sequence-sharded between blocks).

    x_local [rows/N, D] --all-gather--> [rows, D] @ W1_shard^T (+b1, act) -> h [rows, F/N]         (AG -> GEMM)
    h @ W2_shard^T -> partial [rows, D] --reduce-scatter--> y_local [rows/N, D]                     (GEMM -> RS)

* AG -> GEMM is ONE kernel: warp 6 of every CTA of the tcgen05 GEMM pulls its slice of each remote activation chunk
  out of the owner's symmetric buffer (peer loads over NVLink) into the local gathered operand and bumps that chunk's
  arrival counter; the TMA producer starts with the local chunk's tiles and waits (bounded) only for chunks that
  have not landed yet. Each remote byte crosses NVLink once and lands in local HBM, from where TMA reads it.
* GEMM -> RS is ONE kernel: the epilogue adds each fp32 partial 32-column slab into the row owner's fp32 buffer with
  ``red.global.add.v4.f32`` on peer memory; a small finalise step applies bias / gate / residual and re-zeroes.
* ``mode="nccl"`` does the same with all_gather_into_tensor / reduce_scatter_tensor: baseline and oracle.

The reference has no tensor parallelism (serenitymojo/docs/AUDIT_SIMPLETUNER_PARITY_2026-06-11.md:81-110).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import native
from ..ops.functional import _flat2d, _gemm
from ..ops.reference import act_code
from .symm import SymmetricBuffer

SLOT_X_READY, SLOT_X_DONE, SLOT_RS_DONE = 0, 1, 2
_FLAG_BYTES = 512


class TPContext:
    def __init__(self, rows_total: int, dim: int, group=None, mode: str = "fused", symm: Optional[SymmetricBuffer] = None,
                 device=None, dtype=torch.bfloat16):
        self.mode, self.group = mode, group
        if symm is not None:
            self.rank, self.world = symm.rank, symm.world
        else:
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        N = self.world
        assert rows_total % N == 0
        self.rows, self.rl, self.D = rows_total, rows_total // N, dim
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype
        xs_bytes = self.rl * dim * 2
        acc_bytes = self.rl * dim * 4
        self.off_x = _FLAG_BYTES
        self.off_acc = self.off_x + (xs_bytes + 255) // 256 * 256
        total = self.off_acc + acc_bytes
        self.calls = 0
        if mode == "fused":
            native.load(True)
            self.symm = symm if symm is not None else SymmetricBuffer.create(total, group, self.device, False)
            self.flags = self.symm.view(0, 64, torch.int32)
            self.counters = torch.zeros(16, dtype=torch.int32, device=self.device)
            self.x_shard = self.symm.view(self.off_x, self.rl * dim, dtype).view(self.rl, dim)
            self.acc = self.symm.view(self.off_acc, self.rl * dim, torch.float32).view(self.rl, dim)
            self.acc.zero_()
            self.x_gathered = torch.empty(rows_total, dim, dtype=dtype, device=self.device)
            self.ready = torch.zeros(8, dtype=torch.int32, device=self.device)

    @staticmethod
    def symm_bytes(rows_total, dim, world) -> int:
        rl = rows_total // world
        return _FLAG_BYTES + (rl * dim * 2 + 255) // 256 * 256 + rl * dim * 4 + 256

    def _signal(self, slot):
        native.ops().flag_signal(self.symm.ptrs_at(0), slot, self.rank, 0, self.flags, self.counters)

    def _wait(self, slot):
        native.ops().flag_wait(self.flags, slot, self.world, 0, self.counters)

    @torch.no_grad()
    def mlp(self, x_local, w1_shard, b1_shard, w2_shard, b2, act="gelu_tanh", residual=None, gate=None,
            rows_per_group: int = 1):
        """x_local: [rows/N, D]; w1_shard: [F/N, D]; w2_shard: [D, F/N] (this rank's K slice); b2: [D] full.
        Returns y_local [rows/N, D] = residual + gate * (mlp(x) + b2)."""
        x2 = _flat2d(x_local)
        N, r, rl = self.world, self.rank, self.rl
        if self.mode == "nccl" or N == 1:
            if N > 1:
                xg = torch.empty(self.rows, self.D, dtype=x2.dtype, device=x2.device)
                dist.all_gather_into_tensor(xg, x2.contiguous(), group=self.group)
            else:
                xg = x2
            h = ops.linear(xg, w1_shard, b1_shard, act=act)
            part = ops.linear(h, w2_shard).float()
            if N > 1:
                y = torch.empty(rl, self.D, dtype=torch.float32, device=x2.device)
                dist.reduce_scatter_tensor(y, part.contiguous(), group=self.group)
            else:
                y = part
        else:
            if self.calls > 0:
                self._wait(SLOT_X_DONE)                       # peers finished reading my previous x shard
            self.calls += 1
            self.x_shard.copy_(x2)
            self.x_gathered[r * rl:(r + 1) * rl].copy_(x2)
            self._signal(SLOT_X_READY)
            self._wait(SLOT_X_READY)
            h = _gemm([self.x_gathered], [w1_shard], bias=b1_shard, act=act_code(act),
                      gather_ptrs=self.symm.ptrs_at(self.off_x), gather_cfg=[r, 0, rl, rl * self.D * 2],
                      gather_dst=self.x_gathered, gather_ready=self.ready)
            self._signal(SLOT_X_DONE)
            _gemm([h], [w2_shard], out_fp32=True, route_ptrs=self.symm.ptrs_at(self.off_acc), route_cfg=[rl, self.D])
            self._signal(SLOT_RS_DONE)
            self._wait(SLOT_RS_DONE)
            y = self.acc.clone()
            self.acc.zero_()
        if b2 is not None:
            y = y + b2.float()
        y = y.to(x2.dtype)
        if residual is not None or gate is not None:
            res = _flat2d(residual) if residual is not None else torch.zeros_like(y)
            y = ops.gate_residual(res, y, gate, rows_per_group)
        return y.reshape(x_local.shape)


def shard_mlp_weights(w1, b1, w2, rank: int, world: int):
    """Column-parallel first layer (rows of W1), row-parallel second layer (columns of W2)."""
    F = w1.shape[0]
    fl = F // world
    return (w1[rank * fl:(rank + 1) * fl].contiguous(), b1[rank * fl:(rank + 1) * fl].contiguous() if b1 is not None else None,
            w2[:, rank * fl:(rank + 1) * fl].contiguous())
