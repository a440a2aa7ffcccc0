"""Tensor-parallel MLP with the collectives fused into the GEMMs (activations stay sequence-sharded between blocks).

    x_local [rows/N, D] --all-gather--> [rows, D] @ W1_shard^T (+b1, act) -> h [rows, F/N]         (AG -> GEMM)
    h @ W2_shard^T -> partial [rows, D] --reduce-scatter--> y_local [rows/N, D]                     (GEMM -> RS)

* AG -> GEMM is ONE kernel: one thread of warp 6 in every CTA of the tcgen05 GEMM streams its share of each remote
  activation chunk out of the owner's symmetric buffer through two 16 KB shared-memory stages with bulk copies (peer
  memory -> shared -> the local gathered operand) and bumps that chunk's arrival counter; the TMA producer starts with
  the local chunk's tiles and waits (bounded) only for chunks that have not landed yet. Each remote byte crosses
  NVLink once and lands in local HBM, from where TMA reads it.
* GEMM -> RS is ONE kernel plus a tail: the epilogue stores each bf16 partial 32-column slab into slot [this rank] of
  the row owner's staging buffer (plain 16-byte stores over NVLink: half the bytes of fp32 atomics and no read-modify-
  write at the far end); the tail kernel does the all-rank barrier, sums the N slots in fp32 and applies
  bias / gate / residual in the same pass.
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
        x_bytes = rows_total * dim * 2                 # gathered activations: my rows are my shard, the rest arrive
        stage_bytes = N * self.rl * dim * 2            # reduce-scatter staging: one bf16 slot per source rank
        self.off_x = _FLAG_BYTES
        self.off_stage = self.off_x + (x_bytes + 255) // 256 * 256
        total = self.off_stage + stage_bytes
        self.calls = 0
        if mode == "fused":
            native.load(True)
            self.symm = symm if symm is not None else SymmetricBuffer.create(total, group, self.device, False)
            assert self.symm.local.numel() >= total
            self.flags = self.symm.view(0, 64, torch.int32)
            self.x_all = self.symm.view(self.off_x, rows_total * dim, dtype).view(rows_total, dim)
            self.stage = self.symm.view(self.off_stage, N * self.rl * dim, dtype).view(N, self.rl, dim)
            self.ready = torch.zeros(8, dtype=torch.int32, device=self.device)
            chunk = self.rl * dim * 2
            base = self.symm.ptrs_at(self.off_x)
            self.gather_ptrs = [base[c] + c * chunk for c in range(N)]      # rank c's own rows inside ITS buffer

    @staticmethod
    def symm_bytes(rows_total, dim, world) -> int:
        return _FLAG_BYTES + (rows_total * dim * 2 + 255) // 256 * 256 + rows_total * dim * 2 + 256

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
            o = native.ops()
            fptrs = self.symm.ptrs_at(0)
            if self.calls > 0:
                o.flag_wait(self.flags, SLOT_X_DONE, N, self.calls, None)      # peers finished reading my previous rows
            self.calls += 1
            ep = self.calls
            self.x_all[r * rl:(r + 1) * rl].copy_(x2)
            o.flag_barrier(fptrs, self.flags, SLOT_X_READY, r, ep, None)
            h = _gemm([self.x_all], [w1_shard], bias=b1_shard, act=act_code(act),
                      gather_ptrs=self.gather_ptrs, gather_cfg=[r, 0, rl, rl * self.D * 2],
                      gather_dst=self.x_all, gather_ready=self.ready)
            o.flag_signal(fptrs, SLOT_X_DONE, r, ep, self.flags, None)
            # partial rows go straight into slot r of the row owner's staging buffer (bf16 vector stores over NVLink)
            _gemm([h], [w2_shard], route_ptrs=self.symm.ptrs_at(self.off_stage), route_cfg=[rl, self.D, r])
            res = _flat2d(residual).contiguous() if residual is not None else None
            y = o.rs_finalize(fptrs, self.flags, SLOT_RS_DONE, ep, r, self.stage, b2, res, gate, rows_per_group, None)
            return y.reshape(x_local.shape)
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
