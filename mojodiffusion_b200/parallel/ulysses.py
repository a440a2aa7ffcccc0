"""Ulysses sequence parallelism for joint (text + image) attention, fused into the neighbouring kernels.

Every rank keeps 1/N of the text tokens and 1/N of the image tokens for all per-token work (norms, projections,
MLPs, the sampler update). Around attention the layout flips to "all tokens, 1/N of the heads":

* forward all-to-all  = the QKV projection's own epilogue: each 32-column slab of a GEMM output tile is stored
  straight into the buffer of the rank that owns that head (plain peer stores over NVLink into symmetric memory),
  at the token's global row. No separate all-to-all kernel, no staging copy.
* QK-RMSNorm + RoPE and attention then run on the gathered [B, S, 3 * H/N * Dh] buffer of the local heads.
* inverse all-to-all = the attention kernel's own epilogue: each finished query row is stored into the token
  owner's [B, S/N, D] buffer at this rank's head columns, where the output projection (a plain local GEMM) reads it.

Two epoch flags per layer order the phases (producer signals after its kernel, consumer waits before its kernel;
bounded waits). ``mode="nccl"`` performs the same layout changes with ``all_to_all_single``: that is the baseline
and the correctness oracle of the fused path.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .. import ops
from ..ops import native
from ..ops.functional import _flat2d, _gemm
from ..utils.tracing import nvtx_range
from .symm import SymmetricBuffer

SLOT_QKV, SLOT_ATTN = 4, 5
_FLAG_BYTES = 512


class UlyssesContext:
    def __init__(self, B: int, S_txt: int, S_img: int, heads: int, head_dim: int, group=None, mode: str = "fused",
                 symm: Optional[SymmetricBuffer] = None, device=None, dtype=torch.bfloat16):
        self.mode = mode
        self.group = group
        if symm is not None:
            self.rank, self.world = symm.rank, symm.world
        else:
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        N = self.world
        assert heads % N == 0 and S_txt % N == 0 and S_img % N == 0, "heads and token counts must divide by the SP size"
        self.B, self.S_txt, self.S_img, self.H, self.Dh = B, S_txt, S_img, heads, head_dim
        self.S = S_txt + S_img
        self.St, self.Si = S_txt // N, S_img // N
        self.Sl = self.St + self.Si
        self.Hl = heads // N
        self.D = heads * head_dim
        self.Dl = self.Hl * head_dim
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.dtype = dtype
        self.epoch = 0
        qkv_bytes = B * self.S * 3 * self.Dl * 2
        att_bytes = B * self.Sl * self.D * 2
        self.off_qkv = _FLAG_BYTES
        self.off_att = _FLAG_BYTES + (qkv_bytes + 255) // 256 * 256
        total = self.off_att + att_bytes
        if mode == "fused":
            native.load(True)
            self.symm = symm if symm is not None else SymmetricBuffer.create(total, group, self.device, False)
            assert self.symm.local.numel() >= total
            self.flags = self.symm.view(0, 64, torch.int32)
            # device-side epoch counters (signals | waits): the flag sequence survives CUDA-graph replay
            self.counters = torch.zeros(16, dtype=torch.int32, device=self.device)
            self.qkv_g = self.symm.view(self.off_qkv, B * self.S * 3 * self.Dl, dtype).view(B, self.S, 3 * self.Dl)
            self.attn_x = self.symm.view(self.off_att, B * self.Sl * self.D, dtype).view(B, self.Sl, self.D)
        else:
            self.symm = None
            self.qkv_g = torch.empty(B, self.S, 3 * self.Dl, dtype=dtype, device=self.device)
            self.attn_x = torch.empty(B, self.Sl, self.D, dtype=dtype, device=self.device)
            self._local_qkv = {}

    @staticmethod
    def symm_bytes(B, S_txt, S_img, heads, head_dim, world) -> int:
        S, Dl, D = S_txt + S_img, heads // world * head_dim, heads * head_dim
        return _FLAG_BYTES + (B * S * 3 * Dl * 2 + 255) // 256 * 256 + B * (S // world) * D * 2 + 256

    # ---- forward all-to-all inside the QKV projection -----------------------------------------------------
    def scatter_qkv(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], part: str) -> None:
        """x: this rank's [B, S_part/N, D] (already normalised / modulated) rows of stream ``part`` ("txt" or "img");
        weight: [3D, D] packed (q | k | v) x (head, Dh). Output lands in every rank's gathered qkv buffer."""
        Sp = self.St if part == "txt" else self.Si
        base = 0 if part == "txt" else self.S_txt
        x2 = _flat2d(x)
        if self.mode == "fused":
            with nvtx_range("collective/ulysses/qkv_scatter_gemm"):
                _gemm([x2], [weight], bias=bias, route_ptrs=self.symm.ptrs_at(self.off_qkv),
                      route_cfg=[self.Dl, self.D, base + self.rank * Sp, Sp, self.S, 3 * self.Dl])
        else:
            self._local_qkv[part] = ops.linear(x2, weight, bias).view(self.B, Sp, 3, self.world, self.Dl)

    def scatter_qkv_joint(self, x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]) -> None:
        """x: this rank's [B, St + Si, D] rows with the text rows of every sample first (the single-stream layout). One GEMM
        scatters both streams: its epilogue sends rows below ``St`` to the text range and the others to the image range of
        the gathered buffer, so the input is not sliced (a slice of a batch > 1 is not contiguous and would be copied)."""
        if self.mode != "fused":
            self.scatter_qkv(x[:, :self.St], weight, bias, "txt")
            self.scatter_qkv(x[:, self.St:], weight, bias, "img")
            return
        with nvtx_range("collective/ulysses/qkv_scatter_gemm"):
            _gemm([_flat2d(x)], [weight], bias=bias, route_ptrs=self.symm.ptrs_at(self.off_qkv),
                  route_cfg=[self.Dl, self.D, self.rank * self.St, self.Sl, self.S, 3 * self.Dl,
                             self.St, self.S_txt + self.rank * self.Si])

    def finish_scatter(self) -> None:
        """Publish "my projections have landed everywhere" (fused) / run the all-to-all (nccl)."""
        if self.mode == "fused":
            native.ops().flag_signal(self.symm.ptrs_at(0), SLOT_QKV, self.rank, 0, self.flags, self.counters)
            return
        N = self.world
        for part, Sp, base in (("txt", self.St, 0), ("img", self.Si, self.S_txt)):
            loc = self._local_qkv[part]                                   # [B, Sp, 3, N, Dl]
            send = loc.permute(3, 0, 1, 2, 4).contiguous()                # [N(dst), B, Sp, 3, Dl]
            recv = torch.empty_like(send)                                 # [N(src), B, Sp, 3, Dl]
            if N > 1:
                dist.all_to_all_single(recv, send, group=self.group)
            else:
                recv = send
            g = recv.permute(1, 0, 2, 3, 4).reshape(self.B, N * Sp, 3 * self.Dl)
            self.qkv_g[:, base:base + N * Sp] = g

    # ---- attention on the local heads, inverse all-to-all in its epilogue ------------------------------------
    def attention(self, wq_txt, wk_txt, wq_img, wk_img, cos, sin, interleaved: bool = True) -> None:
        Hl, Dh, Dl = self.Hl, self.Dh, self.Dl
        if self.mode == "fused":
            native.ops().flag_wait(self.flags, SLOT_QKV, self.world, 0, self.counters)
        g = self.qkv_g
        ops.qk_norm_rope(g[:, :self.S_txt], Hl, Dh, wq_txt, wk_txt, cos, sin, interleaved=interleaved, pos_offset=0)
        ops.qk_norm_rope(g[:, self.S_txt:], Hl, Dh, wq_img, wk_img, cos, sin, interleaved=interleaved,
                         pos_offset=self.S_txt)
        q = g[..., 0:Dl].unflatten(-1, (Hl, Dh))
        k = g[..., Dl:2 * Dl].unflatten(-1, (Hl, Dh))
        v = g[..., 2 * Dl:3 * Dl].unflatten(-1, (Hl, Dh))
        scale = 1.0 / (Dh ** 0.5)
        if self.mode == "fused":
            col = self.rank * Dl * 2                       # this rank's head columns inside the owner's row (bytes)
            base = self.symm.ptrs_at(self.off_att)
            ra = [p + col for p in base]
            rb = [p + self.St * self.D * 2 + col for p in base]
            with nvtx_range("collective/ulysses/attention_row_scatter"):
                native.ops().attention_fwd(q, k, v, scale, None, False, None, ra, rb,
                                           [self.St, self.S_txt, self.Si, self.Sl * self.D, self.D, Dh])
            native.ops().flag_signal(self.symm.ptrs_at(0), SLOT_ATTN, self.rank, 0, self.flags, self.counters)
        else:
            o = ops.attention(q, k, v, scale).reshape(self.B, self.S, Dl)
            N = self.world
            for Sp, base, dst0 in ((self.St, 0, 0), (self.Si, self.S_txt, self.St)):
                send = o[:, base:base + N * Sp].reshape(self.B, N, Sp, Dl).permute(1, 0, 2, 3).contiguous()
                recv = torch.empty_like(send)
                if N > 1:
                    dist.all_to_all_single(recv, send, group=self.group)
                else:
                    recv = send
                self.attn_x[:, dst0:dst0 + Sp] = recv.permute(1, 2, 0, 3).reshape(self.B, Sp, self.D)

    def finish_attention(self) -> torch.Tensor:
        """Wait until every rank's heads have landed; returns this rank's [B, S_txt/N + S_img/N, D] attention rows."""
        if self.mode == "fused":
            native.ops().flag_wait(self.flags, SLOT_ATTN, self.world, 0, self.counters)
        return self.attn_x

    # ---- helpers ------------------------------------------------------------------------------------------------
    def shard(self, x: torch.Tensor, part: str) -> torch.Tensor:
        """This rank's contiguous token slice of a full [B, S_part, ...] tensor."""
        Sp = self.St if part == "txt" else self.Si
        return x[:, self.rank * Sp:(self.rank + 1) * Sp].contiguous()

    def gather(self, x_local: torch.Tensor) -> torch.Tensor:
        """All-gather token shards [B, S_part/N, C] -> [B, S_part, C] (end of sampling only)."""
        if self.world == 1 or not dist.is_initialized():
            return x_local
        parts = [torch.empty_like(x_local) for _ in range(self.world)]
        dist.all_gather(parts, x_local.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)
