"""Multi-GPU inference of the LTX-2-shaped video DiT with its tokens sharded over the ranks.

Every rank keeps 1/N of the latent tokens (rows) of ONE sample and all weights except the feed-forward ones:

* self-attention - Ulysses: the packed QKV projection, the full-width QK RMSNorm and the rotary embedding run on the local
  rows; the rows-to-heads all-to-all is a pull of each peer's re-packed block over NVLink (one gather kernel after a flag
  barrier); attention runs on all tokens for this rank's heads and its epilogue stores every output row straight into the
  token owner's buffer (the inverse all-to-all fused into the attention kernel).
* text cross-attention - local: queries are the local rows, the context is replicated.
* feed-forward - tensor parallel over the hidden width: the all-gather of the rows happens inside the first GEMM, the
  second GEMM's epilogue stores partial rows into the row owner's staging buffer, a tail kernel sums them and applies
  bias, gate and residual (``TPContext.mlp``).

``mode="nccl"`` performs the same data movement with ``all_to_all_single`` / ``all_gather`` / ``reduce_scatter``: the
baseline. The reference runs this model on one GPU only (serenitymojo/models/dit/ltx2_dit.mojo:518-652 is the block whose
op order is kept here)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import ops
from ..models.layers import packed_projection, timestep_embedding
from ..models.video_dit import VideoDiT
from ..ops import native
from .symm import SymmetricBuffer
from .tensor_parallel import TPContext, shard_mlp_weights

SLOT_SEND, SLOT_ATT = 0, 1
_FLAG_BYTES = 512


class ParallelVideoDiT:
    def __init__(self, model: VideoDiT, grid: Tuple[int, int, int], group=None, mode: str = "fused", device=None):
        self.model, self.grid, self.mode, self.group = model, grid, mode, group
        cfg = model.cfg
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = N = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.S = S = grid[0] * grid[1] * grid[2]
        self.D, self.H, self.Dh = cfg.hidden, cfg.heads, cfg.head_dim
        assert S % N == 0 and self.H % N == 0 and cfg.ffn_hidden % N == 0
        self.Sl, self.Hl = S // N, self.H // N
        self.Dl = self.Hl * self.Dh
        self.tp = TPContext(S, self.D, group, mode, device=self.device)
        self.block_bytes = self.Sl * 3 * self.Dl * 2                       # what one rank sends to one peer
        self.off_send = _FLAG_BYTES
        self.off_att = self.off_send + (N * self.block_bytes + 255) // 256 * 256
        total = self.off_att + self.Sl * self.D * 2
        self.calls = 0
        if mode == "fused" and N > 1:
            native.load(True)
            self.symm = SymmetricBuffer.create(total, group, self.device, False)
            self.flags = self.symm.view(0, 64, torch.int32)
            self.send = self.symm.view(self.off_send, N * self.Sl * 3 * self.Dl, torch.bfloat16).view(N, self.Sl, 3, self.Dl)
            self.attn_x = self.symm.view(self.off_att, self.Sl * self.D, torch.bfloat16).view(1, self.Sl, self.D)
        else:
            self.symm = None
        self.recv = torch.empty(N, self.Sl, 3 * self.Dl, dtype=torch.bfloat16, device=self.device)
        self.ff = []
        for blk in model.transformer_blocks:
            l1, l2 = blk.ff.net["0"].proj, blk.ff.net["2"]
            assert hasattr(l1, "slots") and (self.symm is None or l1.weight.dtype == torch.bfloat16), \
                "the tensor-parallel feed-forward takes plain (bf16 on the fused path) linears, not fp8-resident ones"
            self.ff.append(shard_mlp_weights(l1.weight.detach(), l1.bias.detach() if l1.bias is not None else None,
                                             l2.weight.detach(), self.rank, N) + (l2.bias.detach() if l2.bias is not None else None,))

    def shard(self, x: torch.Tensor) -> torch.Tensor:
        return x[:, self.rank * self.Sl:(self.rank + 1) * self.Sl].contiguous()

    def gather(self, x_local: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x_local
        parts = [torch.empty_like(x_local) for _ in range(self.world)]
        dist.all_gather(parts, x_local.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)

    # ---- self-attention over all tokens for this rank's heads -------------------------------------------------
    def _self_attention(self, qkv: torch.Tensor) -> torch.Tensor:
        """qkv: [1, Sl, 3D] local rows, q / k already normalised and rotated. Returns [1, Sl, D] attention rows."""
        N, r, Sl, Dl, D = self.world, self.rank, self.Sl, self.Dl, self.D
        Hl, Dh = self.Hl, self.Dh
        scale = 1.0 / (Dh ** 0.5)
        packed = qkv.view(Sl, 3, N, Dl).permute(2, 0, 1, 3)                                   # [dst rank, row, q|k|v, Dl]
        if N == 1:
            q, k, v = (qkv.view(1, Sl, 3, Hl, Dh)[:, :, i] for i in range(3))
            return ops.attention(q, k, v, scale).reshape(1, Sl, D)
        if self.symm is None:
            send = packed.contiguous()
            recv = torch.empty_like(send)
            dist.all_to_all_single(recv, send, group=self.group)                              # recv[src] = its rows, my heads
            g = recv.view(1, N * Sl, 3, Hl, Dh)
            o = ops.attention(g[:, :, 0], g[:, :, 1], g[:, :, 2], scale).reshape(N, Sl, Dl)   # [row owner, row, my head cols]
            back = torch.empty_like(o)
            dist.all_to_all_single(back, o.contiguous(), group=self.group)                    # back[src] = my rows, its heads
            return back.permute(1, 0, 2).reshape(1, Sl, D)
        o_ = native.ops()
        fptrs = self.symm.ptrs_at(0)
        self.calls += 1
        ep = self.calls
        self.send.copy_(packed)
        o_.flag_barrier(fptrs, self.flags, SLOT_SEND, r, ep, None)                             # every rank's blocks are in place
        o_.peer_gather(self.symm.ptrs_at(self.off_send + r * self.block_bytes), self.recv, self.block_bytes, r, True)
        g = self.recv.view(1, N * Sl, 3, Hl, Dh)
        col = r * Dl * 2
        route = [p + col for p in self.symm.ptrs_at(self.off_att)]
        o_.attention_fwd(g[:, :, 0], g[:, :, 1], g[:, :, 2], scale, None, False, None, route, route,
                         [1, 0, Sl, Sl * D, D, Dh])                                            # row t -> owner t // Sl, my head columns
        o_.flag_barrier(fptrs, self.flags, SLOT_ATT, r, ep, None)                              # every rank's heads have landed here
        return self.attn_x

    # ---- one block ------------------------------------------------------------------------------------------------
    def _block(self, i: int, x, ctx, temb6, cos, sin, ctx_len):
        blk = self.model.transformer_blocks[i]
        cfg = self.model.cfg
        D, H, Dh, Sl = self.D, self.H, self.Dh, self.Sl
        m = (blk.scale_shift_table[None].float() + temb6.float()).to(x.dtype)
        sh1, sc1, g1, sh2, sc2, g2 = [m[:, j] for j in range(6)]
        a = blk.attn1
        xn = ops.norm_modulate(x, scale=sc1, shift=sh1, eps=1e-6, rms=True)
        qkv = packed_projection(xn, (a.to_q, a.to_k, a.to_v))
        qkv[..., 0:D] = a.q_norm(qkv[..., 0:D])
        qkv[..., D:2 * D] = a.k_norm(qkv[..., D:2 * D])
        qkv = ops.qk_norm_rope(qkv, H, Dh, None, None, cos, sin, interleaved=False, do_norm=False, pos_offset=self.rank * Sl)
        o = self._self_attention(qkv)
        if hasattr(a, "to_gate_logits"):
            g = 2.0 * torch.sigmoid(a.to_gate_logits(xn).float())                            # [1, Sl, H]
            o = (o.view(1, Sl, H, Dh).float() * g[..., None]).to(x.dtype).view(1, Sl, D)
        x = a.to_out[0](o, residual=x, gate=g1, rows_per_group=Sl)
        h = blk.attn2(ops.norm_modulate(x, eps=1e-6, rms=True), ctx, kv_len=ctx_len)
        x = blk.attn2.to_out[0](h, residual=x)
        w1s, b1s, w2s, b2 = self.ff[i]
        xn2 = ops.norm_modulate(x, scale=sc2, shift=sh2, eps=1e-6, rms=True)
        y = self.tp.mlp(xn2[0], w1s, b1s, w2s, b2, "gelu_tanh", residual=x[0], gate=g2, rows_per_group=Sl)
        return y[None]

    @torch.no_grad()
    def forward(self, x_local, context, t, ctx_len: Optional[torch.Tensor] = None):
        """x_local: this rank's [1, S/N, C] latent tokens; context [1, T, ctx_dim] and t [1] replicated."""
        mdl, cfg = self.model, self.model.cfg
        assert x_local.shape[0] == 1 and x_local.shape[1] == self.Sl, "one sample, rows sharded"
        D = cfg.hidden
        dt = mdl.patchify_proj.weight.dtype
        cos, sin = ops.rope_table(mdl.make_ids(*self.grid, device=x_local.device), cfg.axes_dim, cfg.theta)
        te = mdl.adaln_single.emb.timestep_embedder
        emb = te.linear_2(te.linear_1(timestep_embedding(t, 256).to(dt), act="silu"))
        temb6 = mdl.adaln_single.linear(ops.activation(emb, "silu")).reshape(1, 6, D)
        h = mdl.patchify_proj(x_local.to(dt))
        cp = mdl.caption_projection
        ctx = cp.linear_2(cp.linear_1(context.to(dt), act="gelu_tanh"))
        for i in range(len(mdl.transformer_blocks)):
            h = self._block(i, h, ctx, temb6, cos, sin, ctx_len)
        m = (mdl.scale_shift_table[None].float() + emb[:, None].float()).to(h.dtype)
        return mdl.proj_out(ops.norm_modulate(h, scale=m[:, 1], shift=m[:, 0], eps=1e-6))
