"""Mixture-of-experts primitives: token-choice top-k router, grouped expert SwiGLU FFN, gated scatter-add combine.

Design for this hardware: tokens are sorted by expert once (one argsort on the device, no host round trip), every
expert's rows are then a contiguous slice and its FFN is two tcgen05 GEMMs (gate|up fused as one paired-GLU GEMM, then
down); the combine is one ``index_add_`` in fp32. Routing semantics: per token the k largest router logits (ties to the
lower expert index), gating = softmax over the selected logits only (serenitymojo/ops/moe.mojo:1-45,71-140,343-440,535-600).
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import functional as F


def top_k_router(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """logits [T, E] -> (expert_ids [T*k] int64, gating [T*k] fp32), slot s = t*k + j, j ordered by descending logit."""
    T, E = logits.shape
    lf = logits.float()
    # stable descending sort: equal logits keep ascending expert index
    order = torch.sort(lf, dim=1, descending=True, stable=True).indices[:, :k]
    sel = torch.gather(lf, 1, order)
    gating = torch.softmax(sel, dim=1)
    return order.reshape(-1), gating.reshape(-1)


def grouped_expert_ffn(tokens: torch.Tensor, gate_w: torch.Tensor, up_w: torch.Tensor, down_w: torch.Tensor,
                       expert_ids: torch.Tensor, k: int) -> torch.Tensor:
    """tokens [T, H]; gate_w/up_w [E, F, H]; down_w [E, H, F]; expert_ids [T*k]. Returns expert_out [T*k, H]:
    slot s = (t, j) is down_e(silu(x_t gate_e^T) * (x_t up_e^T)) with e = expert_ids[s]."""
    T, H = tokens.shape
    E = gate_w.shape[0]
    slots = expert_ids.numel()
    order = torch.argsort(expert_ids, stable=True)                 # slots grouped by expert
    counts = torch.bincount(expert_ids, minlength=E).tolist()      # one small device->host read per call
    x_sorted = tokens[(order // k)]                                # gather rows once
    out_sorted = torch.empty(slots, H, dtype=tokens.dtype, device=tokens.device)
    lo = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        xs = x_sorted[lo:lo + n]
        w_gu = torch.cat((gate_w[e], up_w[e]), dim=0)              # [2F, H]: one GEMM, paired GLU epilogue on a GPU
        h = F.linear_glu(xs, w_gu, None, act="silu")
        out_sorted[lo:lo + n] = F.linear(h, down_w[e])
        lo += n
    out = torch.empty_like(out_sorted)
    out[order] = out_sorted
    return out


def gated_scatter_add(expert_out: torch.Tensor, gating: torch.Tensor, indices: torch.Tensor, accum: torch.Tensor) -> torch.Tensor:
    """accum[indices[s]] += expert_out[s] * gating[s] through an fp32 accumulator (the k slots of one token add up
    exactly); negative / out-of-range indices are skipped. Updates ``accum`` in place and returns it."""
    ok = (indices >= 0) & (indices < accum.shape[0])
    acc = accum.float()
    acc.index_add_(0, indices[ok], expert_out[ok].float() * gating[ok].float()[:, None])
    accum.copy_(acc.to(accum.dtype))
    return accum


def moe_ffn(tokens: torch.Tensor, router_w: torch.Tensor, gate_w, up_w, down_w, k: int = 2) -> torch.Tensor:
    """Full layer: router logits -> top-k -> grouped FFN -> weighted combine. tokens [T, H], router_w [E, H]."""
    logits = F.linear(tokens, router_w)
    ids, gating = top_k_router(logits, k)
    eo = grouped_expert_ffn(tokens, gate_w, up_w, down_w, ids, k)
    out = torch.zeros_like(tokens)
    token_of_slot = torch.arange(tokens.shape[0], device=tokens.device).repeat_interleave(k)
    return gated_scatter_add(eo, gating, token_of_slot, out)


# ---- expert-choice routing (each expert picks its top-C tokens) ----------------------------------------------------------
def expert_choice_route(affinity: torch.Tensor, capacity: int, route_scale: float = 1.0):
    """affinity [B, E, S] (softmax over experts, transposed) -> (token index [E, B*C] into the flat [B*S] token list,
    gate [E, B*C] fp32). Every (sample, expert) takes its ``capacity`` highest-affinity tokens (ties to the lower token
    index); a token's gates are divided by their sum over all experts that picked it, then multiplied by ``route_scale``
    (serenitymojo/models/dit/nucleus_moe.mojo:27-110)."""
    B, E, S = affinity.shape
    if not 1 <= capacity <= S:
        raise ValueError("expert_choice_route: capacity must lie in [1, tokens per sample]")
    a = affinity.float()
    order = torch.sort(a, dim=2, descending=True, stable=True).indices[:, :, :capacity]        # [B, E, C]
    w = torch.gather(a, 2, order)
    idx = (order + (torch.arange(B, device=a.device) * S)[:, None, None]).permute(1, 0, 2).reshape(E, B * capacity)
    w = w.permute(1, 0, 2).reshape(E, B * capacity)
    tsum = torch.zeros(B * S, dtype=torch.float32, device=a.device).index_add_(0, idx.reshape(-1), w.reshape(-1))
    gate = w / (tsum[idx] + 1e-12) * route_scale
    return idx, gate


def expert_choice_ffn(tokens: torch.Tensor, idx: torch.Tensor, gate: torch.Tensor, gate_up_w: torch.Tensor,
                      down_w: torch.Tensor) -> torch.Tensor:
    """tokens [T, D]; idx / gate [E, P] from ``expert_choice_route``; gate_up_w [E, D, 2I] (gate columns then up columns,
    ``x @ W`` layout); down_w [E, I, D]. Returns sum over picks of gate * (silu(x Wg) * (x Wu)) Wd, accumulated per token
    in fp32, in the dtype of ``tokens``. The experts run as two batched GEMMs over the gathered [E, P, D] rows."""
    E, P = idx.shape
    T, D = tokens.shape
    x = tokens[idx.reshape(-1)].reshape(E, P, D)
    gu = torch.bmm(x, gate_up_w.to(x.dtype))                                              # [E, P, 2I]
    inner = gu.shape[-1] // 2
    h = torch.nn.functional.silu(gu[..., :inner].float()).to(x.dtype) * gu[..., inner:]
    y = torch.bmm(h, down_w.to(x.dtype)).float() * gate[..., None]                          # [E, P, D]
    out = torch.zeros(T, D, dtype=torch.float32, device=tokens.device).index_add_(0, idx.reshape(-1), y.reshape(E * P, D))
    return out.to(tokens.dtype)
