"""Plain PyTorch references of every op in this package.

They are the CPU path (autograd-capable, any dtype) and the numerics oracle of the CUDA kernels: the GPU
tests run a kernel and compare against the function of the same name here evaluated in fp32.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Sequence

import torch
import torch.nn.functional as F

ACT_NONE, ACT_GELU_TANH, ACT_SILU, ACT_GELU_ERF, ACT_SIGMOID, ACT_RELU, ACT_TANH = range(7)

_ACT_NAMES = {
    None: ACT_NONE, "none": ACT_NONE, "identity": ACT_NONE, "gelu_tanh": ACT_GELU_TANH, "gelu": ACT_GELU_ERF,
    "gelu_erf": ACT_GELU_ERF, "silu": ACT_SILU, "swish": ACT_SILU, "sigmoid": ACT_SIGMOID, "relu": ACT_RELU,
    "tanh": ACT_TANH,
}


def act_code(act) -> int:
    if isinstance(act, int):
        return act
    return _ACT_NAMES[act]


def activation(x: torch.Tensor, act) -> torch.Tensor:
    a = act_code(act)
    if a == ACT_NONE:
        return x
    if a == ACT_GELU_TANH:
        return F.gelu(x, approximate="tanh")
    if a == ACT_GELU_ERF:
        return F.gelu(x)
    if a == ACT_SILU:
        return F.silu(x)
    if a == ACT_SIGMOID:
        return torch.sigmoid(x)
    if a == ACT_RELU:
        return F.relu(x)
    if a == ACT_TANH:
        return torch.tanh(x)
    raise ValueError(a)


def _library_mode(x: torch.Tensor, out_dtype=None) -> bool:
    """bf16 tensors on a GPU while the package is forced off its own kernels (``MDB200_FORCE_REFERENCE=1``): the hot
    ops then run as an ordinary PyTorch bf16 program (cuBLAS ``F.linear``, fused SDPA, ``F.layer_norm``, element-wise
    ops in bf16) instead of the fp32 oracle arithmetic below. That is the same-box library baseline of ``bench.py``."""
    return x.is_cuda and x.dtype == torch.bfloat16 and out_dtype is None and os.environ.get("MDB200_FORCE_REFERENCE") == "1"


def _grouped(v: torch.Tensor, y: torch.Tensor, rows_per_group: int) -> torch.Tensor:
    """View of y [rows, D] as [groups, rows_per_group, D] beside v [groups, 1, D] (no gather)."""
    return y.view(v.shape[0], -1, y.shape[-1]) if v.shape[0] > 1 else y.view(1, -1, y.shape[-1])


def _group_expand(v: torch.Tensor, rows: int, rows_per_group: int) -> torch.Tensor:
    """[groups, D] -> [rows, D] where row r uses group r // rows_per_group."""
    if v.shape[0] == 1:
        return v.expand(rows, -1)
    idx = torch.arange(rows, device=v.device) // rows_per_group
    return v[idx]


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
           residual: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, rows_per_group: int = 1,
           extra: Sequence[tuple] = (), out_dtype=None) -> torch.Tensor:
    """``act(x @ w.T + sum_i a_i @ b_i.T + bias)``, then ``residual + gate[group] * value``. 2-D operands."""
    if _library_mode(x, out_dtype):
        y = F.linear(x, w, bias)
        for a2, b2 in extra:
            y = y + F.linear(a2, b2)
        y = activation(y, act)
        if gate is not None:
            g = gate.to(y.dtype)
            y = (_grouped(g, y, rows_per_group) * g[:, None, :]).view(y.shape)
        if residual is not None:
            y = y + residual
        return y
    y = x.float() @ w.float().t()
    for a2, b2 in extra:
        y = y + a2.float() @ b2.float().t()
    if bias is not None:
        y = y + bias.float()
    y = activation(y, act)
    if gate is not None:
        y = y * _group_expand(gate.float(), y.shape[0], rows_per_group)
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def linear_glu(x, w, bias=None, act="silu", act_on_second=False, out_dtype=None):
    """Paired projection: ``h = x @ w.T + b``; halves (a, b) -> ``act(a) * b`` (SwiGLU) or ``a * act(b)`` (GEGLU)."""
    if _library_mode(x, out_dtype):
        a, b = F.linear(x, w, bias).chunk(2, dim=-1)
        return a * activation(b, act) if act_on_second else activation(a, act) * b
    h = x.float() @ w.float().t()
    if bias is not None:
        h = h + bias.float()
    a, b = h.chunk(2, dim=-1)
    y = a * activation(b, act) if act_on_second else activation(a, act) * b
    return y.to(out_dtype or x.dtype)


def glu(h, act="silu", act_on_second=False):
    a, b = h.float().chunk(2, dim=-1)
    y = a * activation(b, act) if act_on_second else activation(a, act) * b
    return y.to(h.dtype)


def norm_modulate(x, weight=None, bias=None, scale=None, shift=None, rows_per_group: int = 1, eps: float = 1e-6,
                  rms: bool = False):
    """LayerNorm or RMSNorm over the last dim, optional affine, then ``* (1 + scale[g]) + shift[g]``. x: [rows, D]."""
    if _library_mode(x):
        D = x.shape[-1]
        if rms:
            y = F.rms_norm(x, (D,), weight, eps)
            if bias is not None:
                y = y + bias
        else:
            y = F.layer_norm(x, (D,), weight, bias, eps)
        if scale is not None:
            sc = scale.to(y.dtype)
            y = (_grouped(sc, y, rows_per_group) * (1 + sc[:, None, :])).view(y.shape)
        if shift is not None:
            sh = shift.to(y.dtype)
            y = (_grouped(sh, y, rows_per_group) + sh[:, None, :]).view(y.shape)
        return y
    xf = x.float()
    if rms:
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    else:
        mu = xf.mean(-1, keepdim=True)
        var = (xf - mu).pow(2).mean(-1, keepdim=True)
        y = (xf - mu) * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight.float()
    if bias is not None:
        y = y + bias.float()
    if scale is not None:
        y = y * (1.0 + _group_expand(scale.float(), y.shape[0], rows_per_group))
    if shift is not None:
        y = y + _group_expand(shift.float(), y.shape[0], rows_per_group)
    return y.to(x.dtype)


def rope_table(pos: torch.Tensor, axes_dim: Sequence[int], theta: float = 10000.0):
    """cos/sin [T, sum(axes_dim)/2] from per-token positions [T, n_axes] (fp64 angle, like the kernel)."""
    cols_c, cols_s = [], []
    for a, d in enumerate(axes_dim):
        half = d // 2
        i = torch.arange(half, dtype=torch.float64, device=pos.device)
        freq = torch.exp(-math.log(theta) * i / half)
        ang = pos[:, a].double()[:, None] * freq[None, :]
        cols_c.append(torch.cos(ang))
        cols_s.append(torch.sin(ang))
    return torch.cat(cols_c, -1).float(), torch.cat(cols_s, -1).float()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, interleaved: bool = True) -> torch.Tensor:
    """x: [..., S, H, Dh]; cos/sin: [S, Dh/2]. Interleaved pairs (2i, 2i+1) or half-split pairs (i, i+Dh/2)."""
    xf = x.float()
    c = cos[:, None, :]
    s = sin[:, None, :]
    if interleaved:
        a = xf[..., 0::2]
        b = xf[..., 1::2]
        ra = a * c - b * s
        rb = a * s + b * c
        out = torch.stack((ra, rb), dim=-1).flatten(-2)
    else:
        half = xf.shape[-1] // 2
        a = xf[..., :half]
        b = xf[..., half:]
        out = torch.cat((a * c - b * s, b * c + a * s), dim=-1)
    return out.to(x.dtype)


def rms_norm_heads(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float()
    return y.to(x.dtype)


def qk_norm_rope(q, k, wq=None, wk=None, cos=None, sin=None, eps=1e-6, interleaved=True, do_norm=True,
                 rope_start: int = 0):
    """q, k: [B, S, H, Dh] -> per-head RMSNorm (weights [Dh]) then rotary on tokens >= rope_start."""
    if do_norm:
        q = rms_norm_heads(q, wq, eps)
        k = rms_norm_heads(k, wk, eps)
    if cos is not None:
        if rope_start > 0:
            q = torch.cat((q[:, :rope_start], apply_rope(q[:, rope_start:], cos[rope_start:], sin[rope_start:], interleaved)), 1)
            k = torch.cat((k[:, :rope_start], apply_rope(k[:, rope_start:], cos[rope_start:], sin[rope_start:], interleaved)), 1)
        else:
            q = apply_rope(q, cos, sin, interleaved)
            k = apply_rope(k, cos, sin, interleaved)
    return q, k


def attention(q, k, v, scale: Optional[float] = None, kv_len: Optional[torch.Tensor] = None,
              return_lse: bool = False):
    """q: [B, Sq, H, Dh], k/v: [B, Skv, H, Dh] -> [B, Sq, H, Dh]; keys >= kv_len[b] are masked."""
    B, Sq, H, Dh = q.shape
    Skv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(Dh)
    if q.is_cuda and kv_len is None and not return_lse:
        # library baseline on a GPU: the flash / cuDNN kernel torch selects, not an S x S fp32 score matrix
        o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(),
                                                             v.transpose(1, 2).contiguous(), scale=scale)
        return o.transpose(1, 2).contiguous()
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    if kv_len is not None:
        mask = torch.arange(Skv, device=q.device)[None, :] >= kv_len.to(q.device)[:, None]
        s = s.masked_fill(mask[:, None, None, :], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    o = torch.einsum("bhqk,bkhd->bqhd", p, v.float()).to(q.dtype)
    if return_lse:
        return o, lse
    return o


def gate_residual(x, y, gate=None, rows_per_group: int = 1, tanh_gate: bool = False):
    """x + gate[g] * y over [rows, D] (gate None: x + y)."""
    if _library_mode(x) and not tanh_gate:
        if gate is None:
            return x + y
        g = gate.to(y.dtype).reshape(-1, y.shape[-1])
        y2 = y.reshape(-1, y.shape[-1])
        return x + (_grouped(g, y2, rows_per_group) * g[:, None, :]).view(y.shape)
    if gate is None:
        return (x.float() + y.float()).to(x.dtype)
    g = gate.float()
    if tanh_gate:
        g = torch.tanh(g)
    x2 = x.reshape(-1, x.shape[-1]).float()
    y2 = y.reshape(-1, y.shape[-1]).float()
    out = x2 + _group_expand(g, x2.shape[0], rows_per_group) * y2
    return out.reshape(x.shape).to(x.dtype)


def cfg_combine(vc, vu, s: float, mode: int):
    """mode 0: vc; 1: vu + s (vc - vu) (textbook); 2: vc + s (vc - vu) (cond-anchored)."""
    if mode == 0:
        return vc.float()
    if mode == 1:
        return vu.float() + s * (vc.float() - vu.float())
    return vc.float() + s * (vc.float() - vu.float())


def cfg_euler(x: torch.Tensor, vc, vu, dt: float, s: float = 1.0, mode: int = 0):
    """fp32 latent update: x + dt * CFG(vc, vu)."""
    return x + dt * cfg_combine(vc, vu, s, mode)


def flow_match(x0: torch.Tensor, eps: torch.Tensor, sigma: torch.Tensor):
    """x_t = (1 - sigma) x0 + sigma eps (bf16 on GPU), target = eps - x0 (fp32)."""
    s = sigma.reshape(-1, *([1] * (x0.dim() - 1))).float()
    xt = (1.0 - s) * x0.float() + s * eps.float()
    return xt, eps.float() - x0.float()


def fp8_quant_rows(x: torch.Tensor):
    """Per-row absmax e4m3 quantisation: returns (q float8_e4m3fn, scale fp32 [rows])."""
    amax = x.float().abs().amax(dim=-1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (x.float() / scale[:, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q, scale


def fp8_dequant(q: torch.Tensor, row_scale=None, tensor_scale: float = 1.0):
    y = q.float()
    y = y * (row_scale.float()[:, None] if row_scale is not None else tensor_scale)
    return y.to(torch.bfloat16)


_E2M1 = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def _e8m0(scales: torch.Tensor) -> torch.Tensor:
    e = scales.to(torch.int32) - 127
    return torch.ldexp(torch.ones(e.shape, dtype=torch.float32, device=scales.device), e)


def mx_dequant(q: torch.Tensor, scales: torch.Tensor, fp4: bool = True) -> torch.Tensor:
    """MX block formats -> bf16 [n_blocks * 32]: ``scales`` uint8 E8M0 (2^(b - 127)) per 32 elements; fp4: ``q`` uint8 with
    two E2M1 values per byte, low nibble first (16 bytes per block); else ``q`` holds E4M3 bytes."""
    sc = _e8m0(scales.reshape(-1))
    if fp4:
        b = q.reshape(-1, 16).to(torch.int32)
        nib = torch.stack((b & 0xF, (b >> 4) & 0xF), dim=-1).reshape(-1, 32)
        lut = torch.tensor(_E2M1, dtype=torch.float32, device=q.device)
        v = lut[nib & 7] * torch.where((nib & 8) != 0, -1.0, 1.0)
    else:
        v = q.reshape(-1, 32).view(torch.float8_e4m3fn).float()
    return (v * sc[:, None]).reshape(-1).to(torch.bfloat16)


def mx_quant(x: torch.Tensor, fp4: bool = True):
    """bf16 -> (packed uint8, E8M0 scale bytes). Block exponent = floor(log2(absmax)) - emax (2 for E2M1, 8 for E4M3),
    elements rounded to nearest-even on the element grid with saturation."""
    v = x.float().reshape(-1, 32)
    amax = v.abs().amax(dim=1)
    e = torch.floor(torch.log2(amax.clamp_min(1e-45))).to(torch.int32) - (2 if fp4 else 8) + 127
    e = torch.where(amax > 0, e.clamp(0, 254), torch.zeros_like(e))
    sc = torch.ldexp(torch.ones(e.shape, dtype=torch.float32, device=x.device), e - 127)
    sc = torch.where(e == 0, torch.full_like(sc, 2.0 ** -127), sc)
    y = v / sc[:, None]
    if fp4:
        a = y.abs()
        bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0], device=x.device)
        # ties go to the even code: codes 0, 2, 4, 6 own their upper boundary, odd codes do not
        m = torch.zeros_like(a, dtype=torch.int32)
        for i, bnd in enumerate(bounds.tolist()):
            m = m + ((a > bnd) if i % 2 == 0 else (a >= bnd)).to(torch.int32)
        nib = m | ((y < 0) | ((y == 0) & torch.signbit(y))).to(torch.int32) * 8
        nib = nib.reshape(-1, 16, 2)
        q = (nib[..., 0] | (nib[..., 1] << 4)).to(torch.uint8).reshape(-1)
    else:
        q = y.clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).reshape(-1)
    return q, e.to(torch.uint8)


def mxfp8_quant_rows(x: torch.Tensor, pad_rows: int = 128):
    """bf16 [rows, K] -> (E4M3 bytes [rows, K], scale chunks [ceil(rows / pad) * pad / 128, K / 128, 512]) in the layout the
    block-scaled tensor-core instruction reads: byte (r % 32) * 16 + (r % 128 // 32) * 4 + (k32 % 4) of chunk
    (r // 128, k32 // 4); unused bytes are 127 (scale 1)."""
    rows, K = x.shape
    q, e = mx_quant(x.contiguous(), fp4=False)
    q = q.reshape(rows, K)
    e = e.reshape(rows, K // 32)
    padded = (rows + pad_rows - 1) // pad_rows * pad_rows
    sf = torch.full((padded // 128, K // 128, 512), 127, dtype=torch.uint8, device=x.device)
    r = torch.arange(rows, device=x.device)[:, None]
    k = torch.arange(K // 32, device=x.device)[None, :]
    sf[(r // 128).expand_as(e), (k // 4).expand_as(e), ((r % 32) * 16 + (r % 128 // 32) * 4 + (k % 4)).expand_as(e)] = e
    return q, sf


def mxfp8_scales_from_chunks(sf: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """Inverse of the chunk layout: scale bytes [rows, K / 32]."""
    r = torch.arange(rows, device=sf.device)[:, None]
    k = torch.arange(K // 32, device=sf.device)[None, :]
    return sf[(r // 128).expand(rows, K // 32), (k // 4).expand(rows, K // 32), ((r % 32) * 16 + (r % 128 // 32) * 4 + (k % 4)).expand(rows, K // 32)]


def gemm_mxfp8(a_q, sfa, b_q, sfb, bias=None):
    """fp32 product of the dequantised operands, rounded to bf16."""
    M, K = a_q.shape
    N = b_q.shape[0]
    a = mx_dequant(a_q.reshape(-1), mxfp8_scales_from_chunks(sfa, M, K).reshape(-1), fp4=False).float().reshape(M, K)
    b = mx_dequant(b_q.reshape(-1), mxfp8_scales_from_chunks(sfb, N, K).reshape(-1), fp4=False).float().reshape(N, K)
    y = a @ b.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(torch.bfloat16)


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, wd, step, grad_scale=1.0):
    """torch.optim.AdamW order, fp32 math; returns new (p, m, v)."""
    g = g.float() * grad_scale
    p = p.float() * (1.0 - lr * wd)
    m = beta1 * m.float() + (1 - beta1) * g
    v = beta2 * v.float() + (1 - beta2) * g * g
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    p = p - (lr / bc1) * (m / (v.sqrt() / math.sqrt(bc2) + eps))
    return p, m, v
