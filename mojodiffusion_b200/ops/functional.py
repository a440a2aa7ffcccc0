"""Public op layer: one function per op, dispatching on the device of its input.

* CUDA tensors run the hand-written sm_100a kernels through ``torch.ops.mdb200`` (bf16 activations). With
  autograd enabled, each op is a ``torch.autograd.Function`` whose backward is again native kernels
  (MN-major tcgen05 GEMMs for dx / dW, norm / activation / rope backward kernels).
* CPU tensors run the pure-torch references (any dtype, ordinary autograd): that is the path of the CPU
  unit tests and of the gloo multi-process plumbing tests.
"""
from __future__ import annotations

import math
from typing import Optional, Sequence

import torch

from . import native, reference as ref
from .reference import act_code

__all__ = [
    "linear", "linear_glu", "lora_linear", "attention", "norm_modulate", "qk_norm_rope", "rope_table", "activation",
    "glu", "gate_residual", "cfg_euler", "flow_match", "mse_loss", "randn", "fp8_quant_rows", "fp8_dequant", "mx_quant", "mx_dequant", "mxfp8_quant_rows", "gemm_mxfp8", "MXFP8Weight",
    "fp8_linear", "qkv_attention", "split_cols", "packed_attention_mlp",
]


def _ops():
    return native.ops()


def _flat2d(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1 or (x2.stride(0) % 8) or (x2.data_ptr() % 16):
        x2 = x2.contiguous()
    return x2


def _gemm(As, Bs, bias=None, residual=None, gate=None, rows_per_group=1, act=0, pair_offset=0, act_on_second=0,
          out=None, out_fp32=False, a_mn=False, b_mn=False, row_scale=None, col_scale=None, alpha=1.0,
          accumulate=False, bn=0, prof=None, route_ptrs=(), route_cfg=(), gather_ptrs=(), gather_cfg=(),
          gather_dst=None, gather_ready=None, split_k=0):
    return _ops().gemm(list(As), list(Bs), bias, residual, gate, rows_per_group, act, pair_offset, act_on_second, out,
                       out_fp32, a_mn, b_mn, row_scale, col_scale, alpha, accumulate, bn, prof, list(route_ptrs),
                       list(route_cfg), list(gather_ptrs), list(gather_cfg), gather_dst, gather_ready, split_k)


_sm_count = {}


def _num_sms(device) -> int:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    n = _sm_count.get(idx)
    if n is None:
        n = _sm_count[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def _gemm_skinny(A, B, a_mn=False, b_mn=False, alpha=1.0):
    """GEMM whose output has far fewer tiles than the GPU has SMs (LoRA down-projections and their gradients: N or M
    of 16..64 against a long reduction): the reduction is split across the idle SMs and the parts are added in fp32."""
    M = A.shape[1] if a_mn else A.shape[0]
    N = B.shape[1] if b_mn else B.shape[0]
    K = A.shape[0] if a_mn else A.shape[1]
    tiles = ((M + 127) // 128) * ((N + 63) // 64)
    kblocks = (K + 63) // 64
    split = min(_num_sms(A.device) // max(tiles, 1), kblocks // 4, 16)
    if split <= 1:
        return _gemm([A], [B], a_mn=a_mn, b_mn=b_mn, alpha=alpha)
    out = torch.zeros(M, N, dtype=torch.float32, device=A.device)
    _gemm([A], [B], a_mn=a_mn, b_mn=b_mn, alpha=alpha, out=out, out_fp32=True, split_k=split, bn=64)
    return out.to(A.dtype)


# --------------------------------------------------------------------------------------------
# linear family
# --------------------------------------------------------------------------------------------
class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, w, bias):
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        return _gemm([x2], [w], bias=bias)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy = _flat2d(dy)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _gemm([dy], [w], b_mn=True)
        if ctx.needs_input_grad[1]:
            dw = _gemm([dy], [x2], a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        return dx, dw, db


class _LoraLinearFn(torch.autograd.Function):
    """y = x W^T + b + scale * (x A^T) B^T with the up-projection folded into the base GEMM as a K segment."""

    @staticmethod
    def forward(ctx, x2, w, bias, A, B, scale):
        t = _gemm_skinny(x2, A)                    # [M, r]
        Bs = B if scale == 1.0 else (B.float() * scale).to(B.dtype)       # [N, r]
        y = _gemm([x2, t], [w, Bs], bias=bias)
        ctx.save_for_backward(x2, w, A, B, t, Bs)
        ctx.scale = scale
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w, A, B, t, Bs = ctx.saved_tensors
        dy = _flat2d(dy)
        dx = dw = db = dA = dB = None
        dt = _gemm_skinny(dy, Bs, b_mn=True)       # [M, r] (already scaled)
        if ctx.needs_input_grad[0]:
            dx = _gemm([dy, dt], [w, A], b_mn=True)
        if ctx.needs_input_grad[1]:
            dw = _gemm([dy], [x2], a_mn=True, b_mn=True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        if ctx.needs_input_grad[3]:
            dA = _gemm_skinny(dt, x2, a_mn=True, b_mn=True)           # [r, K]
        if ctx.needs_input_grad[4]:
            dB = _gemm_skinny(dy, t, a_mn=True, b_mn=True, alpha=ctx.scale)  # [N, r]
        return dx, dw, db, dA, dB, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
           residual: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None, rows_per_group: int = 1,
           extra: Sequence[tuple] = (), out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``act(x @ w.T [+ a_i @ b_i.T ...] + bias)`` then ``residual + gate[row // rows_per_group] * value``.

    x: [..., K]; w: [N, K]; gate: [groups, N]; residual: [..., N]. On a GPU without autograd the whole
    expression is one tcgen05 GEMM launch; with autograd the epilogue pieces become separate differentiable ops.
    """
    lead = x.shape[:-1]
    if not native.use_native(x):
        x2 = x.reshape(-1, x.shape[-1])
        r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
        ex = [(a.reshape(-1, a.shape[-1]), b) for a, b in extra]
        y = ref.linear(x2, w, bias, act, r2, gate, rows_per_group, ex)
        if out is not None:
            out.reshape(-1, out.shape[-1]).copy_(y)
            return out
        return y.reshape(*lead, w.shape[0])
    if (x.shape[-1] % 8 or w.shape[0] % 8) and not extra:
        # rows of 16-byte multiples are a TMA rule: zero-pad the reduction and / or the output width (patch embedders
        # and heads with odd channel counts; small matrices), then drop the padded output columns
        kp, npad = (-x.shape[-1]) % 8, (-w.shape[0]) % 8
        pad = torch.nn.functional.pad
        y = linear(pad(x, (0, kp)), pad(w, (0, kp, 0, npad)), pad(bias, (0, npad)) if bias is not None else None, act,
                   pad(residual, (0, npad)) if residual is not None else None,
                   pad(gate, (0, npad)) if gate is not None else None, rows_per_group)
        y = y[..., :w.shape[0]]
        if out is not None:
            out.copy_(y)
            return out
        return y.contiguous() if npad else y
    x2 = _flat2d(x)
    need_grad = torch.is_grad_enabled() and (x.requires_grad or w.requires_grad or
                                             (bias is not None and bias.requires_grad))
    if not need_grad:
        r2 = _flat2d(residual) if residual is not None else None
        o2 = out.reshape(-1, out.shape[-1]) if out is not None else None
        y = _gemm([x2] + [_flat2d(a) for a, _ in extra], [w] + [b for _, b in extra], bias=bias, residual=r2,
                  gate=gate, rows_per_group=rows_per_group, act=act_code(act), out=o2)
        return out if out is not None else y.reshape(*lead, w.shape[0])
    assert not extra, "extra K segments are an inference-path feature"
    y = _LinearFn.apply(x2, w, bias)
    y = activation(y, act)
    if gate is not None or residual is not None:
        r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else torch.zeros_like(y)
        y = gate_residual(r2, y, gate, rows_per_group)
    y = y.reshape(*lead, w.shape[0])
    if out is not None:
        out.copy_(y)
        return out
    return y


def _pad_rank(A, B):
    """Zero-pad the adapter rank to a multiple of 8 so the [M, r] intermediate keeps 16-byte rows (TMA rule)."""
    r = A.shape[0]
    pad = (-r) % 8
    if pad == 0:
        return A, B
    return torch.nn.functional.pad(A, (0, 0, 0, pad)), torch.nn.functional.pad(B, (0, pad))


def lora_linear(x, w, bias, A, B, scale: float, act=None, residual=None, gate=None, rows_per_group: int = 1,
                out=None):
    """``act(x W^T + b + scale * (x A^T) B^T)`` then the optional gated residual. A: [r, K] (down), B: [N, r] (up).

    GPU: the down projection is one skinny tcgen05 GEMM and the up projection rides in the base GEMM as an extra
    K segment, so the adapter never costs a separate pass over the output.
    """
    lead = x.shape[:-1]
    if not native.use_native(x):
        x2 = x.reshape(-1, x.shape[-1])
        y = x2 @ w.t()
        if bias is not None:
            y = y + bias
        y = y + scale * ((x2 @ A.t().to(x2.dtype)) @ B.t().to(x2.dtype))
        y = ref.activation(y, act)
        if gate is not None or residual is not None:
            r2 = residual.reshape(-1, y.shape[-1]) if residual is not None else torch.zeros_like(y)
            y = ref.gate_residual(r2, y, gate, rows_per_group)
        y = y.reshape(*lead, w.shape[0])
        if out is not None:
            out.copy_(y)
            return out
        return y
    x2 = _flat2d(x)
    A, B = _pad_rank(A, B)
    need_grad = torch.is_grad_enabled() and (x.requires_grad or A.requires_grad or B.requires_grad)
    if need_grad:
        y = _LoraLinearFn.apply(x2, w, bias, A, B, float(scale))
        y = activation(y, act)
        if gate is not None or residual is not None:
            r2 = residual.reshape(-1, y.shape[-1]) if residual is not None else torch.zeros_like(y)
            y = gate_residual(r2, y, gate, rows_per_group)
        y = y.reshape(*lead, w.shape[0])
        if out is not None:
            out.copy_(y)
            return out
        return y
    t = _gemm_skinny(x2, A.contiguous())          # few output tiles: the reduction is split over the idle SMs
    Bs = B if scale == 1.0 else (B.float() * scale).to(B.dtype)
    r2 = _flat2d(residual) if residual is not None else None
    o2 = out.reshape(-1, out.shape[-1]) if out is not None else None
    y = _gemm([x2, t], [w, Bs.contiguous()], bias=bias, residual=r2, gate=gate, rows_per_group=rows_per_group,
              act=act_code(act), out=o2)
    return out if out is not None else y.reshape(*lead, w.shape[0])


class _GluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, act, second):
        ctx.save_for_backward(h)
        ctx.act, ctx.second = act, second
        return _ops().glu_fwd(h, act, second)

    @staticmethod
    def backward(ctx, dy):
        (h,) = ctx.saved_tensors
        return _ops().glu_bwd(h, _flat2d(dy), ctx.act, ctx.second), None, None


def glu(h: torch.Tensor, act="silu", act_on_second: bool = False) -> torch.Tensor:
    """[..., 2F] -> [..., F]: ``act(a) * b`` (SwiGLU) or ``a * act(b)`` (GEGLU) over the two halves."""
    if not native.use_native(h):
        return ref.glu(h, act, act_on_second)
    lead = h.shape[:-1]
    h2 = _flat2d(h)
    if torch.is_grad_enabled() and h.requires_grad:
        y = _GluFn.apply(h2, act_code(act), bool(act_on_second))
    else:
        y = _ops().glu_fwd(h2, act_code(act), bool(act_on_second))
    return y.reshape(*lead, h.shape[-1] // 2)


def linear_glu(x, w, bias=None, act="silu", act_on_second: bool = False):
    """Gated projection in one launch: w is [2F, K] with the two halves stacked (first F rows, second F rows)."""
    lead = x.shape[:-1]
    F_ = w.shape[0] // 2
    if not native.use_native(x):
        return ref.linear_glu(x.reshape(-1, x.shape[-1]), w, bias, act, act_on_second).reshape(*lead, F_)
    need_grad = torch.is_grad_enabled() and (x.requires_grad or w.requires_grad)
    if need_grad:
        return glu(linear(x, w, bias), act, act_on_second)
    y = _gemm([_flat2d(x)], [w], bias=bias, act=act_code(act), pair_offset=F_, act_on_second=int(act_on_second))
    return y.reshape(*lead, F_)


def fp8_linear(x, wq, w_scale, bias=None, act=None, residual=None, gate=None, rows_per_group: int = 1):
    """fp8 (e4m3) weight and activation GEMM: x is quantised per token on the fly, wq [N, K] float8_e4m3fn with
    per-output-channel scales w_scale [N]; both scales are applied in the epilogue."""
    lead = x.shape[:-1]
    if not native.use_native(x):
        w = wq.float() * w_scale.float()[:, None]
        xq, xs = ref.fp8_quant_rows(x.reshape(-1, x.shape[-1]))
        xd = xq.float() * xs[:, None]
        r2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
        return ref.linear(xd, w, bias, act, r2, gate, rows_per_group, out_dtype=x.dtype).reshape(*lead, wq.shape[0])
    x2 = _flat2d(x)
    xq, xs = _ops().fp8_quant_rows(x2)
    r2 = _flat2d(residual) if residual is not None else None
    y = _gemm([xq], [wq], bias=bias, residual=r2, gate=gate, rows_per_group=rows_per_group, act=act_code(act),
              row_scale=xs, col_scale=w_scale)
    return y.reshape(*lead, wq.shape[0])


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, kv_len):
        o, lse = _ops().attention_fwd(q, k, v, scale, kv_len, True, None, [], [], [])
        ctx.save_for_backward(q, k, v, o, lse, kv_len if kv_len is not None else torch.empty(0))
        ctx.scale = scale
        ctx.has_len = kv_len is not None
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, kv_len = ctx.saved_tensors
        from . import attention_bwd
        dq, dk, dv = attention_bwd.backward(q, k, v, o, lse, do, ctx.scale, kv_len if ctx.has_len else None)
        return dq, dk, dv, None, None


class _QKVAttentionFn(torch.autograd.Function):
    """Packed projection buffer -> per-head QK-RMSNorm + RoPE -> attention, as ONE autograd node: the backward writes
    dq / dk / dv straight into the three column ranges of a single gradient buffer and runs the norm/rope backward in
    place on it, so no slice, cat or zero-fill kernels appear around the attention of a training step."""

    @staticmethod
    def forward(ctx, qkv, wq_a, wk_a, wq_b, wk_b, cos, sin, H, Dh, split, interleaved, scale, eps):
        B, S, W = qkv.shape
        D = H * Dh
        post = qkv.clone(memory_format=torch.contiguous_format)
        o_ = _ops()
        if split > 0:
            o_.qk_norm_rope(post[:, :split], wq_a, wk_a, cos, sin, H, Dh, 0, D, eps, interleaved, False, True, 0, 0)
        if split < S:
            o_.qk_norm_rope(post[:, split:], wq_b, wk_b, cos, sin, H, Dh, 0, D, eps, interleaved, False, True, 0, split)
        q, k, v = (post[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3))
        out, lse = o_.attention_fwd(q, k, v, scale, None, True, None, [], [], [])
        ctx.save_for_backward(qkv, post, out, lse, wq_a, wk_a, wq_b, wk_b, cos, sin)
        ctx.cfg = (H, Dh, split, interleaved, scale, eps)
        return out.reshape(B, S, D)

    @staticmethod
    def backward(ctx, do):
        qkv, post, out, lse, wq_a, wk_a, wq_b, wk_b, cos, sin = ctx.saved_tensors
        H, Dh, split, interleaved, scale, eps = ctx.cfg
        B, S, W = post.shape
        D = H * Dh
        from . import attention_bwd
        q, k, v = (post[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3))
        d = torch.empty_like(post)
        outs = [d[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3)]
        attention_bwd.backward(q, k, v, out, lse, do.reshape(B, S, H, Dh), scale, None, outs)
        pre = qkv if qkv.stride() == d.stride() else qkv.contiguous()
        o_ = _ops()
        if split > 0:
            o_.qk_norm_rope_bwd(d[:, :split], pre[:, :split], wq_a, wk_a, cos, sin, H, Dh, 0, D, eps, interleaved, True, 0, 0)
        if split < S:
            o_.qk_norm_rope_bwd(d[:, split:], pre[:, split:], wq_b, wk_b, cos, sin, H, Dh, 0, D, eps, interleaved, True, 0, split)
        return (d,) + (None,) * 12


def qkv_attention(qkv: torch.Tensor, H: int, Dh: int, wq, wk, cos, sin, split: int = 0, wq_first=None, wk_first=None,
                  interleaved: bool = True, scale: Optional[float] = None, eps: float = 1e-6) -> torch.Tensor:
    """Joint attention on a packed projection buffer qkv [B, S, 3*H*Dh] (q | k | v, each (head, Dh)): QK-RMSNorm + RoPE
    then attention; returns [B, S, H*Dh]. Rows before ``split`` use the norm weights ``wq_first`` / ``wk_first`` (the text
    stream of a joint block), the rest ``wq`` / ``wk``. Token t uses rotary row t."""
    B, S, W = qkv.shape
    D = H * Dh
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(Dh)
    wq_first = wq if wq_first is None else wq_first
    wk_first = wk if wk_first is None else wk_first
    if native.use_native(qkv) and torch.is_grad_enabled() and qkv.requires_grad and Dh in (64, 128):
        return _QKVAttentionFn.apply(qkv, wq_first, wk_first, wq, wk, cos, sin, H, Dh, split, interleaved, scale, eps)
    if split > 0:
        a = qk_norm_rope(qkv[:, :split], H, Dh, wq_first, wk_first, cos, sin, eps, interleaved, pos_offset=0)
        b = qk_norm_rope(qkv[:, split:], H, Dh, wq, wk, cos, sin, eps, interleaved, pos_offset=split)
        # without autograd the GPU kernel has normalised the two row ranges of ``qkv`` in place
        post = qkv if (native.use_native(qkv) and not (torch.is_grad_enabled() and qkv.requires_grad)) else torch.cat((a, b), dim=1)
    else:
        post = qk_norm_rope(qkv, H, Dh, wq, wk, cos, sin, eps, interleaved)
    q, k, v = (post[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3))
    return attention(q, k, v, scale).reshape(B, S, D)


class _PackedAttnMlpFn(torch.autograd.Function):
    """[B, S, 3D + F] projection buffer (q | k | v | mlp) -> [B, S, D + F] (attention | act(mlp)) as ONE autograd node.

    The attention output and the activated MLP half are written straight into the two column ranges of the result
    (the input of the block's second projection), and the backward writes dq | dk | dv | dmlp into the column ranges
    of one gradient buffer, so no slice copy, concatenation or zero fill surrounds the attention of a single-stream
    block in a training step. The only copy is the q | k | v range into the buffer that is normalised in place (the
    RMSNorm backward needs the projection as it was)."""

    @staticmethod
    def forward(ctx, h, wq, wk, cos, sin, H, Dh, act, interleaved, scale, eps, glu):
        B, S, W = h.shape
        D = H * Dh
        F_ = (W - 3 * D) // 2 if glu is not None else W - 3 * D
        o_ = _ops()
        h2 = h.view(B * S, W)
        post = torch.empty(B, S, 3 * D, dtype=h.dtype, device=h.device)
        o_.act_strided(h2[:, :3 * D], None, post.view(B * S, 3 * D), 0)
        o_.qk_norm_rope(post, wq, wk, cos, sin, H, Dh, 0, D, eps, interleaved, False, True, 0, 0)
        q, k, v = (post[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3))
        out = torch.empty(B, S, D + F_, dtype=h.dtype, device=h.device)
        _, lse = o_.attention_fwd(q, k, v, scale, None, True, out[..., :D].unflatten(-1, (H, Dh)), [], [], [])
        if glu is not None:
            o_.glu_strided(h2[:, 3 * D:], None, out.view(B * S, D + F_)[:, D:], act, glu)
        else:
            o_.act_strided(h2[:, 3 * D:], None, out.view(B * S, D + F_)[:, D:], act)
        ctx.save_for_backward(h, post, out, lse, wq, wk, cos, sin)
        ctx.cfg = (H, Dh, act, interleaved, scale, eps, glu)
        return out

    @staticmethod
    def backward(ctx, dout):
        h, post, out, lse, wq, wk, cos, sin = ctx.saved_tensors
        H, Dh, act, interleaved, scale, eps, glu = ctx.cfg
        B, S, W = h.shape
        D = H * Dh
        from . import attention_bwd
        o_ = _ops()
        if dout.stride(-1) != 1 or dout.stride(-2) % 8 or dout.data_ptr() % 16:
            dout = dout.contiguous()
        dh = torch.empty_like(h)
        q, k, v = (post[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3))
        outs = [dh[..., i * D:(i + 1) * D].unflatten(-1, (H, Dh)) for i in range(3)]
        attention_bwd.backward(q, k, v, out[..., :D].unflatten(-1, (H, Dh)), lse, dout[..., :D].unflatten(-1, (H, Dh)),
                               scale, None, outs)
        o_.qk_norm_rope_bwd(dh[..., :3 * D], h[..., :3 * D], wq, wk, cos, sin, H, Dh, 0, D, eps, interleaved, True, 0, 0)
        x_mlp, d_mlp, g_mlp = h.view(B * S, W)[:, 3 * D:], dout.reshape(B * S, -1)[:, D:], dh.view(B * S, W)[:, 3 * D:]
        if glu is not None:
            o_.glu_strided(x_mlp, d_mlp, g_mlp, act, glu)
        else:
            o_.act_strided(x_mlp, d_mlp, g_mlp, act)
        return (dh,) + (None,) * 11


def packed_attention_mlp(h: torch.Tensor, H: int, Dh: int, wq, wk, cos, sin, act="gelu_tanh", interleaved: bool = True,
                         scale: Optional[float] = None, eps: float = 1e-6, gated: Optional[bool] = None) -> torch.Tensor:
    """The middle of a single-stream block: h [B, S, 3*H*Dh + F] holds (q | k | v | mlp) of one fused projection; returns
    [B, S, H*Dh + F] = (attention(QK-RMSNorm + RoPE (q, k), v) | act(mlp)), the input of the block's output projection.
    With ``gated`` set (False: act(a) * b, True: a * act(b)) the MLP range is 2F wide (a | b) and contributes F columns."""
    B, S, W = h.shape
    D = H * Dh
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(Dh)
    if (native.use_native(h) and torch.is_grad_enabled() and h.requires_grad and h.dtype == torch.bfloat16
            and h.is_contiguous() and (W - 3 * D) % 16 == 0 and W > 3 * D):
        return _PackedAttnMlpFn.apply(h, wq, wk, cos, sin, H, Dh, act_code(act), interleaved, scale, eps,
                                      None if gated is None else bool(gated))
    qkv, mlp = split_cols(h, 3 * D)
    attn = qkv_attention(qkv, H, Dh, wq, wk, cos, sin, interleaved=interleaved, scale=scale, eps=eps)
    mlp = activation(mlp, act) if gated is None else glu(mlp, act, bool(gated))
    return torch.cat((attn, mlp), dim=-1)


class _SplitColsFn(torch.autograd.Function):
    """[.., a + b] -> contiguous ([.., a], [.., b]); the backward is one concatenation (no zero-filled buffers)."""

    @staticmethod
    def forward(ctx, x, a):
        ctx.a = a
        return x[..., :a].contiguous(), x[..., a:].contiguous()

    @staticmethod
    def backward(ctx, ga, gb):
        return torch.cat((ga, gb), dim=-1), None


def split_cols(x: torch.Tensor, a: int):
    if torch.is_grad_enabled() and x.requires_grad:
        return _SplitColsFn.apply(x, a)
    return x[..., :a], x[..., a:]


def attention(q, k, v, scale: Optional[float] = None, kv_len: Optional[torch.Tensor] = None,
              out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Scaled dot-product attention over [B, S, H, Dh] tensors (any strides with contiguous Dh).

    ``kv_len`` (int32 [B]) masks keys at positions >= kv_len[b]. Sq and Skv may differ (cross attention).
    """
    Dh = q.shape[-1]
    scale = float(scale) if scale is not None else 1.0 / math.sqrt(Dh)
    if not native.use_native(q) or Dh not in (64, 128):     # other head widths (120, 256, ...): the torch statement / library kernel
        o = ref.attention(q, k, v, scale, kv_len)
        if out is not None:
            out.copy_(o)
            return out
        return o
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
        o = _AttentionFn.apply(q, k, v, scale, kv_len)
        if out is not None:
            out.copy_(o)
            return out
        return o
    o, _ = _ops().attention_fwd(q, k, v, scale, kv_len, False, out, [], [], [])
    return o


# --------------------------------------------------------------------------------------------
# norms / rope
# --------------------------------------------------------------------------------------------
class _NormModFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x2, weight, bias, scale, shift, rows_per_group, eps, rms):
        ctx.save_for_backward(x2, weight if weight is not None else torch.empty(0),
                              scale if scale is not None else torch.empty(0))
        ctx.cfg = (rows_per_group, eps, rms, weight is not None, bias is not None, scale is not None,
                   shift is not None)
        return _ops().norm_modulate_fwd(x2, weight, bias, scale, shift, rows_per_group, eps, rms)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, scale = ctx.saved_tensors
        rpg, eps, rms, has_w, has_b, has_sc, has_sh = ctx.cfg
        dy = _flat2d(dy)
        dx = _ops().norm_modulate_bwd(x2, dy, weight if has_w else None, scale if has_sc else None, rpg, eps, rms)
        dw = db = dsc = dsh = None
        need = ctx.needs_input_grad
        if (has_w and need[1]) or (has_b and need[2]) or (has_sc and need[3]) or (has_sh and need[4]):
            # parameter / modulation gradients: column reductions of recomputed normalised rows
            xf = x2.float()
            if rms:
                xh = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
            else:
                mu = xf.mean(-1, keepdim=True)
                xh = (xf - mu) * torch.rsqrt((xf - mu).pow(2).mean(-1, keepdim=True) + eps)
            g = dy.float()
            rows = x2.shape[0]
            groups = scale.shape[0] if has_sc else 1
            one_plus = 1.0 + ref._group_expand(scale.float(), rows, rpg) if has_sc else 1.0
            aff = xh * weight.float() if has_w else xh
            if has_sh and need[4]:
                dsh = g.reshape(groups, -1, g.shape[-1]).sum(1).to(dy.dtype) if has_sc else None
            if has_sc and need[3]:
                dsc = (g * aff).reshape(groups, -1, g.shape[-1]).sum(1).to(dy.dtype)
            if has_w and need[1]:
                dw = (g * one_plus * xh).sum(0).to(weight.dtype)
            if has_b and need[2]:
                db = (g * one_plus).sum(0).to(dy.dtype)
        return dx, dw, db, dsc, dsh, None, None, None


def norm_modulate(x, weight=None, bias=None, scale=None, shift=None, rows_per_group: Optional[int] = None,
                  eps: float = 1e-6, rms: bool = False):
    """LayerNorm / RMSNorm over the last dim, optional affine, then adaLN ``* (1 + scale) + shift``.

    x: [B, S, D] or [rows, D]; scale / shift: [B, D] (one vector per sample) or [1, D].
    """
    D = x.shape[-1]
    if rows_per_group is None:
        rows_per_group = x.shape[-2] if x.dim() >= 3 else x.shape[0]
    sc = scale.reshape(-1, D) if scale is not None else None
    sh = shift.reshape(-1, D) if shift is not None else None
    if not native.use_native(x) or D % 8 or D > 16384:      # the kernel covers rows of 8 .. 16384 elements in steps of 8
        return ref.norm_modulate(x.reshape(-1, D), weight, bias, sc, sh, rows_per_group, eps, rms).reshape(x.shape)
    x2 = _flat2d(x)
    if sc is not None and sh is not None and sc.stride(0) != sh.stride(0):
        sc, sh = sc.contiguous(), sh.contiguous()
    if torch.is_grad_enabled() and (x.requires_grad or (sc is not None and sc.requires_grad)):
        y = _NormModFn.apply(x2, weight, bias, sc, sh, rows_per_group, eps, rms)
    else:
        y = _ops().norm_modulate_fwd(x2, weight, bias, sc, sh, rows_per_group, eps, rms)
    return y.reshape(x.shape)


def rope_table(pos: torch.Tensor, axes_dim: Sequence[int], theta: float = 10000.0):
    """cos/sin tables [T, sum(axes)/2] (fp32) from positions [T, n_axes]."""
    if not native.use_native(pos):
        return ref.rope_table(pos, axes_dim, theta)
    return _ops().rope_table(pos.float().contiguous(), list(axes_dim), float(theta))


class _QKNormRopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, buf, wq, wk, cos, sin, H, Dh, q_off, k_off, eps, interleaved, do_norm, rope_start, pos_offset):
        out = buf.clone()
        _ops().qk_norm_rope(out, wq, wk, cos, sin, H, Dh, q_off, k_off, eps, interleaved, False, do_norm, rope_start,
                            pos_offset)
        ctx.save_for_backward(buf, wq if wq is not None else torch.empty(0), wk if wk is not None else torch.empty(0),
                              cos if cos is not None else torch.empty(0), sin if sin is not None else torch.empty(0))
        ctx.cfg = (H, Dh, q_off, k_off, eps, interleaved, do_norm, rope_start, pos_offset, wq is not None,
                   cos is not None)
        return out

    @staticmethod
    def backward(ctx, dout):
        buf, wq, wk, cos, sin = ctx.saved_tensors
        H, Dh, q_off, k_off, eps, inter, do_norm, rope_start, pos_offset, has_w, has_rope = ctx.cfg
        d = dout.clone(memory_format=torch.contiguous_format)
        xb = buf if buf.stride() == d.stride() else buf.contiguous()
        _ops().qk_norm_rope_bwd(d, xb, wq if has_w else None, wk if has_w else None, cos if has_rope else None,
                                sin if has_rope else None, H, Dh, q_off, k_off, eps, inter, do_norm, rope_start,
                                pos_offset)
        return (d,) + (None,) * 13


def qk_norm_rope(qkv: torch.Tensor, H: int, Dh: int, wq=None, wk=None, cos=None, sin=None, eps: float = 1e-6,
                 interleaved: bool = True, do_norm: bool = True, rope_start: int = 0, q_off: int = 0,
                 k_off: Optional[int] = None, pos_offset: int = 0):
    """Per-head RMSNorm of q and k followed by rotary embedding, on a packed projection buffer.

    qkv: [B, S, W] (a view with contiguous last dim is fine) where q occupies columns [q_off, q_off + H*Dh) and
    k [k_off, k_off + H*Dh) (default: right after q), each laid out (head, Dh). cos / sin: [positions, Dh/2] fp32;
    token t of the view uses row ``t + pos_offset``; positions before ``rope_start`` are normalised but not
    rotated. Returns a tensor of the same shape (the input itself, updated in place, when autograd is off).
    """
    B, S, W = qkv.shape
    k_off = q_off + H * Dh if k_off is None else k_off
    if not native.use_native(qkv):
        q = qkv[..., q_off:q_off + H * Dh].reshape(B, S, H, Dh)
        k = qkv[..., k_off:k_off + H * Dh].reshape(B, S, H, Dh)
        c = cos[pos_offset:pos_offset + S] if cos is not None else None
        s_ = sin[pos_offset:pos_offset + S] if sin is not None else None
        q2, k2 = ref.qk_norm_rope(q, k, wq, wk, c, s_, eps, interleaved, do_norm, max(0, rope_start - pos_offset))
        out = qkv.clone()
        out[..., q_off:q_off + H * Dh] = q2.reshape(B, S, H * Dh)
        out[..., k_off:k_off + H * Dh] = k2.reshape(B, S, H * Dh)
        return out
    assert qkv.stride(2) == 1
    if torch.is_grad_enabled() and qkv.requires_grad:
        return _QKNormRopeFn.apply(qkv.contiguous(), wq, wk, cos, sin, H, Dh, q_off, k_off, eps, interleaved, do_norm,
                                   rope_start, pos_offset)
    _ops().qk_norm_rope(qkv, wq, wk, cos, sin, H, Dh, q_off, k_off, eps, interleaved, False, do_norm, rope_start,
                        pos_offset)
    return qkv


# --------------------------------------------------------------------------------------------
# pointwise
# --------------------------------------------------------------------------------------------
class _ActFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, act):
        ctx.save_for_backward(x)
        ctx.act = act
        return _ops().act_fwd(x, None, act)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return _ops().act_bwd(x, dy.contiguous(), None, ctx.act), None


def activation(x: torch.Tensor, act) -> torch.Tensor:
    a = act_code(act)
    if a == ref.ACT_NONE:
        return x
    if not native.use_native(x) or x.dtype != torch.bfloat16 or x.numel() % 8:
        return ref.activation(x, a)
    xc = x.contiguous()
    if torch.is_grad_enabled() and x.requires_grad:
        return _ActFn.apply(xc, a)
    return _ops().act_fwd(xc, None, a)


class _GateResFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, y, gate, rows_per_group, tanh_gate):
        ctx.save_for_backward(y, gate if gate is not None else torch.empty(0))
        ctx.cfg = (rows_per_group, tanh_gate, gate is not None)
        return _ops().gate_residual(x, y, gate, rows_per_group, tanh_gate)

    @staticmethod
    def backward(ctx, dout):
        y, gate = ctx.saved_tensors
        rpg, tanh_gate, has_gate = ctx.cfg
        dx = dout
        if not has_gate:
            return dx, dout, None, None, None
        D = y.shape[-1]
        d2 = dout.reshape(-1, D)
        dy = _ops().gate_mul(dout.contiguous(), gate, rpg, tanh_gate)
        dgate = None
        if ctx.needs_input_grad[2]:
            g = torch.tanh(gate.float()) if tanh_gate else gate.float()
            prod = (d2.float() * y.reshape(-1, D).float())
            groups = gate.shape[0]
            if groups == 1:
                dg = prod.sum(0, keepdim=True)
            else:
                dg = prod.reshape(groups, -1, D).sum(1)
            if tanh_gate:
                dg = dg * (1 - g * g)
            dgate = dg.to(gate.dtype)
        return dx, dy, dgate, None, None


def gate_residual(x, y, gate=None, rows_per_group: Optional[int] = None, tanh_gate: bool = False):
    """``x + gate[row // rows_per_group] * y`` (gate [groups, D] or None for a plain add)."""
    D = x.shape[-1]
    if rows_per_group is None:
        rows_per_group = x.shape[-2] if x.dim() >= 3 else x.shape[0]
    g = gate.reshape(-1, D) if gate is not None else None
    if not native.use_native(x) or x.dtype != torch.bfloat16:
        return ref.gate_residual(x, y, g, rows_per_group, tanh_gate)
    xc, yc = x.contiguous(), y.contiguous()
    if torch.is_grad_enabled() and (x.requires_grad or y.requires_grad or (g is not None and g.requires_grad)):
        return _GateResFn.apply(xc, yc, g, rows_per_group, tanh_gate)
    return _ops().gate_residual(xc, yc, g, rows_per_group, tanh_gate)


def cfg_euler(x: torch.Tensor, vc, vu=None, dt: float = 0.0, s: float = 1.0, mode: int = 0,
              x_bf16: Optional[torch.Tensor] = None) -> torch.Tensor:
    """In-place sampler step on the fp32 latent ``x``: ``x += dt * CFG(vc, vu)``; also refreshes the bf16 copy."""
    if not native.use_native(x):
        x.copy_(ref.cfg_euler(x, vc, vu, dt, s, mode))
        if x_bf16 is not None:
            x_bf16.copy_(x)
        return x
    _ops().cfg_euler(x, vc.contiguous(), vu.contiguous() if vu is not None else None, x_bf16, dt, s, mode)
    return x


def flow_match(x0, eps, sigma):
    """(x_t, target) for rectified flow: ``x_t = (1-sigma) x0 + sigma eps`` (bf16 on GPU), ``target = eps - x0``."""
    if not native.use_native(x0):
        return ref.flow_match(x0, eps, sigma)
    return _ops().flow_match(x0.float().contiguous(), eps.float().contiguous(), sigma.float().contiguous())


class _MseFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pred, target):
        loss, grad = _ops().mse_loss(pred, target, True, 1.0)
        ctx.save_for_backward(grad)
        return loss

    @staticmethod
    def backward(ctx, dl):
        (grad,) = ctx.saved_tensors
        return grad * dl.to(grad.dtype), None


def mse_loss(pred: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
    """mean((pred - target)^2) with fp32 accumulation; pred bf16, target fp32 on the GPU path."""
    if not native.use_native(pred) or pred.dtype != torch.bfloat16:
        return (pred.float() - target.float()).pow(2).mean()
    p, t = pred.contiguous(), target.float().contiguous()
    if torch.is_grad_enabled() and pred.requires_grad:
        return _MseFn.apply(p, t)
    return _ops().mse_loss(p, t, False, 1.0)[0]


def randn(shape, seed: int, offset: int = 0, dtype=torch.float32, device="cpu") -> torch.Tensor:
    """Seeded standard normal noise. On a GPU: counter-based Philox + Box-Muller kernel (same seed -> same tensor
    for any launch geometry); on CPU: torch.Generator."""
    device = torch.device(device)
    if device.type != "cuda":
        g = torch.Generator().manual_seed(int(seed) + int(offset))
        return torch.randn(*shape, generator=g, dtype=torch.float32).to(dtype)
    like = torch.empty(0, device=device)
    native.load(True)
    out = _ops().randn(list(shape), int(seed), int(offset), dtype == torch.bfloat16, like)
    return out if dtype in (torch.float32, torch.bfloat16) else out.to(dtype)


def fp8_quant_rows(x):
    if not native.use_native(x):
        return ref.fp8_quant_rows(x)
    return _ops().fp8_quant_rows(_flat2d(x))


def mx_dequant(q, scales, fp4: bool = True, shape=None):
    """MXFP4 (E2M1 pairs per byte) or MXFP8 (E4M3 bytes) blocks of 32 with E8M0 scale bytes -> bf16. ``shape`` reshapes
    the flat result (gpt-oss expert weights: blocks [.., G, 16] + scales [.., G] -> [.., G * 32])."""
    if not native.use_native(q):
        y = ref.mx_dequant(q, scales, fp4)
    else:
        y = _ops().mx_dequant(q.contiguous().reshape(-1), scales.contiguous().reshape(-1), bool(fp4))
    if shape is None and fp4 and q.dim() >= 2 and q.shape[-1] == 16:
        shape = tuple(q.shape[:-2]) + (q.shape[-2] * 32,)
    return y.reshape(shape) if shape is not None else y


def mx_quant(x, fp4: bool = True):
    """bf16 -> (packed bytes, E8M0 scale bytes) over consecutive blocks of 32 elements."""
    if not native.use_native(x):
        return ref.mx_quant(x, fp4)
    return _ops().mx_quant(x.contiguous().to(torch.bfloat16), bool(fp4))


def mxfp8_quant_rows(x, pad_rows: int = 128):
    """bf16 [rows, K] -> (E4M3 bytes, scale chunks in the tensor core's layout). ``pad_rows`` 128 for the activation (A)
    operand of ``gemm_mxfp8``, 256 for the weight (B) operand."""
    if not native.use_native(x):
        return ref.mxfp8_quant_rows(x, pad_rows)
    return _ops().mxfp8_quant_rows(x.to(torch.bfloat16), int(pad_rows))


def gemm_mxfp8(a_q, sfa, b_q, sfb, bias=None):
    """[M, K] x [N, K]^T -> bf16 [M, N] with both operands in MXFP8 (hardware block scaling, fp32 accumulation)."""
    if not native.use_native(a_q):
        return ref.gemm_mxfp8(a_q, sfa, b_q, sfb, bias)
    return _ops().gemm_mxfp8(a_q.contiguous(), sfa.contiguous(), b_q.contiguous(), sfb.contiguous(), bias)


class MXFP8Weight:
    """A linear weight [N, K] held in MXFP8 (quantised once); ``linear(x)`` quantises the activation rows on the fly."""

    def __init__(self, weight: torch.Tensor, bias: Optional[torch.Tensor] = None):
        self.q, self.sf = mxfp8_quant_rows(weight.detach().to(torch.bfloat16).contiguous(), 256)
        self.bias = bias.detach().to(torch.bfloat16).contiguous() if bias is not None else None
        self.out_features, self.in_features = weight.shape

    def linear(self, x: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, self.in_features).to(torch.bfloat16).contiguous()
        aq, asf = mxfp8_quant_rows(x2, 128)
        return gemm_mxfp8(aq, asf, self.q, self.sf, self.bias).reshape(*x.shape[:-1], self.out_features)


def fp8_dequant(q, row_scale=None, tensor_scale: float = 1.0):
    if not native.use_native(q):
        return ref.fp8_dequant(q, row_scale, tensor_scale)
    return _ops().fp8_dequant(q.contiguous(), row_scale, float(tensor_scale))
