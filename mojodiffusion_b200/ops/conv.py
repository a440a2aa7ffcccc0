"""Image ops in NHWC: convolution (implicit GEMM on tcgen05 through 4-D TMA boxes), GroupNorm+SiLU, nearest 2x
upsample, 2x2 average pool, pixel (un)shuffle and latent patchify helpers.

The native convolution covers stride 1 with "same" padding and Cin a multiple of 64 (the bulk of every VAE / UNet);
other shapes (the 3- or 4-channel stem, strided down-sampling convs) use ``torch.nn.functional.conv2d``.
Reference: serenitymojo/ops/conv.mojo:46-209 (im2col + GEMM), serenitymojo/models/vae/decoder2d.mojo:150-362,
serenitymojo/ops/pixelshuffle.mojo:144-770, serenitymojo/ops/layout.mojo:44-383.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

from . import native
from .reference import act_code, activation


def conv2d_nhwc_reference(x, w_ohwi, bias=None, stride: int = 1, padding=1, act=None, residual=None):
    """x [N,H,W,Cin], w [Cout,KH,KW,Cin] -> [N,Ho,Wo,Cout]; fp32 math."""
    pad = (padding, padding) if isinstance(padding, int) else tuple(padding)
    y = F.conv2d(x.permute(0, 3, 1, 2).float(), w_ohwi.permute(0, 3, 1, 2).float(),
                 bias.float() if bias is not None else None, stride=stride, padding=pad)
    y = activation(y, act).permute(0, 2, 3, 1)
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def _native_conv_ok(x, w_ohwi, pad) -> bool:
    KH, KW = w_ohwi.shape[1], w_ohwi.shape[2]
    return native.use_native(x) and x.dtype == torch.bfloat16 and 2 * pad[0] == KH - 1 and 2 * pad[1] == KW - 1


def _pad_channels(t, mult: int, dim: int = -1):
    c = t.shape[dim]
    extra = (-c) % mult
    if extra == 0:
        return t
    shape = list(t.shape)
    shape[dim] = extra
    return torch.cat((t, t.new_zeros(shape)), dim=dim)


def _conv_same_native(x, w_ohwi, bias, pad, act=None, residual=None):
    """Stride-1 "same" convolution on the implicit-GEMM kernel for ANY channel counts: input channels are zero-padded to a
    multiple of 64 (the 3- / 4-channel stems), output channels to a multiple of 8 (the 3- / 4-channel heads)."""
    Cout, Cin = w_ohwi.shape[0], w_ohwi.shape[3]
    xp, wp = _pad_channels(x, 64), _pad_channels(w_ohwi, 64)
    if Cout % 8:
        wp = _pad_channels(wp, 8, 0)
        bias = _pad_channels(bias, 8, 0) if bias is not None else None
        residual = _pad_channels(residual, 8) if residual is not None else None
    y = native.ops().conv2d_nhwc(xp.contiguous(), wp.contiguous(), bias, pad[0], pad[1], act_code(act),
                                 residual.contiguous() if residual is not None else None)
    return y[..., :Cout] if Cout % 8 else y


def _rotated(w_ohwi):
    """Weights of the input-gradient convolution: spatially flipped, input / output channels exchanged ([Cin, KH, KW, Cout])."""
    return w_ohwi.flip(1, 2).permute(3, 1, 2, 0).contiguous()


def conv2d_weight_grad(x, dy, KH: int, KW: int, pad):
    """dW [Cout, KH, KW, Cin] of a stride-1 "same" convolution as KH * KW GEMMs over the pixels. Both tensors are
    zero-padded by the kernel radius and flattened to [pixels', C]; a tap is then a constant offset between the two
    flat index spaces (the zero border makes every wrap-around term vanish), so each tap is one MN-major GEMM on two
    contiguous slices, fp32 accumulation (serenitymojo/ops/conv2d_backward.mojo:73-182)."""
    from .functional import _gemm
    N, H, W, Cin = x.shape
    Cout = dy.shape[-1]
    ph, pw = pad
    Wp = W + 2 * pw
    xp = torch.nn.functional.pad(x, (0, 0, pw, pw, ph, ph)).reshape(-1, Cin)
    dyp = torch.nn.functional.pad(dy, (0, 0, pw, pw, ph, ph)).reshape(-1, Cout)
    P = xp.shape[0]
    dw = torch.empty(Cout, KH, KW, Cin, dtype=torch.float32, device=x.device)
    for kh in range(KH):
        for kw in range(KW):
            off = (kh - ph) * Wp + (kw - pw)                       # x index = dy index + off
            a = dyp[max(0, -off):P - max(0, off)]
            b = xp[max(0, off):P - max(0, -off)]
            if native.use_native(x) and x.dtype == torch.bfloat16 and Cin % 8 == 0 and Cout % 8 == 0:
                dw[:, kh, kw] = _gemm([a], [b], a_mn=True, b_mn=True, out_fp32=True)
            else:
                dw[:, kh, kw] = a.float().t() @ b.float()
    return dw


class _Conv2dFn(torch.autograd.Function):
    """Convolution with native forward and native input gradient (the same kernel on the rotated weights; a stride-2
    layer is the stride-1 result sampled at every second position, its gradient scattered back before the rotation).
    Weight and bias gradients are computed only when asked for."""

    @staticmethod
    def forward(ctx, x, w, bias, stride, pad, offset):
        y = _conv_same_native(x, w, bias, pad)
        if stride > 1:
            y = y[:, offset::stride, offset::stride].contiguous()
        ctx.save_for_backward(x, w)
        ctx.meta = (stride, pad, offset, bias is not None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        stride, pad, offset, has_bias = ctx.meta
        dy = dy.contiguous()
        if stride > 1:
            full = dy.new_zeros(x.shape[0], x.shape[1], x.shape[2], dy.shape[-1])
            full[:, offset::stride, offset::stride] = dy
            dy = full
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = _conv_same_native(dy, _rotated(w), None, pad).to(x.dtype)
        if ctx.needs_input_grad[1]:
            dw = conv2d_weight_grad(x, dy, w.shape[1], w.shape[2], pad).to(w.dtype)
        if has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(dim=(0, 1, 2)).to(w.dtype)
        return dx, dw, db, None, None, None


def conv2d_nhwc(x, w_ohwi, bias=None, stride: int = 1, padding=1, act=None, residual=None, offset: int = 0):
    """``stride`` 2 samples the stride-1 "same" result at ``offset::2`` (offset 0: symmetric padding as in the UNet
    down-samplers; offset 1: the right / bottom padded stride-2 convolution of the LDM encoders)."""
    pad = (padding, padding) if isinstance(padding, int) else tuple(padding)
    KH, KW, Cin = w_ohwi.shape[1], w_ohwi.shape[2], w_ohwi.shape[3]
    ok = _native_conv_ok(x, w_ohwi, pad)
    if ok and torch.is_grad_enabled() and (x.requires_grad or w_ohwi.requires_grad or (bias is not None and bias.requires_grad)):
        y = _Conv2dFn.apply(x, w_ohwi, bias, stride, pad, offset)
        if act is not None:
            from . import functional as Fn
            y = Fn.activation(y, act)
        return y + residual if residual is not None else y
    if ok and stride == 1:
        if Cin % 64 == 0 and w_ohwi.shape[0] % 8 == 0:
            res = residual.contiguous() if residual is not None else None
            return native.ops().conv2d_nhwc(x.contiguous(), w_ohwi.contiguous(), bias, pad[0], pad[1], act_code(act), res)
        return _conv_same_native(x, w_ohwi, bias, pad, act, residual)
    if ok and stride == 2:
        y = _conv_same_native(x, w_ohwi, bias, pad, act)[:, offset::2, offset::2].contiguous()
        return y + residual if residual is not None else y
    if offset:
        raise NotImplementedError("offset sampling is defined for the native path")
    return conv2d_nhwc_reference(x, w_ohwi, bias, stride, pad, act, residual)


class _GroupNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, groups, eps, act):
        ctx.save_for_backward(x, weight, bias)
        ctx.meta = (groups, eps, act)
        return native.ops().group_norm_nhwc(x.contiguous(), weight, bias, groups, eps, act)

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias = ctx.saved_tensors
        groups, eps, act = ctx.meta
        need_w = weight is not None and (ctx.needs_input_grad[1] or ctx.needs_input_grad[2])
        dx, dw, db = native.ops().group_norm_nhwc_bwd(x.contiguous(), dy.contiguous(), weight, bias, groups, eps, act, bool(need_w))
        return (dx if ctx.needs_input_grad[0] else None, dw.to(weight.dtype) if need_w and ctx.needs_input_grad[1] else None,
                db.to(weight.dtype) if need_w and bias is not None and ctx.needs_input_grad[2] else None, None, None, None)


def group_norm_nhwc(x, weight=None, bias=None, groups: int = 32, eps: float = 1e-6, act=None):
    """GroupNorm over (H, W, C/G) per sample and group on an NHWC tensor, optional fused SiLU."""
    a = act_code(act)
    if native.use_native(x) and x.dtype == torch.bfloat16 and a in (0, 2) and x.shape[-1] % 8 == 0:
        if torch.is_grad_enabled() and (x.requires_grad or (weight is not None and weight.requires_grad)):
            return _GroupNormFn.apply(x, weight, bias, groups, eps, a)
        if not torch.is_grad_enabled():
            return native.ops().group_norm_nhwc(x.contiguous(), weight, bias, groups, eps, a)
    N, H, W, C = x.shape
    xf = x.float().reshape(N, H * W, groups, C // groups)
    mu = xf.mean(dim=(1, 3), keepdim=True)
    var = (xf - mu).pow(2).mean(dim=(1, 3), keepdim=True)
    y = ((xf - mu) * torch.rsqrt(var + eps)).reshape(N, H, W, C)
    if weight is not None:
        y = y * weight.float() + (bias.float() if bias is not None else 0.0)
    return activation(y, act).to(x.dtype)


def upsample_nearest2x_nhwc(x):
    if native.use_native(x) and not torch.is_grad_enabled() and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
        return native.ops().upsample2x_nhwc(x.contiguous())
    return x.repeat_interleave(2, dim=1).repeat_interleave(2, dim=2)


def avgpool2x_nhwc(x):
    if native.use_native(x) and not torch.is_grad_enabled() and x.dtype == torch.bfloat16:
        return native.ops().avgpool2x_nhwc(x.contiguous())
    N, H, W, C = x.shape
    return x.float().reshape(N, H // 2, 2, W // 2, 2, C).mean(dim=(2, 4)).to(x.dtype)


# ---- layout helpers (index math; views where possible) ---------------------------------------------------
def pixel_shuffle_nhwc(x, r: int):
    """[N,H,W,C*r*r] -> [N,H*r,W*r,C] (channel order c, ry, rx as torch.nn.PixelShuffle)."""
    N, H, W, Crr = x.shape
    C = Crr // (r * r)
    return x.reshape(N, H, W, C, r, r).permute(0, 1, 4, 2, 5, 3).reshape(N, H * r, W * r, C)


def pixel_unshuffle_nhwc(x, r: int):
    N, Hr, Wr, C = x.shape
    H, W = Hr // r, Wr // r
    return x.reshape(N, H, r, W, r, C).permute(0, 1, 3, 5, 2, 4).reshape(N, H, W, C * r * r)


def depth_to_space_3d(x, ft: int, fh: int, fw: int):
    """[N,T,H,W,C*ft*fh*fw] -> [N,T*ft,H*fh,W*fw,C] (video VAE up-sampling; serenitymojo/ops/pixelshuffle.mojo)."""
    N, T, H, W, Cf = x.shape
    C = Cf // (ft * fh * fw)
    x = x.reshape(N, T, H, W, C, ft, fh, fw).permute(0, 1, 5, 2, 6, 3, 7, 4)
    return x.reshape(N, T * ft, H * fh, W * fw, C)


def space_to_depth_3d(x, ft: int, fh: int, fw: int):
    N, Tt, Hh, Ww, C = x.shape
    T, H, W = Tt // ft, Hh // fh, Ww // fw
    x = x.reshape(N, T, ft, H, fh, W, fw, C).permute(0, 1, 3, 5, 7, 2, 4, 6)
    return x.reshape(N, T, H, W, C * ft * fh * fw)


def patchify_3d(z, pt: int, ph: int, pw: int):
    """[B,C,T,H,W] -> tokens [B, (T/pt)(H/ph)(W/pw), C*pt*ph*pw] (serenitymojo/ops/patchify3d.mojo:159)."""
    B, C, T, H, W = z.shape
    z = z.reshape(B, C, T // pt, pt, H // ph, ph, W // pw, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
    return z.reshape(B, (T // pt) * (H // ph) * (W // pw), C * pt * ph * pw)


def unpatchify_3d(x, grid, C: int, pt: int, ph: int, pw: int):
    B = x.shape[0]
    T, H, W = grid
    x = x.reshape(B, T, H, W, C, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
    return x.reshape(B, C, T * pt, H * ph, W * pw)


def conv3d_ndhwc(x, w_otohwi, bias=None, act=None, temporal_pad: str = "replicate"):
    """3-D convolution on [N, T, H, W, Cin] with weights [Cout, KT, KH, KW, Cin], stride 1, "same" output size.

    The spatial taps run in the 2-D implicit-GEMM kernel with all N*T frames as its batch; the KT temporal taps are KT such
    launches over time-shifted views that accumulate through the kernel's residual input, so no im2col volume is ever
    materialised. ``temporal_pad``: "replicate" repeats the first and last frame (the non-causal video-VAE rule,
    serenitymojo/models/vae/ltx2_vae_decoder.mojo:52-59), "zeros" pads with zero frames
    (serenitymojo/models/vae/conv3d.mojo)."""
    N, T, H, W, Cin = x.shape
    Cout, KT, KH, KW, _ = w_otohwi.shape
    pt = (KT - 1) // 2
    if pt > 0:
        if temporal_pad == "replicate":
            xp = torch.cat([x[:, :1]] * pt + [x] + [x[:, -1:]] * pt, dim=1)
        elif temporal_pad == "causal":
            xp = torch.cat([x[:, :1]] * (KT - 1) + [x], dim=1)              # only the past: first frame repeated
        else:
            z = x.new_zeros(N, pt, H, W, Cin)
            xp = torch.cat((z, x, z), dim=1)
    else:
        xp = x
    acc = None
    for dt in range(KT):
        frames = xp[:, dt:dt + T].reshape(N * T, H, W, Cin)
        last = dt == KT - 1
        acc = conv2d_nhwc(frames, w_otohwi[:, dt], bias if dt == 0 else None, 1, (KH // 2, KW // 2), None, acc)
        if last and act is not None:
            acc = activation(acc.float(), act).to(acc.dtype)
    return acc.reshape(N, T, H, W, Cout)


def conv3d_ndhwc_reference(x, w_otohwi, bias=None, act=None, temporal_pad: str = "replicate"):
    """The same operation through ``torch.nn.functional.conv3d`` in fp32."""
    KT, KH, KW = w_otohwi.shape[1:4]
    xc = x.permute(0, 4, 1, 2, 3).float()
    pt = (KT - 1) // 2
    if pt > 0 and temporal_pad == "causal":
        xc = torch.cat([xc[:, :, :1]] * (KT - 1) + [xc], dim=2)
    elif pt > 0:
        xc = F.pad(xc, (0, 0, 0, 0, pt, pt), mode="replicate" if temporal_pad == "replicate" else "constant")
    y = F.conv3d(xc, w_otohwi.permute(0, 4, 1, 2, 3).float(), bias.float() if bias is not None else None,
                 padding=(0, KH // 2, KW // 2))
    return activation(y, act).permute(0, 2, 3, 4, 1).to(x.dtype)
