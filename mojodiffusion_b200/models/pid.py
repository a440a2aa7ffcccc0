"""PiD / PixelDiT 4x super-resolution decoder: a pixel-space flow model that turns a low-quality 16-channel latent plus a caption
into RGB pixels.

* patch stream: 16 x 16 RGB patches (unfold order: channel, row, column) -> ``s_embedder``; 14 dual-stream MMDiT blocks of width
  1536 (24 heads of 64) over image patches and caption tokens: per-stream ``Linear(silu(t_emb)) -> 6`` modulation chunks (shift,
  scale, gate for attention and for the SwiGLU feed-forward), RMS pre-norms, SEPARATE qkv projections per stream, per-head
  QK-RMSNorm, interleaved-pair rotation (image: NTK-scaled 2-D table; text: 1-D table), joint attention over [text, image],
  per-stream output projections with bias;
* low-quality branch: the latent is nearest-upsampled to the patch grid, run through two 3 x 3 convolutions and four pre-activation
  residual blocks (GroupNorm(4) -> SiLU -> conv, twice) into 512-wide tokens; before every second MMDiT block a per-point head
  maps them to 1536 and a gate injects them: ``s += sigmoid(content_proj([s, lq]) - exp(log_alpha) * sigma) * lq``;
* timestep: cos-first sinusoid with max period 10 (not 10 000) -> Linear -> SiLU -> Linear;
* caption: Linear + RMSNorm + learned position embedding (first 300 rows);
* pixel stream: every pixel -> Linear(3 -> 16) + a 2-D sin / cos position, grouped per patch as [B L, 256, 16]; two PiT blocks
  conditioned on ``silu(t_emb + s)`` of the patch: per-PIXEL modulation from ``Linear(1536 -> 6 * 16 * 256)``, the patch's pixels
  compressed to ONE 1152-wide token (``compress_to_attn``), rotary attention (16 heads of 72, NTK 2-D table) across patches,
  expanded back (``expand_from_attn``), then an exact-GELU MLP per pixel; final RMSNorm(16) + Linear(16 -> 3), folded to the image.

NTK table (dim d, grid H x W, reference grid 64): per axis ``theta_axis = 1e4 * (size / 64) ** (d/2 / (d/2 - 2))``; positions
``linspace(0, 16, size)``; frequency pair k uses ``theta_axis ** (-4 k / d)``; even table columns carry the column axis, odd ones
the row axis.

Behaviour: serenitymojo/models/pid/pid_net.mojo:1-36 (forward order), :166-205 (residual block), :445-474 (latent branch), :610-680
(wiring); serenitymojo/models/pid/pid_ops.mojo:5-42 (patch order, NTK table, timestep sinusoid, gate);
serenitymojo/models/pid/pixeldit_block.mojo:8-33 (MMDiT block); serenitymojo/models/pid/pit_block.mojo:6-28 (PiT block);
serenitymojo/models/pid/parity/gen_pid_net_reference.py:143-160 (position tables). Convolution weights are stored
[out, kh, kw, in] here (``remap_pid_keys`` permutes the checkpoint's).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from ..ops import conv as C
from .layers import Linear, RMSNorm, init_module_weights


@dataclass
class PidConfig:
    hidden: int = 1536
    groups: int = 24
    patch_depth: int = 14
    pixel_depth: int = 2
    pixel_dim: int = 16
    pixel_attn: int = 1152
    pixel_groups: int = 16
    patch_size: int = 16
    lq_channels: int = 16
    lq_hidden: int = 512
    lq_interval: int = 2
    lq_groups: int = 4
    txt_dim: int = 2304
    txt_max: int = 300
    ffn_inner: int = 4096
    freq_dim: int = 256
    rope_ref: int = 64
    name: str = "pid-sr4x"

    @property
    def head_dim(self):
        return self.hidden // self.groups


def tiny_pid_config() -> PidConfig:
    return PidConfig(hidden=64, groups=4, patch_depth=4, pixel_depth=1, pixel_dim=4, pixel_attn=48, pixel_groups=4, patch_size=4,
                     lq_channels=4, lq_hidden=16, txt_dim=24, txt_max=12, ffn_inner=96, freq_dim=16, rope_ref=4, name="tiny-pid")


def pid_timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10.0) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat((args.cos(), args.sin()), -1)


def ntk_rope_2d(dim: int, H: int, W: int, ref_h: int, ref_w: int, theta: float = 1.0e4, scale: float = 16.0, device=None):
    """cos / sin [H W, dim / 2]; column 2 k: column-axis angle, column 2 k + 1: row-axis angle, pair frequency theta_axis ** (-4 k / dim)."""
    axis = dim // 2
    p = axis / (axis - 2) if axis > 2 else 0.0
    th_h, th_w = theta * (H / ref_h) ** p, theta * (W / ref_w) ** p
    k = torch.arange(dim // 4, dtype=torch.float64)
    fh, fw = th_h ** (-4.0 * k / dim), th_w ** (-4.0 * k / dim)
    ys = torch.linspace(0, scale, H, dtype=torch.float64) if H > 1 else torch.zeros(1, dtype=torch.float64)
    xs = torch.linspace(0, scale, W, dtype=torch.float64) if W > 1 else torch.zeros(1, dtype=torch.float64)
    ax = (xs[None, :, None] * fw[None, None]).expand(H, W, -1)
    ay = (ys[:, None, None] * fh[None, None]).expand(H, W, -1)
    ang = torch.stack((ax, ay), -1).reshape(H * W, dim // 2)
    return ang.cos().float().to(device), ang.sin().float().to(device)


def text_rope_1d(n: int, head_dim: int, theta: float = 1.0e4, device=None):
    ang = torch.arange(n, dtype=torch.float32)[:, None] / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))[None]
    return ang.cos().to(device), ang.sin().to(device)


def sincos_pos_2d(dim: int, H: int, W: int, device=None) -> torch.Tensor:
    """[H W, dim]: first half from the column index, second half from the row index, each [sin | cos] over dim / 4 frequencies."""
    omega = 1.0 / 10000.0 ** (torch.arange(dim // 4, dtype=torch.float64) / (dim // 4))
    col = torch.arange(W, dtype=torch.float64)[None, :].expand(H, W).reshape(-1)
    row = torch.arange(H, dtype=torch.float64)[:, None].expand(H, W).reshape(-1)
    one = lambda p: torch.cat(((p[:, None] * omega[None]).sin(), (p[:, None] * omega[None]).cos()), 1)
    return torch.cat((one(col), one(row)), 1).float().to(device)


def _rope_pairs(x, cos, sin):
    c, s = cos[None, :, None].to(x.dtype), sin[None, :, None].to(x.dtype)
    a, b = x[..., 0::2], x[..., 1::2]
    return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)


def _attend(q, k, v):
    if q.shape[-1] in (64, 128) or not q.is_cuda:
        return ops.attention(q, k, v)
    return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)


class _Proj(nn.Module):
    def __init__(self, i, o, dtype, device, norm=False):
        super().__init__()
        self.proj = Linear(i, o, True, dtype, device)
        if norm:
            self.norm = RMSNorm(o, 1e-6, dtype, device)


class _SwiGLU(nn.Module):
    def __init__(self, d, inner, dtype, device):
        super().__init__()
        self.w1, self.w2, self.w3 = Linear(d, inner, False, dtype, device), Linear(inner, d, False, dtype, device), Linear(d, inner, False, dtype, device)

    def forward(self, x):
        return self.w2(self.w1(x, act="silu") * self.w3(x))


class _JointAttn(nn.Module):
    def __init__(self, c: PidConfig, dtype, device):
        super().__init__()
        D, hd = c.hidden, c.head_dim
        for s in "xy":
            setattr(self, "qkv_" + s, Linear(D, 3 * D, False, dtype, device))
            setattr(self, "q_norm_" + s, RMSNorm(hd, 1e-6, dtype, device))
            setattr(self, "k_norm_" + s, RMSNorm(hd, 1e-6, dtype, device))
            setattr(self, "proj_" + s, Linear(D, D, True, dtype, device))


class PidMMDiTBlock(nn.Module):
    def __init__(self, c: PidConfig, dtype, device):
        super().__init__()
        self.c = c
        D = c.hidden
        self.adaLN_modulation_img = nn.ModuleList([Linear(D, 6 * D, True, dtype, device)])
        self.adaLN_modulation_txt = nn.ModuleList([Linear(D, 6 * D, True, dtype, device)])
        for n in ("norm_x1", "norm_y1", "norm_x2", "norm_y2"):
            setattr(self, n, RMSNorm(D, 1e-6, dtype, device))
        self.attn = _JointAttn(c, dtype, device)
        self.mlp_x, self.mlp_y = _SwiGLU(D, c.ffn_inner, dtype, device), _SwiGLU(D, c.ffn_inner, dtype, device)

    def forward(self, x, y, cond, img_rope, txt_rope):
        c, a = self.c, self.attn
        B, Nx, D = x.shape
        Ny = y.shape[1]
        H, hd = c.groups, c.head_dim
        mx, my = self.adaLN_modulation_img[0](cond), self.adaLN_modulation_txt[0](cond)
        ch = lambda m, j: m[:, j * D:(j + 1) * D]

        def qkv(h, s, rope):
            q, k, v = getattr(a, "qkv_" + s)(h).unflatten(-1, (3, H, hd)).unbind(2)
            return _rope_pairs(getattr(a, "q_norm_" + s)(q), *rope), _rope_pairs(getattr(a, "k_norm_" + s)(k), *rope), v

        qx, kx, vx = qkv(self.norm_x1(x, scale=ch(mx, 1), shift=ch(mx, 0)), "x", img_rope)
        qy, ky, vy = qkv(self.norm_y1(y, scale=ch(my, 1), shift=ch(my, 0)), "y", txt_rope)
        o = _attend(torch.cat((qy, qx), 1), torch.cat((ky, kx), 1), torch.cat((vy, vx), 1)).reshape(B, Ny + Nx, D)
        x = ops.gate_residual(x, a.proj_x(o[:, Ny:]), ch(mx, 2), Nx)
        y = ops.gate_residual(y, a.proj_y(o[:, :Ny]), ch(my, 2), Ny)
        x = ops.gate_residual(x, self.mlp_x(self.norm_x2(x, scale=ch(mx, 4), shift=ch(mx, 3))), ch(mx, 5), Nx)
        y = ops.gate_residual(y, self.mlp_y(self.norm_y2(y, scale=ch(my, 4), shift=ch(my, 3))), ch(my, 5), Ny)
        return x, y


class _RotaryAttn(nn.Module):
    def __init__(self, dim, heads, dtype, device):
        super().__init__()
        self.heads = heads
        self.qkv = Linear(dim, 3 * dim, False, dtype, device)
        self.proj = Linear(dim, dim, True, dtype, device)
        self.q_norm, self.k_norm = RMSNorm(dim // heads, 1e-6, dtype, device), RMSNorm(dim // heads, 1e-6, dtype, device)

    def forward(self, x, rope):
        B, N, D = x.shape
        q, k, v = self.qkv(x).unflatten(-1, (3, self.heads, D // self.heads)).unbind(2)
        return self.proj(_attend(_rope_pairs(self.q_norm(q), *rope), _rope_pairs(self.k_norm(k), *rope), v).reshape(B, N, D))


class _Mlp(nn.Module):
    def __init__(self, d, hidden, dtype, device):
        super().__init__()
        self.fc1, self.fc2 = Linear(d, hidden, True, dtype, device), Linear(hidden, d, True, dtype, device)


class PiTBlock(nn.Module):
    def __init__(self, c: PidConfig, dtype, device):
        super().__init__()
        self.c = c
        Cp, P2 = c.pixel_dim, c.patch_size ** 2
        self.adaLN_modulation = nn.ModuleList([Linear(c.hidden, 6 * Cp * P2, True, dtype, device)])
        self.norm1, self.norm2 = RMSNorm(Cp, 1e-6, dtype, device), RMSNorm(Cp, 1e-6, dtype, device)
        self.compress_to_attn = Linear(P2 * Cp, c.pixel_attn, True, dtype, device)
        self.expand_from_attn = Linear(c.pixel_attn, P2 * Cp, True, dtype, device)
        self.attn = _RotaryAttn(c.pixel_attn, c.pixel_groups, dtype, device)
        self.mlp = _Mlp(Cp, 4 * Cp, dtype, device)

    def forward(self, x, s_cond, B: int, rope):
        """x [B L, P2, Cp], s_cond [B L, hidden]."""
        c = self.c
        BL, P2, Cp = x.shape
        m = self.adaLN_modulation[0](s_cond).reshape(BL, P2, 6 * Cp)
        sh1, sc1, g1, sh2, sc2, g2 = m.chunk(6, -1)
        h = self.norm1(x) * (1 + sc1) + sh1
        t = self.attn(self.compress_to_attn(h.reshape(BL, P2 * Cp)).reshape(B, BL // B, c.pixel_attn), rope)
        x = x + g1 * self.expand_from_attn(t.reshape(BL, c.pixel_attn)).reshape(BL, P2, Cp)
        h = self.norm2(x) * (1 + sc2) + sh2
        return x + g2 * self.mlp.fc2(self.mlp.fc1(h, act="gelu"))


class _ConvP(nn.Module):
    def __init__(self, cin, cout, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(cout, 3, 3, cin, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cout, dtype=dtype, device=device))

    def forward(self, x, act=None):
        return C.conv2d_nhwc(x, self.weight, self.bias, 1, 1, act)


class _GN(nn.Module):
    def __init__(self, ch, dtype, device):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(ch, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(ch, dtype=dtype, device=device))


class _ResBlock(nn.Module):
    def __init__(self, ch, groups, dtype, device):
        super().__init__()
        self.groups = groups
        self.block = nn.ModuleDict({"0": _GN(ch, dtype, device), "2": _ConvP(ch, ch, dtype, device), "3": _GN(ch, dtype, device),
                                    "5": _ConvP(ch, ch, dtype, device)})

    def forward(self, x):
        b = self.block
        h = b["2"](C.group_norm_nhwc(x, b["0"].weight, b["0"].bias, self.groups, 1e-5, "silu"))
        return x + b["5"](C.group_norm_nhwc(h, b["3"].weight, b["3"].bias, self.groups, 1e-5, "silu"))


class _Gate(nn.Module):
    def __init__(self, d, dtype, device):
        super().__init__()
        self.content_proj = Linear(2 * d, d, True, dtype, device)
        self.log_alpha = nn.Parameter(torch.zeros((), dtype=dtype, device=device))

    def forward(self, x, lq, sigma: float):
        logit = self.content_proj(torch.cat((x, lq), -1)).float() - torch.exp(self.log_alpha.float()) * sigma
        return x + (torch.sigmoid(logit) * lq.float()).to(x.dtype)


class LQProjection(nn.Module):
    def __init__(self, c: PidConfig, dtype, device):
        super().__init__()
        n = (c.patch_depth + c.lq_interval - 1) // c.lq_interval
        self.latent_proj = nn.ModuleDict({"0": _ConvP(c.lq_channels, c.lq_hidden, dtype, device), "2": _ConvP(c.lq_hidden, c.lq_hidden, dtype, device),
                                          **{str(3 + i): _ResBlock(c.lq_hidden, c.lq_groups, dtype, device) for i in range(4)}})
        self.output_heads = nn.ModuleList([Linear(c.lq_hidden, c.hidden, True, dtype, device) for _ in range(n)])
        self.gate_modules = nn.ModuleList([_Gate(c.hidden, dtype, device) for _ in range(n)])

    def tokens(self, latent, ph: int, pw: int):
        """latent [B, C, zh, zw] -> [B, ph pw, lq_hidden] (nearest resize to the patch grid first)."""
        B, _, zh, zw = latent.shape
        iy = (torch.arange(ph, device=latent.device) * zh) // ph
        ix = (torch.arange(pw, device=latent.device) * zw) // pw
        x = latent[:, :, iy][:, :, :, ix].permute(0, 2, 3, 1).contiguous()
        lp = self.latent_proj
        h = lp["2"](lp["0"](x, "silu"))
        for i in range(3, 7):
            h = lp[str(i)](h)
        return h.reshape(B, ph * pw, -1)


class PidNet(nn.Module):
    """forward(x [B, 3, H, W] noisy pixels, t [B] (already multiplied by the time scale), caption [B, Lt, 2304], lq_latent
    [B, 16, zh, zw], sigma) -> velocity [B, 3, H, W]."""

    def __init__(self, cfg: PidConfig, dtype=torch.bfloat16, device=None):
        super().__init__()
        self.cfg = cfg
        D, ps = cfg.hidden, cfg.patch_size
        self.s_embedder = _Proj(3 * ps * ps, D, dtype, device)
        te = nn.Module()
        te.mlp = nn.ModuleDict({"0": Linear(cfg.freq_dim, D, True, dtype, device), "2": Linear(D, D, True, dtype, device)})
        self.t_embedder = te
        self.y_embedder = _Proj(cfg.txt_dim, D, dtype, device, norm=True)
        self.y_pos_embedding = nn.Parameter(torch.zeros(1, cfg.txt_max, D, dtype=dtype, device=device))
        self.lq_proj = LQProjection(cfg, dtype, device)
        self.patch_blocks = nn.ModuleList([PidMMDiTBlock(cfg, dtype, device) for _ in range(cfg.patch_depth)])
        self.pixel_embedder = _Proj(3, cfg.pixel_dim, dtype, device)
        self.pixel_blocks = nn.ModuleList([PiTBlock(cfg, dtype, device) for _ in range(cfg.pixel_depth)])
        fl = nn.Module()
        fl.norm = RMSNorm(cfg.pixel_dim, 1e-6, dtype, device)
        fl.linear = Linear(cfg.pixel_dim, 3, True, dtype, device)
        self.final_layer = fl

    @torch.no_grad()
    def forward(self, x, t, caption, lq_latent, sigma: float = 0.0):
        c = self.cfg
        B, _, H, W = x.shape
        ps = c.patch_size
        ph, pw = H // ps, W // ps
        L, P2 = ph * pw, ps * ps
        dev, dt = x.device, self.s_embedder.proj.weight.dtype
        x = x.to(dt)
        lq_tok = self.lq_proj.tokens(lq_latent.to(dt), ph, pw)
        s = self.s_embedder.proj(F.unfold(x, ps, stride=ps).transpose(1, 2))
        te = self.t_embedder.mlp
        t_emb = te["2"](te["0"](pid_timestep_embedding(t, c.freq_dim).to(dt), act="silu"))
        cond = ops.activation(t_emb, "silu")
        Lt = caption.shape[1]
        y = self.y_embedder.norm(self.y_embedder.proj(caption.to(dt))) + self.y_pos_embedding[:, :Lt]
        img_rope = ntk_rope_2d(c.head_dim, ph, pw, c.rope_ref, c.rope_ref, device=dev)
        txt_rope = text_rope_1d(Lt, c.head_dim, device=dev)
        for i, blk in enumerate(self.patch_blocks):
            if i % c.lq_interval == 0:
                j = i // c.lq_interval
                s = self.lq_proj.gate_modules[j](s, self.lq_proj.output_heads[j](lq_tok), sigma)
            s, y = blk(s, y, cond, img_rope, txt_rope)
        s_cond = ops.activation((s + t_emb[:, None]).reshape(B * L, c.hidden).contiguous(), "silu")
        px = self.pixel_embedder.proj(x.permute(0, 2, 3, 1)) + sincos_pos_2d(c.pixel_dim, H, W, dev).to(dt).reshape(1, H, W, -1)
        px = px.reshape(B, ph, ps, pw, ps, c.pixel_dim).permute(0, 1, 3, 2, 4, 5).reshape(B * L, P2, c.pixel_dim)
        pix_rope = ntk_rope_2d(c.pixel_attn // c.pixel_groups, ph, pw, c.rope_ref, c.rope_ref, device=dev)
        for blk in self.pixel_blocks:
            px = blk(px, s_cond, B, pix_rope)
        out = self.final_layer.linear(self.final_layer.norm(px))                               # [B L, P2, 3]
        out = out.reshape(B, L, P2, 3).permute(0, 3, 2, 1).reshape(B, 3 * P2, L)
        return F.fold(out.float(), (H, W), ps, stride=ps)

    def init_weights(self, seed: int = 0, std: float = 0.02):
        init_module_weights(self, seed, std)
        g = torch.Generator().manual_seed(seed + 2)
        with torch.no_grad():
            for m in self.modules():
                if isinstance(m, _ConvP):
                    fan = m.weight.shape[1] * m.weight.shape[2] * m.weight.shape[3]
                    m.weight.copy_((torch.randn(m.weight.shape, generator=g) / fan ** 0.5).to(m.weight.dtype))
        return self


def remap_pid_keys(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint convolution weights [out, in, kh, kw] -> [out, kh, kw, in]."""
    return {k: (v.permute(0, 2, 3, 1).contiguous() if v.dim() == 4 and k.startswith("lq_proj.latent_proj.") else v) for k, v in sd.items()}
