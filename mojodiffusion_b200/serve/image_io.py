"""Init / mask / reference image input of the serving workers: PNG load, channel handling, Lanczos-3 resampling.

    load_image_rgb(path)          -> float [1, 3, H, W] in [-1, 1]   (gray -> 3 planes, alpha composited over white)
    load_mask(path)               -> float [1, 1, H, W] in [0, 1]    (alpha plane when it carries information, else luminance)
    resize_lanczos(x, h, w)       -> separable Lanczos-3, kernel widened by the reduction ratio when shrinking (anti-aliased)
    fit_image(x, h, w, mode)      -> "stretch" | "crop" (centre crop to the aspect, then resize) | "pad" (letterbox)

The control plane's hires second pass hands the base image over as ``init_image`` with the target size; the resampling
happens here, in the worker (serenitymojo/serve/image_io.mojo, serenity-server/crates/server/src/main.rs:1812-1830).
"""
from __future__ import annotations

import math
from typing import Tuple

import numpy as np
import torch

from ..io.png import load_png


def _to_float(img: np.ndarray) -> torch.Tensor:
    a = torch.from_numpy(np.ascontiguousarray(img))
    if a.dtype == torch.uint8:
        return a.float() / 255.0
    if a.dtype in (torch.int16, torch.uint16, torch.int32):
        return a.float() / 65535.0
    return a.float()


def load_image_rgb(path: str) -> torch.Tensor:
    img, _ = load_png(path)
    t = _to_float(img)
    if t.dim() == 2:
        t = t[..., None]
    c = t.shape[-1]
    if c == 1:
        rgb = t.expand(-1, -1, 3)
    elif c == 2:                                           # gray + alpha
        rgb = (t[..., :1] * t[..., 1:] + (1.0 - t[..., 1:])).expand(-1, -1, 3)
    elif c == 4:
        rgb = t[..., :3] * t[..., 3:] + (1.0 - t[..., 3:])
    else:
        rgb = t[..., :3]
    return (rgb.permute(2, 0, 1)[None] * 2.0 - 1.0).contiguous()


def load_mask(path: str) -> torch.Tensor:
    img, _ = load_png(path)
    t = _to_float(img)
    if t.dim() == 2:
        m = t
    elif t.shape[-1] in (2, 4) and float(t[..., -1].min()) < 1.0:
        m = 1.0 - t[..., -1]                               # transparent = to be repainted
    elif t.shape[-1] >= 3:
        m = 0.299 * t[..., 0] + 0.587 * t[..., 1] + 0.114 * t[..., 2]
    else:
        m = t[..., 0]
    return m[None, None].clamp(0.0, 1.0).contiguous()


def _lanczos_matrix(n_in: int, n_out: int, a: int = 3) -> torch.Tensor:
    """[n_out, n_in] resampling weights (pixel centres aligned, edges clamped, rows normalised)."""
    scale = n_in / n_out
    support = a * max(scale, 1.0)
    centres = (torch.arange(n_out, dtype=torch.float64) + 0.5) * scale - 0.5
    lo = torch.floor(centres - support).to(torch.int64)
    taps = int(math.ceil(2 * support)) + 2
    idx = lo[:, None] + torch.arange(taps)[None, :]
    x = (idx.to(torch.float64) - centres[:, None]) / max(scale, 1.0)
    wgt = torch.where(x.abs() < a, torch.sinc(x) * torch.sinc(x / a), torch.zeros_like(x))
    wgt = wgt / wgt.sum(dim=1, keepdim=True)
    m = torch.zeros(n_out, n_in, dtype=torch.float64)
    m.scatter_add_(1, idx.clamp(0, n_in - 1), wgt)
    return m.float()


def resize_lanczos(x: torch.Tensor, h: int, w: int) -> torch.Tensor:
    """x [B, C, H, W] -> [B, C, h, w]."""
    H, W = x.shape[-2:]
    if (H, W) == (h, w):
        return x
    y = x.float()
    if W != w:
        y = torch.matmul(y, _lanczos_matrix(W, w).t().to(y.device))
    if H != h:
        y = torch.matmul(_lanczos_matrix(H, h).to(y.device), y)
    return y.to(x.dtype) if x.dtype.is_floating_point else y


def fit_image(x: torch.Tensor, h: int, w: int, mode: str = "stretch", pad_value: float = 0.0) -> torch.Tensor:
    H, W = x.shape[-2:]
    if mode == "stretch":
        return resize_lanczos(x, h, w)
    if mode == "crop":
        r = max(h / H, w / W)
        ch, cw = min(H, int(round(h / r))), min(W, int(round(w / r)))
        y0, x0 = (H - ch) // 2, (W - cw) // 2
        return resize_lanczos(x[..., y0:y0 + ch, x0:x0 + cw], h, w)
    if mode == "pad":
        r = min(h / H, w / W)
        nh, nw = max(1, int(round(H * r))), max(1, int(round(W * r)))
        out = torch.full((*x.shape[:-2], h, w), pad_value, dtype=torch.float32)
        y0, x0 = (h - nh) // 2, (w - nw) // 2
        out[..., y0:y0 + nh, x0:x0 + nw] = resize_lanczos(x, nh, nw).float()
        return out
    raise ValueError(f"unknown fit mode '{mode}'")


def image_size(path: str) -> Tuple[int, int]:
    img, _ = load_png(path)
    return int(img.shape[1]), int(img.shape[0])
