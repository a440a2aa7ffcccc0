"""Image filters on RGBA fp32 images [H, W, 4]: SmartDenoise, HQDN3D, Guided, Deband, ColorBalance, CAS, USM, LUT3D,
WaterRipple, Soul, Sway, Star, Lighting, Jitter. On a CUDA tensor each call runs the kernels of ``csrc/shader_filters.cu``;
on a CPU tensor (or with ``reference=True``) the vectorised numpy statement of the same formulas below runs instead and
serves as the oracle of the kernels (every operation rounds to fp32, like the kernels built without fast-math / FMA).

Formulas and default parameters: shader_denoise_ref.py:63-300, shader_color_adv_ref.py:55-235,
shader_effects_ref.py:70-420 (CUDA-style originals: shader_denoise.mojo, shader_color_adv.mojo, shader_effects.mojo)."""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np
import torch

from . import native

OPS = {"smartdenoise": 0, "hqdn3d": 1, "guided": 2, "deband": 3, "colorbalance": 4, "cas": 5, "usm": 6, "lut3d": 7,
       "waterripple": 8, "soul": 9, "sway": 10, "star": 11, "lighting": 12, "jitter": 13}
f32 = np.float32


def test_image(H: int = 128, W: int = 128) -> np.ndarray:
    """Gradient background with a bright rectangle and a bright disc (the synthetic image the filters are checked on)."""
    ys, xs = np.mgrid[0:H, 0:W].astype(f32)
    r = (xs + ys) / f32(W + H - 2)
    g = xs / f32(W - 1)
    b = ys / f32(H - 1)
    rect = (xs >= 20) & (xs < 50) & (ys >= 20) & (ys < 50)
    disc = (xs - 90) ** 2 + (ys - 90) ** 2 < 18 * 18
    for m, c in ((rect, (0.95, 0.9, 0.1)), (disc, (0.1, 0.85, 0.95))):
        r = np.where(m, f32(c[0]), r)
        g = np.where(m, f32(c[1]), g)
        b = np.where(m, f32(c[2]), b)
    return np.stack([np.clip(r, 0, 1), np.clip(g, 0, 1), np.clip(b, 0, 1), np.ones_like(r)], -1).astype(f32)


def to_u8(img) -> np.ndarray:
    a = np.asarray(img, dtype=f32)
    a = np.where(np.isfinite(a), a, f32(1.0))
    return np.clip(np.floor(a * f32(255.0) + f32(0.5)), 0, 255).astype(np.uint8)


def psnr_u8(a, b) -> float:
    d = to_u8(a).astype(np.float64) - to_u8(b).astype(np.float64)
    mse = float((d * d).mean())
    return float("inf") if mse == 0 else 10.0 * math.log10(255.0 * 255.0 / mse)


# ---- host-side tables ------------------------------------------------------------------------------------------------
def hqdn3d_lut(luma_spatial: float = 4.0, chroma_spatial: float = 3.0, luma_tmp: float = 6.0) -> np.ndarray:
    """int32 [4, 8192]: (luma spatial, luma temporal, chroma spatial, chroma temporal) low-pass coefficient tables."""
    s_ls = luma_spatial
    s_cs = chroma_spatial * s_ls / luma_spatial
    s_lt = luma_tmp * s_ls / luma_spatial
    s_ct = s_lt * s_cs / s_ls
    lut = np.zeros((4, 8192), dtype=np.int32)
    i = np.arange(-4096, 4096, dtype=np.float64)
    ff = ((i * 32) + 16 - 1) / 512.0
    simil = np.maximum(0.0, 1.0 - np.abs(ff) / 255.0)
    for cls, strength in enumerate((s_ls, s_lt, s_cs, s_ct)):
        gamma = math.log(0.25) / math.log(1.0 - min(strength, 252.0) / 255.0 - 0.00001)
        cv = (simil ** gamma) * 256.0 * ff
        lut[cls] = np.where(cv >= 0, np.trunc(cv + 0.5), np.trunc(cv - 0.5)).astype(np.int32)
    return lut


def gaussian_taps(sigma: float, radius: int = 7) -> np.ndarray:
    d = np.arange(2 * radius + 1, dtype=f32) - f32(radius)
    w = np.exp(-(d * d) / f32(2.0 * sigma * sigma)).astype(f32)
    return (w / w.sum()).astype(f32)


def identity_lut(n: int = 17) -> np.ndarray:
    ri = np.arange(n, dtype=f32) / f32(n - 1)
    R, G, B = np.meshgrid(ri, ri, ri, indexing="ij")
    return np.stack([R, G, B, np.zeros_like(R)], -1).astype(f32)


# ---- numpy reference -------------------------------------------------------------------------------------------------------
def _ld(img, xi, yi):
    H, W = img.shape[:2]
    return img[np.clip(yi, 0, H - 1), np.clip(xi, 0, W - 1)]


def _grid(img):
    H, W = img.shape[:2]
    ys, xs = np.mgrid[0:H, 0:W]
    return xs, ys, H, W


def _uv(img):
    xs, ys, H, W = _grid(img)
    return xs.astype(f32) / f32(W - 1), ys.astype(f32) / f32(H - 1), H, W


def _tex(uv, n):
    return (uv * f32(n - 1)).astype(np.int64)


def _fract(x):
    return (x - np.floor(x)).astype(f32)


def _smoothstep(e0, e1, x):
    t = np.clip((x - f32(e0)) / f32(f32(e1) - f32(e0)), 0, 1).astype(f32)
    return (t * t * (f32(3.0) - f32(2.0) * t)).astype(f32)


def ref_smartdenoise(img, sigma=1.2, ksigma=2.0, threshold=0.2):
    sigma, ksigma, threshold = f32(sigma), f32(ksigma), f32(threshold)
    xs, ys, H, W = _grid(img)
    ig = f32(0.454545454545455)
    radius = f32(round(float(ksigma * sigma)))
    radq = radius * radius
    isq = f32(0.5) / (sigma * sigma)
    isq_pi = f32(0.31830988618379067) * isq
    itq = f32(0.5) / (threshold * threshold)
    it_pi = f32(0.3989422804014327) / threshold
    rgb = img[..., :3]
    cpow = np.power(rgb, ig).astype(f32)
    z = np.zeros((H, W), f32)
    acc = np.zeros((H, W, 3), f32)
    dx = -radius
    while dx <= radius:
        pt = f32(math.sqrt(float(radq - dx * dx)))
        dy = -pt
        while dy <= pt:
            bf = f32(math.exp(-float((dx * dx + dy * dy) * isq))) * isq_pi
            ix = (xs.astype(f32) + dx).astype(np.int64)          # truncation toward zero
            iy = (ys.astype(f32) + dy).astype(np.int64)
            w = _ld(img, ix, iy)[..., :3]
            d = np.power(w, ig).astype(f32) - cpow
            dot = (d[..., 0] * d[..., 0] + d[..., 1] * d[..., 1] + d[..., 2] * d[..., 2]).astype(f32)
            df = (np.exp(-(dot * itq)).astype(f32) * it_pi * bf).astype(f32)
            z = z + df
            acc = acc + df[..., None] * w
            dy = f32(dy + f32(1.0))
        dx = f32(dx + f32(1.0))
    out = np.empty_like(img)
    out[..., :3] = acc / z[..., None]
    out[..., 3] = 1.0
    return out


def ref_hqdn3d(img, lut=None):
    lut = hqdn3d_lut() if lut is None else lut
    r, g, b = (img[..., k].astype(np.float64) for k in range(3))
    c01 = lambda v: np.clip(v.astype(f32), 0, 1)
    yuv = [c01(0.262700 * r + 0.678000 * g + 0.059300 * b), c01(0.5 + (-0.139630 * r + -0.360370 * g + 0.500000 * b)),
           c01(0.5 + (0.500000 * r + -0.459786 * g + -0.040214 * b))]

    def lowpass(cur, cls):
        num = -cur
        dt = np.where(num >= 0, num // 16, -((-num) // 16))
        return cur + lut[cls][np.clip(dt + 4096, 0, 8191)]

    res = []
    for k, ch in enumerate(yuv):
        sp, tm = (0, 1) if k == 0 else (2, 3)
        pa = lowpass((ch * f32(65535.0)).astype(np.int64) + 128, sp)
        pa = lowpass(pa, sp)
        res.append((lowpass(pa, tm).astype(f32) / f32(65535.0)).astype(np.float64))
    yy, uu, vv = res[0], res[1] - 0.5, res[2] - 0.5
    out = np.empty_like(img)
    out[..., 0] = c01(yy + 1.474600 * vv)
    out[..., 1] = c01(yy + -0.164553 * uu + -0.571353 * vv)
    out[..., 2] = c01(yy + 1.881400 * uu)
    out[..., 3] = img[..., 3]
    return out


def _box(field, r):
    xs, ys, H, W = _grid(field)
    anchor, wv = r // 2, f32(1.0) / f32(r)
    tmp = np.zeros_like(field)
    for k in range(r):
        tmp = tmp + wv * _ld(field, xs - anchor + k, ys)
    out = np.zeros_like(field)
    for k in range(r):
        out = out + wv * _ld(tmp, xs, ys - anchor + k)
    return out.astype(f32)


def ref_guided(img, radius=4, eps=1e-4):
    mI = img.copy()
    mII = img.copy()
    mII[..., :3] = img[..., :3] * img[..., :3]
    bI, bII = _box(mI, radius), _box(mII, radius)
    var = bII[..., :3] - bI[..., :3] * bI[..., :3]
    a = var / (var + f32(eps))
    b = bI[..., :3] * (f32(1.0) - a)
    out = img.copy()
    out[..., :3] = np.clip(a * img[..., :3] + b, 0, 1)
    return out


def ref_deband(img, rng=16.0, direction=2.0 * math.pi, threshold=0.01):
    xs, ys, H, W = _grid(img)
    arg = xs.astype(f32) * f32(12.9898) + ys.astype(f32) * f32(78.233)
    r = np.sin(arg.astype(np.float64)).astype(f32) * f32(43758.545)
    fr = r - np.floor(r.astype(np.float64)).astype(f32)
    dirv = fr * f32(direction)
    dist = (fr * f32(rng)).astype(np.int64)
    xp = (np.cos(dirv.astype(np.float64)).astype(f32) * dist.astype(f32)).astype(np.int64)
    yp = (np.sin(dirv.astype(np.float64)).astype(f32) * dist.astype(f32)).astype(np.int64)
    refs = [_ld(img, xs + xp, ys + yp), _ld(img, xs + xp, ys - yp), _ld(img, xs - xp, ys - yp), _ld(img, xs - xp, ys + yp)]
    avg = ((refs[0] + refs[1] + refs[2] + refs[3]) / f32(4.0)).astype(f32)
    flat = np.ones(img.shape, bool)
    for q in refs:
        flat &= np.abs(img - q) < f32(threshold)
    out = np.where(flat, avg, img)
    out[..., 3] = img[..., 3]
    return out.astype(f32)


def ref_colorbalance(img, params=(0.3, -0.2, 0.1, -0.1, 0.25, -0.15, 0.2, -0.1, 0.3)):
    p = [f32(v) for v in params]
    rgb = img[..., :3]
    l = rgb.max(-1) + rgb.min(-1)
    a, b, scale = f32(4.0), f32(0.333), f32(0.7)
    out = img.copy()
    for c in range(3):
        s = p[c] * np.clip((b - l) * a + f32(0.5), 0, 1) * scale
        m = p[3 + c] * np.clip((l - b) * a + f32(0.5), 0, 1) * np.clip((f32(1.0) - l - b) * a + f32(0.5), 0, 1) * scale
        h = p[6 + c] * np.clip((l + b - f32(1.0)) * a + f32(0.5), 0, 1) * scale
        out[..., c] = np.clip(rgb[..., c] + s + m + h, 0, 1)
    return out


def ref_cas(img, strength=0.8):
    xs, ys, H, W = _grid(img)
    n = {(dx, dy): _ld(img, xs + dx, ys + dy)[..., :3] for dx in (-1, 0, 1) for dy in (-1, 0, 1)}
    a, b, c, d, e, f, g, h, i = (n[k] for k in ((-1, -1), (0, -1), (1, -1), (-1, 0), (0, 0), (1, 0), (-1, 1), (0, 1), (1, 1)))
    mn = np.minimum.reduce([d, e, f, b, h])
    mn = mn + np.minimum.reduce([mn, a, c, g, i])
    mx = np.maximum.reduce([d, e, f, b, h])
    mx = mx + np.maximum.reduce([mx, a, c, g, i])
    amp = np.sqrt(np.clip(np.minimum(mn, f32(2.0) - mx) / mx, 0, 1)).astype(f32)
    w = amp / f32(strength)
    out = img.copy()
    out[..., :3] = ((b + d + f + h) * w + e) / (f32(1.0) + f32(4.0) * w)
    return out


def ref_usm(img, sigma=3.0, amount=1.5, threshold=0.0):
    xs, ys, H, W = _grid(img)
    k = gaussian_taps(sigma)
    tmp = np.zeros_like(img)
    for t in range(15):
        tmp = tmp + k[t] * _ld(img, xs + t - 7, ys)
    blur = np.zeros_like(img)
    for t in range(15):
        blur = blur + k[t] * _ld(tmp, xs, ys + t - 7)
    diff = img[..., :3] - blur[..., :3]
    out = img.copy()
    out[..., :3] = np.clip(np.where(np.abs(diff) >= f32(threshold), img[..., :3] + f32(amount) * diff, img[..., :3]), 0, 1)
    return out


def ref_lut3d(img, lut=None):
    lut = identity_lut() if lut is None else lut
    N = lut.shape[0]
    sc = f32(N - 1)
    fr, fg, fb = (np.clip(img[..., k], 0, 1) * sc for k in range(3))
    r0, g0, b0 = (np.clip(v.astype(np.int64), 0, N - 2) for v in (fr, fg, fb))
    dr, dg, db = ((v - i0).astype(f32)[..., None] for v, i0 in ((fr, r0), (fg, g0), (fb, b0)))
    L = lambda ro, go, bo: lut[r0 + ro, g0 + go, b0 + bo, :3]
    c00 = L(0, 0, 0) * (1 - db) + L(0, 0, 1) * db
    c01 = L(0, 1, 0) * (1 - db) + L(0, 1, 1) * db
    c10 = L(1, 0, 0) * (1 - db) + L(1, 0, 1) * db
    c11 = L(1, 1, 0) * (1 - db) + L(1, 1, 1) * db
    c0 = c00 * (1 - dg) + c01 * dg
    c1 = c10 * (1 - dg) + c11 * dg
    out = img.copy()
    out[..., :3] = c0 * (1 - dr) + c1 * dr
    return out


def ref_waterripple(img, freq=24.0, amount=0.03):
    uvx, uvy, H, W = _uv(img)
    dx, dy = uvx - f32(0.5), uvy - f32(0.5)
    ln = np.sqrt(dx * dx + dy * dy).astype(f32)
    with np.errstate(divide="ignore", invalid="ignore"):
        fac = (f32(amount) * np.abs(np.sin(ln * f32(freq)).astype(f32))) / ln
        sx, sy = np.nan_to_num(uvx + dx * fac), np.nan_to_num(uvy + dy * fac)
    return _ld(img, _tex(sx.astype(f32), W), _tex(sy.astype(f32), H)).copy()


def _phase(progress_in, count, shrink):
    duration = f32(1.0) / f32(count)
    p = f32(progress_in)
    p = f32(f32(p - duration * f32(math.floor(float(p / duration)))) / duration)
    if shrink == 1 and p > 0.5:
        p = f32(f32(1.0) - p)
    return p, duration


def ref_soul(img, progress=0.37, count=1, max_scale=1.8, max_alpha=0.4, shrink=0):
    uvx, uvy, H, W = _uv(img)
    p, _ = _phase(progress, count, shrink)
    alpha = f32(max_alpha) * (f32(1.0) - p)
    scale = f32(1.0) + (f32(max_scale) - f32(1.0)) * p
    wx = np.clip(f32(0.5) + (uvx - f32(0.5)) / scale, 0, 1).astype(f32)
    wy = np.clip(f32(0.5) + (uvy - f32(0.5)) / scale, 0, 1).astype(f32)
    a = _ld(img, _tex(wx, W), _tex(wy, H))
    b = _ld(img, _tex(uvx, W), _tex(uvy, H))
    return (a * (f32(1.0) - alpha) + b * alpha).astype(f32)


def ref_sway(img, speed=7.4, strength=20.0, density=20.0, horizontal=1):
    uvx, uvy, H, W = _uv(img)
    wave = np.sin((uvy + f32(speed)) * f32(density)).astype(f32) * f32(strength) / f32(1000.0)
    if horizontal == 1:
        uvx = uvx + wave
    else:
        uvy = uvy + wave
    return _ld(img, _tex(np.clip(uvx, 0, 1).astype(f32), W), _tex(np.clip(uvy, 0, 1).astype(f32), H)).copy()


def ref_jitter(img, progress=0.37, count=1, max_scale=1.1, offset=0.02, shrink=0):
    uvx, uvy, H, W = _uv(img)
    p, _ = _phase(progress, count, shrink)
    offc = f32(offset) * p
    scale = f32(1.0) + (f32(max_scale) - f32(1.0)) * p
    scx = np.clip(f32(0.5) + (uvx - f32(0.5)) / scale, 0, 1).astype(f32)
    scy = np.clip(f32(0.5) + (uvy - f32(0.5)) / scale, 0, 1).astype(f32)
    c = lambda v: np.clip(v, 0, 1).astype(f32)
    r = _ld(img, _tex(c(scx + offc), W), _tex(c(scy + offc), H))
    b = _ld(img, _tex(c(scx - offc), W), _tex(c(scy - offc), H))
    m = _ld(img, _tex(scx, W), _tex(scy, H))
    return np.stack([r[..., 0], m[..., 1], b[..., 2], m[..., 3]], -1).astype(f32)


_SPI = f32(3.1415)


def _star_random(px, py):
    px, py = _fract(px * f32(123.45)), _fract(py * f32(345.67))
    d = (px * px + py * py) + f32(45.32) * (px + py)
    return _fract((px + d) * (py + d))


def _star_core(ux, uy, flaresize, rot):
    d = np.sqrt(ux * ux + uy * uy).astype(f32)
    with np.errstate(divide="ignore"):
        core = f32(0.05) / d
    ang = f32(-2.0) * _SPI * f32(rot)
    c, s = np.cos(np.array(ang, f32)), np.sin(np.array(ang, f32))
    ux, uy = c * ux - s * uy, s * ux + c * uy
    core = core + np.maximum(f32(1.0) - np.abs(ux * uy * f32(3000.0)), 0) * flaresize
    ang2 = _SPI * f32(0.25)
    c2, s2 = np.cos(np.array(ang2, f32)), np.sin(np.array(ang2, f32))
    nx, ny = c2 * ux - s2 * uy, s2 * ux + c2 * uy
    core = core + np.maximum(f32(1.0) - np.abs(nx * ny * f32(3000.0)), 0) * f32(0.3) * flaresize
    return (core * _smoothstep(1.0, 0.05, d)).astype(f32)


def ref_star(img, progress=0.37, speed=10.0, layers=2.0, red=1.0, green=0.1, blue=0.9):
    uvx, uvy, H, W = _uv(img)
    progress, speed, layers = f32(progress), f32(speed), f32(layers)
    colp = [f32(red), f32(green), f32(blue)]
    dtime, rot, stepi = progress * speed * f32(0.01), progress * speed * f32(0.09), f32(1.0) / layers
    col = [np.zeros((H, W), f32) for _ in range(3)]
    tx, ty = uvx, uvy
    i = f32(0.0)
    while i < f32(1.0):
        depth = f32(_fract(np.array(i + dtime, f32)))
        lscale = f32(64.0) + (f32(0.01) - f32(64.0)) * depth
        fader = depth * f32(_smoothstep(0.1, 1.1, np.array(depth, f32)))
        loff = i * (f32(3430.00) + f32(_fract(np.array(i, f32))))
        ang = np.array(rot * i * f32(-10.0), f32)
        c, s = np.cos(ang), np.sin(ang)
        tx, ty = (c * tx - s * ty).astype(f32), (s * tx + c * ty).astype(f32)
        sfx, sfy = tx * lscale + loff, ty * lscale + loff
        gvx, gvy, idx, idy = _fract(sfx) - f32(0.5), _fract(sfy) - f32(0.5), np.floor(sfx).astype(f32), np.floor(sfy).astype(f32)
        lc = [np.zeros((H, W), f32) for _ in range(3)]
        for yy in (-1, 0, 1):
            for xx in (-1, 0, 1):
                ox, oy = f32(xx), f32(yy)
                rn = _star_random(idx + ox, idy + oy)
                rpx = gvx - ox - (rn - f32(0.5))
                rpy = gvy - oy - (_fract(rn * f32(45.0)) - f32(0.5))
                size = _fract(rn * f32(1356.33))
                st = _star_core(rpx, rpy, _smoothstep(0.9, 1.0, size), rot)
                seed = _fract(rn * f32(2150.0)) * (f32(3.0) * _SPI) * progress
                m = f32(0.4) * np.sin(np.array(progress, f32))
                dim = f32(15.0) / layers
                for k in range(3):
                    cc = np.sin(colp[k] * seed).astype(f32) * m + f32(0.6)
                    cc = cc * ((colp[k] + size) if k == 2 else colp[k])
                    lc[k] = lc[k] + st * size * cc * dim
        for k in range(3):
            col[k] = col[k] + lc[k] * fader
        i = f32(i + stepi)
    out = img.copy()
    for k in range(3):
        out[..., k] = img[..., k] + col[k]
    return out


def _rgb2hcv(r, g, b):
    lt = g < b
    px, py = np.where(lt, b, g), np.where(lt, g, b)
    pz, pw = np.where(lt, f32(-1.0), f32(0.0)), np.where(lt, f32(2.0 / 3.0), f32(-1.0 / 3.0))
    lt2 = r < px
    qx, qy, qz, qw = np.where(lt2, px, r), py, np.where(lt2, pw, pz), np.where(lt2, r, px)
    c = qx - np.minimum(qw, qy)
    h = np.abs((qw - qy) / (f32(6.0) * c + f32(1.0e-10)) + qz)
    return h.astype(f32), c.astype(f32), qx.astype(f32)


def ref_lighting(img, progress=0.37, count=1, saturation=0.3, light=0.3):
    p, duration = _phase(progress, count, 0)
    hue = f32(abs(f32(np.sin(np.array(p * (f32(3.1415926) / duration), f32))))) * f32(360.0) / f32(360.0)
    r, g, b = img[..., 0], img[..., 1], img[..., 2]
    fh, c, fv = _rgb2hcv(r, g, b)
    fs = c / (fv + f32(1.0e-10))
    fh = fh + hue
    fv = np.clip(fv + f32(saturation) / f32(10.0), 0, 1).astype(f32)
    m = [fv * ((f32(1.0) - fs) + np.clip(np.abs(_fract(fh + K) * f32(6.0) - f32(3.0)) - f32(1.0), 0, 1) * fs)
         for K in (f32(1.0), f32(2.0 / 3.0), f32(1.0 / 3.0))]
    lh, lc, lv = _rgb2hcv(*[v.astype(f32) for v in m])
    z = lv - lc * f32(0.5)
    az = np.abs(f32(2.0) * z - f32(1.0))
    ls = np.clip(lc / (f32(1.0) - az + f32(1.0e-10)) + f32(saturation) * f32(0.5), 0, 1).astype(f32)
    hr = np.clip(np.abs(lh * f32(6.0) - f32(3.0)) - f32(1.0), 0, 1)
    hg = np.clip(f32(2.0) - np.abs(lh * f32(6.0) - f32(2.0)), 0, 1)
    hb = np.clip(f32(2.0) - np.abs(lh * f32(6.0) - f32(4.0)), 0, 1)
    cc = (f32(1.0) - az) * ls
    out = img.copy()
    for k, hk in enumerate((hr, hg, hb)):
        out[..., k] = ((hk - f32(0.5)) * cc + z) * (f32(1.0) - f32(light)) + f32(1.0) * f32(light)
    return out.astype(f32)


REFERENCE = {"smartdenoise": ref_smartdenoise, "hqdn3d": ref_hqdn3d, "guided": ref_guided, "deband": ref_deband,
             "colorbalance": ref_colorbalance, "cas": ref_cas, "usm": ref_usm, "lut3d": ref_lut3d,
             "waterripple": ref_waterripple, "soul": ref_soul, "sway": ref_sway, "star": ref_star,
             "lighting": ref_lighting, "jitter": ref_jitter}


# ---- public API ----------------------------------------------------------------------------------------------------------------
def _params(name: str, kw: dict):
    g = kw.get
    if name == "smartdenoise":
        return [g("sigma", 1.2), g("ksigma", 2.0), g("threshold", 0.2)], None
    if name == "hqdn3d":
        return [], torch.from_numpy(kw["lut"] if "lut" in kw else hqdn3d_lut())
    if name == "guided":
        return [g("radius", 4), g("eps", 1e-4)], None
    if name == "deband":
        return [g("rng", 16.0), float(f32(g("direction", 2.0 * math.pi))), g("threshold", 0.01)], None
    if name == "colorbalance":
        return list(g("params", (0.3, -0.2, 0.1, -0.1, 0.25, -0.15, 0.2, -0.1, 0.3))), None
    if name == "cas":
        return [g("strength", 0.8)], None
    if name == "usm":
        return [g("amount", 1.5), g("threshold", 0.0)] + [float(v) for v in gaussian_taps(g("sigma", 3.0))], None
    if name == "lut3d":
        lut = kw["lut"] if "lut" in kw else identity_lut()
        return [lut.shape[0]], torch.from_numpy(np.ascontiguousarray(lut, dtype=f32))
    if name == "waterripple":
        return [g("freq", 24.0), g("amount", 0.03)], None
    if name == "soul":
        return [g("progress", 0.37), g("count", 1), g("max_scale", 1.8), g("max_alpha", 0.4), g("shrink", 0)], None
    if name == "sway":
        return [g("speed", 7.4), g("strength", 20.0), g("density", 20.0), g("horizontal", 1)], None
    if name == "star":
        return [g("progress", 0.37), g("speed", 10.0), g("layers", 2.0), g("red", 1.0), g("green", 0.1), g("blue", 0.9)], None
    if name == "lighting":
        return [g("progress", 0.37), g("count", 1), g("saturation", 0.3), g("light", 0.3)], None
    if name == "jitter":
        return [g("progress", 0.37), g("count", 1), g("max_scale", 1.1), g("offset", 0.02), g("shrink", 0)], None
    raise KeyError(name)


def image_filter(name: str, img: torch.Tensor, reference: bool = False, **kw) -> torch.Tensor:
    """Apply filter ``name`` to an RGBA fp32 image [H, W, 4]. Keyword arguments are the filter's parameters (defaults as
    in the formulas' source)."""
    if name not in OPS:
        raise KeyError(f"unknown filter '{name}'; have {sorted(OPS)}")
    if img.dim() != 3 or img.shape[-1] != 4:
        raise ValueError("image_filter wants [H, W, 4]")
    if img.is_cuda and not reference:
        native.load(True)
        params, aux = _params(name, kw)
        if aux is not None:
            aux = aux.to(img.device)
        return native.ops().image_filter(OPS[name], img.float().contiguous(), [float(p) for p in params], aux)
    out = REFERENCE[name](img.detach().float().cpu().numpy(), **kw)
    return torch.from_numpy(np.ascontiguousarray(out, dtype=f32)).to(img.device)
