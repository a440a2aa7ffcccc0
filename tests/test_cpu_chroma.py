"""Chroma-shaped MMDiT: modulation-row bookkeeping, key inventory and forward parity with a plain-PyTorch statement."""
import math

import torch
import torch.nn.functional as F

from mojodiffusion_b200.models.chroma import ChromaDiT, chroma_config, tiny_chroma_config
from mojodiffusion_b200.models.mmdit import MMDiT


def _ln(x):
    return F.layer_norm(x, x.shape[-1:], eps=1e-6)


def _rms(x, w):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w


def _sin(t, dim):
    half = dim // 2
    f = torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)
    a = t[..., None] * f
    return torch.cat((a.cos(), a.sin()), -1)


def _rope(x, ids, axes, theta):
    ang = torch.cat([ids[:, a].double()[:, None] * (theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d))[None]
                     for a, d in enumerate(axes)], -1)
    c, s = ang.cos().float()[None, :, None], ang.sin().float()[None, :, None]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), -1).flatten(-2)


def _plain(sd, cfg, img, txt, t, hw):
    D, H, Dh = cfg.hidden, cfg.heads, cfg.head_dim
    lin = lambda x, k: F.linear(x, sd[k + ".weight"], sd[k + ".bias"])
    B, S_txt = img.shape[0], txt.shape[1]
    rows, q = cfg.mod_rows, cfg.approx_in // 4
    a_in = torch.cat((_sin(t * 1000.0, q)[:, None].expand(B, rows, q), _sin(torch.zeros(B), q)[:, None].expand(B, rows, q),
                      _sin(torch.arange(rows).float() * 1000.0, 2 * q)[None].expand(B, rows, 2 * q)), -1)
    h = lin(a_in, "distilled_guidance_layer.in_proj")
    for j in range(cfg.approx_layers):
        p = f"distilled_guidance_layer.layers.{j}"
        h = h + lin(F.silu(lin(_rms(h, sd[f"distilled_guidance_layer.norms.{j}.weight"]), p + ".linear_1")), p + ".linear_2")
    mod = lin(h, "distilled_guidance_layer.out_proj")                          # [B, rows, D]
    row = lambda r: mod[:, r:r + 1]
    ids = MMDiT.make_ids(hw[0], hw[1], S_txt)
    heads = lambda v: v.unflatten(-1, (H, Dh))
    sdpa = lambda q_, k_, v_: F.scaled_dot_product_attention(q_.transpose(1, 2), k_.transpose(1, 2), v_.transpose(1, 2)).transpose(1, 2).flatten(-2)
    img, txt = lin(img, "x_embedder"), lin(txt, "context_embedder")
    ns, nd = cfg.depth_single, cfg.depth_double
    for i in range(nd):
        p = f"transformer_blocks.{i}."
        bi, bt = 3 * ns + 6 * i, 3 * ns + 6 * nd + 6 * i
        xi = (1 + row(bi + 1)) * _ln(img) + row(bi)
        xt = (1 + row(bt + 1)) * _ln(txt) + row(bt)
        qq = torch.cat((_rms(heads(lin(xt, p + "attn.add_q_proj")), sd[p + "attn.norm_added_q.weight"]),
                        _rms(heads(lin(xi, p + "attn.to_q")), sd[p + "attn.norm_q.weight"])), 1)
        kk = torch.cat((_rms(heads(lin(xt, p + "attn.add_k_proj")), sd[p + "attn.norm_added_k.weight"]),
                        _rms(heads(lin(xi, p + "attn.to_k")), sd[p + "attn.norm_k.weight"])), 1)
        vv = torch.cat((heads(lin(xt, p + "attn.add_v_proj")), heads(lin(xi, p + "attn.to_v"))), 1)
        o = sdpa(_rope(qq, ids, cfg.axes_dim, cfg.theta), _rope(kk, ids, cfg.axes_dim, cfg.theta), vv)
        img = img + row(bi + 2) * lin(o[:, S_txt:], p + "attn.to_out.0")
        txt = txt + row(bt + 2) * lin(o[:, :S_txt], p + "attn.to_add_out")
        img = img + row(bi + 5) * lin(F.gelu(lin((1 + row(bi + 4)) * _ln(img) + row(bi + 3), p + "ff.net.0.proj"), approximate="tanh"), p + "ff.net.2")
        txt = txt + row(bt + 5) * lin(F.gelu(lin((1 + row(bt + 4)) * _ln(txt) + row(bt + 3), p + "ff_context.net.0.proj"), approximate="tanh"), p + "ff_context.net.2")
    x = torch.cat((txt, img), 1)
    for i in range(ns):
        p = f"single_transformer_blocks.{i}."
        xn = (1 + row(3 * i + 1)) * _ln(x) + row(3 * i)
        qq = _rope(_rms(heads(lin(xn, p + "attn.to_q")), sd[p + "attn.norm_q.weight"]), ids, cfg.axes_dim, cfg.theta)
        kk = _rope(_rms(heads(lin(xn, p + "attn.to_k")), sd[p + "attn.norm_k.weight"]), ids, cfg.axes_dim, cfg.theta)
        o = sdpa(qq, kk, heads(lin(xn, p + "attn.to_v")))
        x = x + row(3 * i + 2) * lin(torch.cat((o, F.gelu(lin(xn, p + "proj_mlp"), approximate="tanh")), -1), p + "proj_out")
    return lin((1 + row(rows - 1)) * _ln(x[:, S_txt:]) + row(rows - 2), "proj_out")


def test_chroma_forward_matches_plain_statement():
    cfg = tiny_chroma_config()
    m = ChromaDiT(cfg, torch.float32, "cpu").init_weights(5, std=0.05)
    with torch.no_grad():
        for n, prm in m.named_parameters():
            if prm.dim() == 1:
                gen = torch.Generator().manual_seed(len(n))
                prm.copy_((1.0 if "norm" in n else 0.0) + 0.1 * torch.randn(prm.shape, generator=gen))
    g = torch.Generator().manual_seed(0)
    hw, S_txt = (4, 6), 5
    img = torch.randn(2, 24, cfg.in_channels, generator=g)
    txt = torch.randn(2, S_txt, cfg.context_dim, generator=g)
    t = torch.tensor([0.3, 0.8])
    with torch.no_grad():
        got = m(img, txt, t, hw)
        want = _plain(m.state_dict(), cfg, img, txt, t, hw)
    assert torch.allclose(got, want, atol=3e-4, rtol=2e-3), float((got - want).abs().max())


def test_chroma_sizes_and_rows():
    cfg = chroma_config()
    assert cfg.mod_rows == 344
    with torch.device("meta"):
        m = ChromaDiT(cfg, torch.bfloat16, "meta")
    sd = m.state_dict()
    assert tuple(sd["distilled_guidance_layer.in_proj.weight"].shape) == (5120, 64)
    assert tuple(sd["distilled_guidance_layer.out_proj.weight"].shape) == (3072, 5120)
    assert "distilled_guidance_layer.norms.4.weight" in sd and "distilled_guidance_layer.layers.4.linear_2.bias" in sd
    assert tuple(sd["single_transformer_blocks.37.proj_out.weight"].shape) == (3072, 3072 + 12288)
    assert "transformer_blocks.18.ff_context.net.0.proj.weight" in sd and "transformer_blocks.0.attn.norm_added_k.weight" in sd
    assert not any("modulation" in k or "norm1.linear" in k for k in sd)
    n = sum(v.numel() for v in sd.values())
    assert 8.6e9 < n < 9.2e9, n
