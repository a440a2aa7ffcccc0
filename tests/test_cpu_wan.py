"""Wan2.2-shaped video DiT: sizes / keys and forward parity against a plain-PyTorch statement of the block."""
import torch
import torch.nn.functional as F

from mojodiffusion_b200.models.layers import timestep_embedding
from mojodiffusion_b200.models.wan import WanDiT, tiny_wan_config, wan22_ti2v_5b_config


def _ln(x, w=None, b=None):
    return F.layer_norm(x, x.shape[-1:], w, b, eps=1e-6)


def _rms(x, w):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w


def _rope(x, ids, axes, theta):
    ang = torch.cat([ids[:, a].double()[:, None] * (theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d))[None]
                     for a, d in enumerate(axes)], -1)
    c, s = ang.cos().float()[None, :, None], ang.sin().float()[None, :, None]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), -1).flatten(-2)


def _sdpa(q, k, v):
    return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(-2)


def _plain(sd, cfg, z, text, t):
    D, H, Dh = cfg.dim, cfg.heads, cfg.head_dim
    lin = lambda x, k: F.linear(x, sd[k + ".weight"], sd[k + ".bias"])
    heads = lambda v: v.unflatten(-1, (H, Dh))
    B, C, Fr, Hh, Ww = z.shape
    x = F.conv3d(z, sd["patch_embedding.weight"], sd["patch_embedding.bias"], stride=cfg.patch)
    f, h, w = x.shape[2:]
    x = x.flatten(2).transpose(1, 2)
    ids = WanDiT.make_ids(f, h, w)
    e = lin(F.silu(lin(timestep_embedding(t, cfg.freq_dim), "time_embedding.0")), "time_embedding.2")
    e0 = lin(F.silu(e), "time_projection.1").unflatten(1, (6, D))
    ctx = lin(F.gelu(lin(text, "text_embedding.0"), approximate="tanh"), "text_embedding.2")
    for i in range(cfg.depth):
        p = f"blocks.{i}."
        m = (sd[p + "modulation"] + e0).unbind(1)
        m = [v[:, None] for v in m]
        xn = _ln(x) * (1 + m[1]) + m[0]
        q = _rope(heads(_rms(lin(xn, p + "self_attn.q"), sd[p + "self_attn.norm_q.weight"])), ids, cfg.axes_dim, cfg.theta)
        k = _rope(heads(_rms(lin(xn, p + "self_attn.k"), sd[p + "self_attn.norm_k.weight"])), ids, cfg.axes_dim, cfg.theta)
        x = x + m[2] * lin(_sdpa(q, k, heads(lin(xn, p + "self_attn.v"))), p + "self_attn.o")
        xn = _ln(x, sd[p + "norm3.weight"], sd[p + "norm3.bias"])
        q = heads(_rms(lin(xn, p + "cross_attn.q"), sd[p + "cross_attn.norm_q.weight"]))
        k = heads(_rms(lin(ctx, p + "cross_attn.k"), sd[p + "cross_attn.norm_k.weight"]))
        x = x + lin(_sdpa(q, k, heads(lin(ctx, p + "cross_attn.v"))), p + "cross_attn.o")
        xn = _ln(x) * (1 + m[4]) + m[3]
        x = x + m[5] * lin(F.gelu(lin(xn, p + "ffn.0"), approximate="tanh"), p + "ffn.2")
    hm = (sd["head.modulation"] + e[:, None]).unbind(1)
    out = lin(_ln(x) * (1 + hm[1][:, None]) + hm[0][:, None], "head.head")
    pt, ph, pw = cfg.patch
    out = out.reshape(B, f, h, w, pt, ph, pw, cfg.out_dim)
    return torch.einsum("bfhwpqrc->bcfphqwr", out).reshape(B, cfg.out_dim, Fr, Hh, Ww)


def test_wan_forward_matches_plain_statement():
    cfg = tiny_wan_config()
    m = WanDiT(cfg, torch.float32, "cpu").init_weights(6, std=0.05)
    with torch.no_grad():
        for n, prm in m.named_parameters():
            if prm.dim() == 1:
                gen = torch.Generator().manual_seed(len(n))
                prm.copy_((1.0 if "norm" in n and n.endswith("weight") else 0.0) + 0.1 * torch.randn(prm.shape, generator=gen))
    g = torch.Generator().manual_seed(0)
    z = torch.randn(2, cfg.in_dim, 3, 4, 6, generator=g)
    text = torch.randn(2, 5, cfg.text_dim, generator=g)
    t = torch.tensor([0.3, 0.8])
    with torch.no_grad():
        got = m(z, text, t)
        want = _plain(m.state_dict(), cfg, z, text, t)
    assert got.shape == z.shape
    assert torch.allclose(got, want, atol=3e-4, rtol=2e-3), float((got - want).abs().max())


def test_wan_sizes_and_keys():
    cfg = wan22_ti2v_5b_config()
    assert cfg.axes_dim == (44, 42, 42)
    with torch.device("meta"):
        m = WanDiT(cfg, torch.bfloat16, "meta")
    sd = m.state_dict()
    assert tuple(sd["patch_embedding.weight"].shape) == (3072, 48, 1, 2, 2)
    assert tuple(sd["blocks.29.ffn.0.weight"].shape) == (14336, 3072)
    assert tuple(sd["blocks.0.modulation"].shape) == (1, 6, 3072) and tuple(sd["head.modulation"].shape) == (1, 2, 3072)
    assert tuple(sd["head.head.weight"].shape) == (48 * 4, 3072)
    for k in ("blocks.3.self_attn.norm_q.weight", "blocks.3.cross_attn.norm_k.weight", "blocks.3.norm3.bias",
              "text_embedding.2.bias", "time_projection.1.weight"):
        assert k in sd, k
    n = sum(v.numel() for v in sd.values())
    assert 4.6e9 < n < 5.4e9, n


def test_wan_vace_control_branch():
    """Wan-VACE: an untrained (zero-initialised) control branch leaves the output unchanged, a trained one changes it in
    proportion to ``control_scale``, hints land after base layers 0, 2, ..., and the checkpoint keys carry the control names."""
    import torch
    from mojodiffusion_b200.models.wan import WanVaceDiT, tiny_wan_vace_config, wan21_vace_14b_config
    cfg = tiny_wan_vace_config()
    m = WanVaceDiT(cfg, torch.float32).init_weights(0)
    z, txt, t = torch.randn(1, 8, 2, 8, 8), torch.randn(1, 6, 96), torch.tensor([0.5])
    c = torch.randn(1, cfg.vace_in_dim, 2, 8, 8)
    with torch.no_grad():
        base = m(z, txt, t)
        assert torch.equal(m(z, txt, t, control=c), base)
        for blk in m.vace_blocks:
            blk.after_proj.weight.normal_(0, 0.05)
        m.vace_blocks[0].before_proj.weight.normal_(0, 0.05)
        full = m(z, txt, t, control=c)
        assert (full - base).abs().max() > 1e-3
        assert torch.equal(m(z, txt, t, control=c, control_scale=0.0), base)
        short = m(z, txt, t, control=c[:, :, :1])                      # a shorter control clip is zero-padded in tokens
        assert short.shape == base.shape and torch.isfinite(short).all()
    keys = set(m.state_dict())
    assert {"vace_patch_embedding.weight", "vace_blocks.0.before_proj.weight", "vace_blocks.1.after_proj.bias"} <= keys
    assert "vace_blocks.1.before_proj.weight" not in keys
    assert [m.vace_layer(i) for i in range(cfg.vace_blocks)] == [0, 2]
    big = wan21_vace_14b_config()
    assert (big.dim, big.depth, big.heads, big.head_dim, big.vace_in_dim, big.vace_blocks) == (5120, 40, 40, 128, 96, 8)
