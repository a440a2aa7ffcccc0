"""FLUX.2 Klein-shaped MMDiT: checkpoint key inventory and forward parity against a plain-PyTorch statement of the block
op graph (LayerNorm -> modulate -> QKV -> per-head RMSNorm -> joint interleaved RoPE -> SDPA -> gated residual ->
SwiGLU MLP), plus a LoRA training step that lowers the loss."""
import math

import torch
import torch.nn.functional as F

from mojodiffusion_b200.models.flux2 import Flux2DiT, klein_9b_config, tiny_flux2_config
from mojodiffusion_b200.models.layers import timestep_embedding


def _ln(x):
    return F.layer_norm(x, x.shape[-1:], eps=1e-6)


def _rms(x, w):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w


def _rope(x, ids, axes, theta):
    # x: [B, S, H, Dh]; interleaved pairs, per axis frequencies theta^(-2i/axis_dim)
    ang = []
    for a, d in enumerate(axes):
        inv = theta ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)
        ang.append(ids[:, a].double()[:, None] * inv[None])
    ang = torch.cat(ang, -1)                                    # [S, Dh/2]
    c, s = ang.cos().float()[None, :, None], ang.sin().float()[None, :, None]
    x0, x1 = x[..., 0::2], x[..., 1::2]
    return torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), -1).flatten(-2)


def _attn(q, k, v):
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return o.transpose(1, 2).flatten(-2)


def _reference_forward(sd, cfg, img, txt, t, hw):
    D, H, Dh, Fh = cfg.hidden, cfg.heads, cfg.head_dim, cfg.mlp_hidden
    S_txt = txt.shape[1]
    ids = Flux2DiT.make_ids(hw[0], hw[1], S_txt)
    lin = lambda x, k: x @ sd[k].t()
    img, txt = lin(img, "img_in.weight"), lin(txt, "txt_in.weight")
    vec = lin(F.silu(lin(timestep_embedding(t, cfg.time_dim), "time_in.in_layer.weight")), "time_in.out_layer.weight")
    vs = F.silu(vec)
    mi = lin(vs, "double_stream_modulation_img.lin.weight")[:, None].chunk(6, -1)
    mt = lin(vs, "double_stream_modulation_txt.lin.weight")[:, None].chunk(6, -1)
    ms = lin(vs, "single_stream_modulation.lin.weight")[:, None].chunk(3, -1)

    def heads(x):
        return x.unflatten(-1, (H, Dh))

    for i in range(cfg.depth_double):
        p = f"double_blocks.{i}."
        qs, ks, vs_ = [], [], []
        for name, x, m in (("txt", txt, mt), ("img", img, mi)):
            q, k, v = lin((1 + m[1]) * _ln(x) + m[0], p + f"{name}_attn.qkv.weight").chunk(3, -1)
            qs.append(_rms(heads(q), sd[p + f"{name}_attn.norm.query_norm.scale"]))
            ks.append(_rms(heads(k), sd[p + f"{name}_attn.norm.key_norm.scale"]))
            vs_.append(heads(v))
        q, k, v = torch.cat(qs, 1), torch.cat(ks, 1), torch.cat(vs_, 1)
        a = _attn(_rope(q, ids, cfg.axes_dim, cfg.theta), _rope(k, ids, cfg.axes_dim, cfg.theta), v)
        outs = []
        for name, x, m, part in (("txt", txt, mt, a[:, :S_txt]), ("img", img, mi, a[:, S_txt:])):
            x = x + m[2] * lin(part, p + f"{name}_attn.proj.weight")
            g, u = lin((1 + m[4]) * _ln(x) + m[3], p + f"{name}_mlp.0.weight").chunk(2, -1)
            outs.append(x + m[5] * lin(F.silu(g) * u, p + f"{name}_mlp.2.weight"))
        txt, img = outs
    x = torch.cat((txt, img), 1)
    for i in range(cfg.depth_single):
        p = f"single_blocks.{i}."
        f = lin((1 + ms[1]) * _ln(x) + ms[0], p + "linear1.weight")
        q, k, v = f[..., :3 * D].chunk(3, -1)
        g, u = f[..., 3 * D:].chunk(2, -1)
        q = _rope(_rms(heads(q), sd[p + "norm.query_norm.scale"]), ids, cfg.axes_dim, cfg.theta)
        k = _rope(_rms(heads(k), sd[p + "norm.key_norm.scale"]), ids, cfg.axes_dim, cfg.theta)
        x = x + ms[2] * lin(torch.cat((_attn(q, k, heads(v)), F.silu(g) * u), -1), p + "linear2.weight")
    x = x[:, S_txt:]
    shift, scale = lin(vs, "final_layer.adaLN_modulation.1.weight")[:, None].chunk(2, -1)
    return lin((1 + scale) * _ln(x) + shift, "final_layer.linear.weight")


def test_klein_key_inventory_and_sizes():
    cfg = klein_9b_config()
    with torch.device("meta"):
        m = Flux2DiT(cfg, torch.bfloat16, "meta")
    keys = set(m.state_dict())
    want = {"img_in.weight", "txt_in.weight", "time_in.in_layer.weight", "time_in.out_layer.weight",
            "double_stream_modulation_img.lin.weight", "double_stream_modulation_txt.lin.weight",
            "single_stream_modulation.lin.weight", "final_layer.adaLN_modulation.1.weight", "final_layer.linear.weight"}
    for i in range(8):
        for s in ("img", "txt"):
            want |= {f"double_blocks.{i}.{s}_attn.qkv.weight", f"double_blocks.{i}.{s}_attn.proj.weight",
                     f"double_blocks.{i}.{s}_attn.norm.query_norm.scale", f"double_blocks.{i}.{s}_attn.norm.key_norm.scale",
                     f"double_blocks.{i}.{s}_mlp.0.weight", f"double_blocks.{i}.{s}_mlp.2.weight"}
    for i in range(24):
        want |= {f"single_blocks.{i}.linear1.weight", f"single_blocks.{i}.linear2.weight",
                 f"single_blocks.{i}.norm.query_norm.scale", f"single_blocks.{i}.norm.key_norm.scale"}
    assert keys == want
    sd = m.state_dict()
    assert tuple(sd["single_blocks.0.linear1.weight"].shape) == (3 * 4096 + 2 * 12288, 4096)
    assert tuple(sd["double_blocks.0.img_mlp.0.weight"].shape) == (2 * 12288, 4096)
    n = sum(p.numel() for p in m.parameters())
    assert 8.5e9 < n < 9.5e9, n


def test_flux2_forward_matches_plain_torch_statement():
    cfg = tiny_flux2_config()
    m = Flux2DiT(cfg, torch.float32, "cpu").init_weights(3, std=0.05)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(".scale"):
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=torch.Generator().manual_seed(len(n))))
    g = torch.Generator().manual_seed(0)
    hw, S_txt = (4, 6), 5
    img = torch.randn(2, hw[0] * hw[1], cfg.in_channels, generator=g)
    txt = torch.randn(2, S_txt, cfg.context_dim, generator=g)
    t = torch.tensor([0.3, 0.8])
    with torch.no_grad():
        got = m(img, txt, t, hw)
        want = _reference_forward(m.state_dict(), cfg, img, txt, t, hw)
    assert got.shape == (2, 24, cfg.in_channels)
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-3), float((got - want).abs().max())


def test_flux2_lora_step_reduces_loss():
    from mojodiffusion_b200.training import lora as L
    cfg = tiny_flux2_config()
    m = Flux2DiT(cfg, torch.float32, "cpu").init_weights(1, std=0.05)
    slots = L.inject_lora_by_name(m, {n: n for n in m.lora_target_names()}, rank=4, alpha=4.0)
    params = L.lora_parameters(slots)
    assert len(slots) == 2 * 2 * 4 + 2 * 2
    opt = torch.optim.AdamW(params, lr=2e-3)
    g = torch.Generator().manual_seed(0)
    x0 = torch.randn(1, 16, cfg.in_channels, generator=g)
    eps = torch.randn(1, 16, cfg.in_channels, generator=g)
    txt = torch.randn(1, 4, cfg.context_dim, generator=g)
    t = torch.tensor([0.5])
    m.gradient_checkpointing = True
    m.train()
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = (m((1 - t) * x0 + t * eps, txt, t, (4, 4)) - (eps - x0)).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss))
    assert losses[-1] < losses[0] * 0.98, losses
