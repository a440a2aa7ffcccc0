"""SD3.5-shaped MMDiT: key inventory / sizes and forward parity against a plain-PyTorch statement of the joint block."""
import torch
import torch.nn.functional as F

from mojodiffusion_b200.models.layers import timestep_embedding
from mojodiffusion_b200.models.sd3 import SD3MMDiT, sd35_large_config, sd35_medium_config, tiny_sd3_config


def _ln(x):
    return F.layer_norm(x, x.shape[-1:], eps=1e-6)


def _rms(x, w):
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * w


def _sdpa(q, k, v):
    return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(-2)


def _plain(sd, cfg, z, context, t, pooled):
    D, H, Dh, p = cfg.hidden, cfg.heads, cfg.head_dim, cfg.patch
    lin = lambda x, k: F.linear(x, sd[k + ".weight"], sd[k + ".bias"])
    B, C, Hh, Ww = z.shape
    h, w = Hh // p, Ww // p
    x = F.conv2d(z, sd["x_embedder.proj.weight"], sd["x_embedder.proj.bias"], stride=p).flatten(2).transpose(1, 2)
    G = cfg.pos_grid
    pe = sd["pos_embed"].reshape(1, G, G, D)[:, (G - h) // 2:(G - h) // 2 + h, (G - w) // 2:(G - w) // 2 + w].reshape(1, h * w, D)
    x = x + pe
    c = lin(F.silu(lin(timestep_embedding(t, cfg.time_dim), "t_embedder.mlp.0")), "t_embedder.mlp.2") \
        + lin(F.silu(lin(pooled, "y_embedder.mlp.0")), "y_embedder.mlp.2")
    cs = F.silu(c)
    ctx = lin(context, "context_embedder")
    heads = lambda v: v.unflatten(-1, (H, Dh))
    for i in range(cfg.depth):
        pc, px = f"joint_blocks.{i}.context_block.", f"joint_blocks.{i}.x_block."
        last, dual = i == cfg.depth - 1, i < cfg.dual_attention_blocks
        mc = lin(cs, pc + "adaLN_modulation.1")[:, None].chunk(2 if last else 6, -1)
        mx = lin(cs, px + "adaLN_modulation.1")[:, None].chunk(9 if dual else 6, -1)
        qc, kc, vc = lin((1 + mc[1]) * _ln(ctx) + mc[0], pc + "attn.qkv").chunk(3, -1)
        qx, kx, vx = lin((1 + mx[1]) * _ln(x) + mx[0], px + "attn.qkv").chunk(3, -1)
        q = torch.cat((_rms(heads(qc), sd[pc + "attn.ln_q.weight"]), _rms(heads(qx), sd[px + "attn.ln_q.weight"])), 1)
        k = torch.cat((_rms(heads(kc), sd[pc + "attn.ln_k.weight"]), _rms(heads(kx), sd[px + "attn.ln_k.weight"])), 1)
        a = _sdpa(q, k, torch.cat((heads(vc), heads(vx)), 1))
        S_ctx = ctx.shape[1]
        x_new = x + mx[2] * lin(a[:, S_ctx:], px + "attn.proj")
        if dual:
            q2, k2, v2 = lin((1 + mx[7]) * _ln(x) + mx[6], px + "attn2.qkv").chunk(3, -1)
            a2 = _sdpa(_rms(heads(q2), sd[px + "attn2.ln_q.weight"]), _rms(heads(k2), sd[px + "attn2.ln_k.weight"]), heads(v2))
            x_new = x_new + mx[8] * lin(a2, px + "attn2.proj")
        x = x_new
        x = x + mx[5] * lin(F.gelu(lin((1 + mx[4]) * _ln(x) + mx[3], px + "mlp.fc1"), approximate="tanh"), px + "mlp.fc2")
        if not last:
            ctx = ctx + mc[2] * lin(a[:, :S_ctx], pc + "attn.proj")
            ctx = ctx + mc[5] * lin(F.gelu(lin((1 + mc[4]) * _ln(ctx) + mc[3], pc + "mlp.fc1"), approximate="tanh"), pc + "mlp.fc2")
    shift, scale = lin(cs, "final_layer.adaLN_modulation.1")[:, None].chunk(2, -1)
    o = lin((1 + scale) * _ln(x) + shift, "final_layer.linear")
    o = o.reshape(B, h, w, p, p, C)
    return torch.einsum("nhwpqc->nchpwq", o).reshape(B, C, Hh, Ww)


def test_sd3_forward_matches_plain_statement():
    cfg = tiny_sd3_config()
    m = SD3MMDiT(cfg, torch.float32, "cpu").init_weights(4, std=0.05)
    with torch.no_grad():
        for n, prm in m.named_parameters():
            if "ln_" in n:
                prm.copy_(1.0 + 0.1 * torch.randn(prm.shape, generator=torch.Generator().manual_seed(len(n))))
            if n.endswith(".bias"):
                prm.copy_(0.05 * torch.randn(prm.shape, generator=torch.Generator().manual_seed(len(n) + 7)))
    g = torch.Generator().manual_seed(0)
    z = torch.randn(2, cfg.in_channels, 8, 12, generator=g)
    context = torch.randn(2, 7, cfg.context_dim, generator=g)
    pooled = torch.randn(2, cfg.pooled_dim, generator=g)
    t = torch.tensor([0.25, 0.9])
    with torch.no_grad():
        got = m(z, context, t, pooled)
        want = _plain(m.state_dict(), cfg, z, context, t, pooled)
    assert got.shape == z.shape
    assert torch.allclose(got, want, atol=3e-4, rtol=2e-3), float((got - want).abs().max())


def test_sd35_sizes_and_keys():
    for cfg, n_lo, n_hi in ((sd35_large_config(), 7.5e9, 8.6e9), (sd35_medium_config(), 2.0e9, 2.9e9)):
        with torch.device("meta"):
            m = SD3MMDiT(cfg, torch.bfloat16, "meta")
        sd = m.state_dict()
        n = sum(v.numel() for v in sd.values())
        assert n_lo < n < n_hi, (cfg.name, n)
        last = cfg.depth - 1
        assert f"joint_blocks.{last}.context_block.attn.qkv.weight" in sd
        assert f"joint_blocks.{last}.context_block.attn.proj.weight" not in sd            # pre_only
        assert f"joint_blocks.{last}.context_block.mlp.fc1.weight" not in sd
        assert tuple(sd[f"joint_blocks.{last}.context_block.adaLN_modulation.1.weight"].shape) == (2 * cfg.hidden, cfg.hidden)
        assert tuple(sd["x_embedder.proj.weight"].shape) == (cfg.hidden, 16, 2, 2)
        assert tuple(sd["pos_embed"].shape) == (1, cfg.pos_grid ** 2, cfg.hidden)
        has_dual = "joint_blocks.0.x_block.attn2.qkv.weight" in sd
        assert has_dual == (cfg.dual_attention_blocks > 0)
        if has_dual:
            assert tuple(sd["joint_blocks.0.x_block.adaLN_modulation.1.weight"].shape) == (9 * cfg.hidden, cfg.hidden)
            assert "joint_blocks.13.x_block.attn2.qkv.weight" not in sd
