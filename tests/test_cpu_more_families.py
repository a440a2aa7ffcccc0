"""ERNIE-Image and Anima single-stream families: forward contracts, checkpoint key names, masks, adapters, schedules, and a
few optimisation steps through the shared family trainer."""
import torch

from mojodiffusion_b200.models import anima as A
from mojodiffusion_b200.models import ernie as E
from mojodiffusion_b200.runtime import default_manifest_by_id
from mojodiffusion_b200.runtime.adapters import adapter_for, schedule_for


def test_ernie_forward_mask_and_keys():
    cfg = E.tiny_ernie_config()
    m = E.ErnieImage(cfg, dtype=torch.float32)
    g = torch.Generator().manual_seed(0)
    with torch.no_grad():
        m.init_weights(0)
        img, txt = torch.randn(2, 16, cfg.in_channels, generator=g), torch.randn(2, 6, cfg.text_dim, generator=g)
        s = torch.tensor([0.3, 0.9])
        out = m(img, txt, s, (4, 4))
        assert out.shape == img.shape and torch.isfinite(out).all()
        masked = m(img, txt, s, (4, 4), text_len=torch.tensor([3, 6]))
        assert (masked - out)[0].abs().max() > 1e-6 and torch.equal(masked[1], out[1])      # only the padded sample changes
        txt2 = txt.clone()
        txt2[0, 3:] = 7.0                                                                  # padded text keys are ignored
        assert torch.allclose(m(img, txt2, s, (4, 4), text_len=torch.tensor([3, 6]))[0], masked[0], atol=1e-5)
    keys = set(m.state_dict())
    for k in ("x_embedder.proj.weight", "time_embedding.linear_2.bias", "text_proj.weight", "adaLN_modulation.1.weight",
              "layers.1.adaLN_sa_ln.weight", "layers.0.self_attention.to_out.0.weight", "layers.0.self_attention.norm_k.weight",
              "layers.0.mlp.gate_proj.weight", "layers.1.mlp.linear_fc2.weight", "final_norm.linear.weight", "final_linear.bias"):
        assert k in keys, k
    assert "text_proj.bias" not in keys and m.adaLN_modulation["1"].weight.shape[0] == 6 * cfg.hidden
    sig = E.ernie_sigmas(50, 3.0)
    assert len(sig) == 51 and sig[0] == 1.0 and sig[-1] == 0.0 and abs(sig[25] - 3 * 0.5 / (1 + 2 * 0.5)) < 1e-6
    full = E.ernie_config()
    assert (full.hidden, full.heads, full.depth, full.ffn_hidden, full.theta, full.axes_dim) == (4096, 32, 36, 12288, 256.0, (32, 48, 48))


def test_anima_forward_patch_layout_and_keys():
    cfg = A.tiny_anima_config()
    m = A.Anima(cfg, dtype=torch.float32)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        m.init_weights(0)
        z, ctx = torch.randn(2, 4, 1, 8, 8, generator=g), torch.randn(2, 5, cfg.context_dim, generator=g)
        s = torch.tensor([0.2, 0.7])
        out = m(z, ctx, s)
        assert out.shape == z.shape and torch.isfinite(out).all()
        assert m(z[:, :, 0], ctx, s).shape == (2, 4, 8, 8)                                  # images may come 4-D
        tok, grid = m.patchify(z)
        assert tok.shape == (2, 16, cfg.patch_in) and grid == (1, 4, 4)
        # token (row 1, col 2) holds channel c at in-patch (dy, dx) in slot (c * 2 + dy) * 2 + dx; the mask channel is zero
        c, dy, dx = 3, 1, 0
        assert tok[1, 1 * 4 + 2, (c * 2 + dy) * 2 + dx] == z[1, c, 0, 2 * 1 + dy, 2 * 2 + dx]
        assert float(tok[..., 4 * 4:].abs().max()) == 0.0
        y = torch.arange(2 * 16 * cfg.patch_out, dtype=torch.float32).reshape(2, 16, cfg.patch_out)
        img = m.unpatchify(y, grid)
        assert img[1, c, 0, 2 * 1 + dy, 2 * 2 + dx] == y[1, 1 * 4 + 2, (dy * 2 + dx) * 4 + c]      # output slots are (dy, dx, c)
        short = m(z, ctx, s, ctx_len=torch.tensor([2, 5]))
        assert (short - out)[0].abs().max() > 1e-6 and torch.equal(short[1], out[1])
    keys = set(m.state_dict())
    for k in ("net.x_embedder.proj.1.weight", "net.t_embedder.1.linear_2.weight", "net.t_embedding_norm.weight",
              "net.blocks.0.self_attn.q_norm.weight", "net.blocks.1.cross_attn.k_proj.weight", "net.blocks.0.mlp.layer2.weight",
              "net.blocks.0.adaln_modulation_cross_attn.2.weight", "net.final_layer.adaln_modulation.1.weight", "net.final_layer.linear.weight"):
        assert k in keys, k
    assert not any(k.endswith(".bias") for k in keys)
    assert m.net.blocks[0].cross_attn.k_proj.weight.shape == (cfg.hidden, cfg.context_dim)
    assert A.anima_config().patch_in == 68 and A.anima_config().patch_out == 64


def test_both_families_train_through_the_family_trainer():
    from mojodiffusion_b200.io.config import TrainConfig
    from mojodiffusion_b200.training.family_trainer import FamilyTrainer
    from mojodiffusion_b200.training.optim import FusedAdamW
    for mid, C, D in (("ernie-image", 16, 96), ("anima", 4, 96)):
        man = default_manifest_by_id(mid)
        model = man.build(tiny=True, dtype=torch.float32)
        with torch.no_grad():
            model.init_weights(0)
        ad = adapter_for(man)
        slots = ad.inject_lora(model, rank=4, alpha=4.0)
        params = [p for s in slots for p in (s.down, s.up)]
        cfg = TrainConfig()
        cfg.learning_rate, cfg.seed = 2e-3, 5
        tr = FamilyTrainer(ad, model, params, FusedAdamW(params, lr=2e-3), cfg)
        g = torch.Generator().manual_seed(2)
        batch = {"latent": torch.randn(2, C, 8, 8, generator=g), "text_embedding": torch.randn(2, 6, D, generator=g), "text_mask": torch.ones(2, 6)}
        losses = [float(tr.step(batch)) for _ in range(6)]
        assert all(l == l for l in losses) and all(float(s.up.abs().sum()) > 0 for s in slots)
        assert slots[0].key.startswith("transformer.layers.0." if mid == "ernie-image" else "diffusion_model.net.blocks.0.")
        sig = schedule_for(man, man.schedule.steps, 1024)
        assert len(sig) == man.schedule.steps + 1 and sig[0] == 1.0 and sig[-1] == 0.0


def test_asymflux2_velocity_oklab_and_sampler():
    """AsymFLUX.2: the one-projection velocity equals the two-branch statement, Oklab round-trips, the gamut clamp and the
    orthogonal guidance behave as defined, and the pixel-space sampler runs on a tiny transformer."""
    import dataclasses
    from mojodiffusion_b200.models import asymflux2 as A
    from mojodiffusion_b200.models.flux2 import Flux2DiT, tiny_flux2_config
    torch.manual_seed(0)
    B, N, D, R = 2, 16, 768, 32
    P = torch.linalg.qr(torch.randn(D, R))[0]
    ua, xt = torch.randn(B, N, D), torch.randn(B, N, D)
    cal = A.compute_calibration(0.7, 0.3)
    assert abs(cal.k - 1.0 / (0.3 + 0.7 * 0.7)) < 1e-12 and abs(cal.cal_timestep - 0.7 * cal.k) < 1e-12
    sub = lambda z: (z @ P) @ P.t()
    sk = cal.s * cal.k
    want = sk * sub(ua) + (1 - sk) / cal.sigma * sub(xt) + ((xt - sub(xt)) + cal.s * (ua - sub(ua))) / cal.sigma
    assert (A.asymflow_velocity(ua, xt, cal, P) - want).abs().max() < 1e-4
    tiny = A.compute_calibration(1e-7, 0.3)                          # sigma below the floor is clamped
    assert torch.isfinite(A.asymflow_velocity(ua, xt, tiny, P)).all()
    rgb = torch.rand(2, 3, 8, 8) * 2 - 1
    assert (A.oklab_decode(A.oklab_encode(rgb)) - rgb).abs().max() < 1e-3
    white = A.oklab_encode(torch.ones(1, 3, 1, 1))
    assert abs(float(white[0, 0]) * A.OKLAB_STD + A.OKLAB_MEAN[0] - 1.0) < 1e-3       # L of white is 1
    x = torch.randn(1, 3, 8, 8) * 3
    v = A.clamp_denoised_oklab(x, torch.zeros_like(x), 0.5)
    den = A.oklab_decode(x - v * 0.5)
    assert den.min() >= -1 - 1e-4 and den.max() <= 1 + 1e-4
    pos, neg, par = torch.randn(2, 3, 4, 4), torch.randn(2, 3, 4, 4), torch.randn(2, 3, 4, 4)
    b = A.guidance_bias(pos, neg, 4.0, 1.0, par)
    assert (b * par).mean((1, 2, 3)).abs().max() < 1e-5              # fully orthogonalised
    assert torch.equal(A.guidance_bias(pos, neg, 4.0, 0.0, par), (pos - neg) * 3.0)
    sig = A.sigma_schedule(4, A.dynamic_shift(1024, 1024))
    assert abs(A.dynamic_shift(1024, 1024) - 17.0) < 1e-9 and abs(A.dynamic_shift(2048, 2048) - 34.0) < 1e-9
    assert sig[0] == 1.0 and sig[-1] == 0.0 and all(a > b for a, b in zip(sig, sig[1:]))
    cfg = dataclasses.replace(tiny_flux2_config(), in_channels=768)
    m = A.AsymFlux2(Flux2DiT(cfg, torch.float32).init_weights(0), P, 0.3)
    img = m.sample(torch.randn(1, 3, 32, 32), torch.randn(1, 8, cfg.context_dim), torch.randn(1, 8, cfg.context_dim), steps=3)
    assert img.shape == (1, 3, 32, 32) and torch.isfinite(img).all() and img.abs().max() <= 1 + 1e-4


def test_ideogram4_matches_plain_torch_statement():
    """Ideogram-4: the model equals a plain-torch statement of the published forward (rotate-half rotary with full-width
    interleaved three-axis tables, separate w1 / w3, masks from the indicator), and reference checkpoint keys load."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models.ideogram4 import (IND_IMAGE, IND_TEXT, Ideogram4DiT, mrope_table, remap_ideogram4_keys,
                                                     scalar_embedding, tiny_ideogram4_config)
    torch.manual_seed(0)
    cfg = tiny_ideogram4_config()
    m = Ideogram4DiT(cfg, torch.float32).init_weights(3)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    # a checkpoint in reference naming: w1 / w3 separate
    ref_sd = {}
    for k, v in m.state_dict().items():
        if k.endswith("feed_forward.w13.weight"):
            ref_sd[k.replace("w13", "w1")], ref_sd[k.replace("w13", "w3")] = v[:cfg.mlp_hidden].clone(), v[cfg.mlp_hidden:].clone()
        else:
            ref_sd[k] = v.clone()
    m2 = Ideogram4DiT(cfg, torch.float32)
    m2.load_state_dict(remap_ideogram4_keys(ref_sd))
    L, D, H, Dh = 12, cfg.hidden, cfg.heads, cfg.head_dim
    ind = torch.tensor([[3] * 4 + [2] * 6 + [0] * 2])
    pos = torch.stack([torch.zeros(L), torch.arange(L).float() * 7.0, torch.arange(L).float() * 3.0], 1)
    x, llm, t = torch.randn(1, L, cfg.in_channels), torch.randn(1, L, cfg.llm_dim), torch.tensor([0.4])
    got = m2(x, llm, t, ind, pos)

    sd = ref_sd
    lin = lambda v, name, bias=True: F.linear(v, sd[name + ".weight"], sd.get(name + ".bias") if bias else None)
    rms = lambda v, w, eps: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w
    half = Dh // 2
    # full-width tables, slot d -> axis by the interleave rule
    inv = 1.0 / (cfg.theta ** (torch.arange(0, Dh, 2).float() / Dh))
    fr = [pos[:, a:a + 1] * inv[None] for a in range(3)]
    f = fr[0].clone()
    for d in range(half):
        if d % 3 == 1 and d < cfg.mrope_section[1] * 3:
            f[:, d] = fr[1][:, d]
        elif d % 3 == 2 and d < cfg.mrope_section[2] * 3:
            f[:, d] = fr[2][:, d]
    emb = torch.cat((f, f), -1).double()
    cosf, sinf = emb.cos().float()[None, :, None], emb.sin().float()[None, :, None]
    rot = lambda v: torch.cat((-v[..., half:], v[..., :half]), -1)
    c0, s0 = mrope_table(pos, Dh, cfg.mrope_section, cfg.theta)
    assert (c0 - cosf[0, :, 0, :half]).abs().max() < 1e-4 and (s0 - sinf[0, :, 0, :half]).abs().max() < 1e-4
    far = torch.tensor([[65536.0, 65536.0, 65536.0]])                      # large positions: the angle is reduced in float64
    cf, _ = mrope_table(far, Dh, cfg.mrope_section, cfg.theta)
    inv32 = torch.exp(-(torch.arange(half).float() / half) * math.log(cfg.theta))
    assert (cf[0] - (far[0, 0] * inv32).double().cos().float()).abs().max() < 1e-6
    # conditioning
    hh = D // 2
    fq = torch.exp(-torch.arange(hh).float() * math.log(1e4) / (hh - 1))
    a = t[:, None] * 1e4 * fq[None]
    te = torch.cat((a.sin(), a.cos()), -1)
    assert (te - scalar_embedding(t, D)).abs().max() < 1e-3
    c = lin(F.silu(lin(te, "t_embedding.mlp_in")), "t_embedding.mlp_out")
    ada = F.silu(lin(c, "adaln_proj"))[:, None]
    im, tm = (ind == IND_IMAGE)[..., None].float(), (ind == IND_TEXT)[..., None].float()
    h = lin(x * im, "input_proj") * im + lin(rms(llm * tm, sd["llm_cond_norm.weight"], 1e-6), "llm_cond_proj") * tm
    h = h + sd["embed_image_indicator.weight"][(ind == IND_IMAGE).long()]
    for i in range(cfg.depth):
        p = f"layers.{i}."
        mod = lin(ada, p + "adaln_modulation")
        sc1, g1, sc2, g2 = 1 + mod[..., :D], torch.tanh(mod[..., D:2 * D]), 1 + mod[..., 2 * D:3 * D], torch.tanh(mod[..., 3 * D:])
        qkv = lin(rms(h, sd[p + "attention_norm1.weight"], 1e-5) * sc1, p + "attention.qkv", False).reshape(1, L, 3, H, Dh)
        q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
        q, k = rms(q, sd[p + "attention.norm_q.weight"], 1e-5), rms(k, sd[p + "attention.norm_k.weight"], 1e-5)
        q, k = q * cosf + rot(q) * sinf, k * cosf + rot(k) * sinf
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(1, L, D)
        h = h + g1 * rms(lin(o, p + "attention.o", False), sd[p + "attention_norm2.weight"], 1e-5)
        u = rms(h, sd[p + "ffn_norm1.weight"], 1e-5) * sc2
        ff = lin(F.silu(lin(u, p + "feed_forward.w1", False)) * lin(u, p + "feed_forward.w3", False), p + "feed_forward.w2", False)
        h = h + g2 * rms(ff, sd[p + "ffn_norm2.weight"], 1e-5)
    fs = 1 + lin(F.silu(ada), "final_layer.adaln_modulation")
    want = lin(F.layer_norm(h, (D,), eps=1e-6) * fs, "final_layer.linear")
    assert (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_hunyuan15_matches_plain_torch_statement():
    """HunyuanVideo-1.5: equals a plain-torch statement with [video, text] row order, rotate-half rotary on the video rows
    only and separate q / k / v projections; checkpoint key names are the published ones."""
    import torch.nn.functional as F
    from mojodiffusion_b200.models.hunyuan15 import Hunyuan15DiT, tiny_hunyuan15_config
    from mojodiffusion_b200.models.layers import timestep_embedding
    torch.manual_seed(1)
    cfg = tiny_hunyuan15_config()
    m = Hunyuan15DiT(cfg, torch.float32).init_weights(5)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    for k in ("img_in.proj.weight", "time_in.mlp.0.weight", "double_blocks.1.img_attn_q_norm.weight", "double_blocks.0.txt_mlp.fc2.bias",
              "double_blocks.0.img_mod.linear.weight", "final_layer.adaLN_modulation.1.bias", "final_layer.linear.weight"):
        assert k in sd, k
    B, Fr, Hh, Ww, St = 1, 2, 3, 4, 5
    D, H, Dh = cfg.hidden, cfg.heads, cfg.head_dim
    z, txt, t = torch.randn(B, cfg.in_channels, Fr, Hh, Ww), torch.randn(B, St, D), torch.tensor([0.3])
    got = m(z, txt, t)
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd[n + ".bias"])
    rms = lambda v, w: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * w
    img = F.conv3d(z, sd["img_in.proj.weight"], sd["img_in.proj.bias"]).flatten(2).transpose(1, 2)
    vec = lin(F.silu(lin(timestep_embedding(t, 256), "time_in.mlp.0")), "time_in.mlp.2")
    vs = F.silu(vec)
    half = Dh // 2
    pos = torch.stack(torch.meshgrid(torch.arange(Fr), torch.arange(Hh), torch.arange(Ww), indexing="ij"), -1).reshape(-1, 3).float()
    ang = []
    for a, d in enumerate(cfg.axes_dim):
        inv = cfg.theta ** (-torch.arange(0, d, 2).float() / d)
        ang.append(pos[:, a:a + 1] * inv[None])
    ang = torch.cat(ang, -1)                                      # [S_img, Dh/2]
    cosf, sinf = torch.cat((ang.cos(), ang.cos()), -1)[None, :, None], torch.cat((ang.sin(), ang.sin()), -1)[None, :, None]
    rot = lambda v: torch.cat((-v[..., half:], v[..., :half]), -1)
    mod = lambda v, sc, sh: F.layer_norm(v, (D,), eps=cfg.eps) * (1 + sc[:, None]) + sh[:, None]
    S_img = img.shape[1]
    for i in range(cfg.depth):
        p = f"double_blocks.{i}."
        im = lin(vs, p + "img_mod.linear").chunk(6, -1)
        tm = lin(vs, p + "txt_mod.linear").chunk(6, -1)
        def qkv(x, s, rope):
            q, k, v = (lin(x, p + f"{s}_attn_{c}").reshape(B, -1, H, Dh) for c in "qkv")
            q, k = rms(q, sd[p + f"{s}_attn_q_norm.weight"]), rms(k, sd[p + f"{s}_attn_k_norm.weight"])
            if rope:
                q, k = q * cosf + rot(q) * sinf, k * cosf + rot(k) * sinf
            return q, k, v
        iq, ik, iv = qkv(mod(img, im[1], im[0]), "img", True)
        tq, tk, tv = qkv(mod(txt, tm[1], tm[0]), "txt", False)
        q, k, v = torch.cat((iq, tq), 1), torch.cat((ik, tk), 1), torch.cat((iv, tv), 1)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(B, -1, D)
        img = img + im[2][:, None] * lin(a[:, :S_img], p + "img_attn_proj")
        txt = txt + tm[2][:, None] * lin(a[:, S_img:], p + "txt_attn_proj")
        img = img + im[5][:, None] * lin(F.gelu(lin(mod(img, im[4], im[3]), p + "img_mlp.fc1"), approximate="tanh"), p + "img_mlp.fc2")
        txt = txt + tm[5][:, None] * lin(F.gelu(lin(mod(txt, tm[4], tm[3]), p + "txt_mlp.fc1"), approximate="tanh"), p + "txt_mlp.fc2")
    fm = lin(vs, "final_layer.adaLN_modulation.1")
    out = lin(mod(img, fm[:, D:], fm[:, :D]), "final_layer.linear")
    want = out.reshape(B, Fr, Hh, Ww, cfg.out_channels).permute(0, 4, 1, 2, 3)
    assert got.shape == want.shape and (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_kandinsky5_matches_plain_torch_statement():
    """Kandinsky-5: equals a plain-torch statement (pair-rotation rotary, separate q / k / v, per-head softmax cross
    attention, exact GELU) and carries the published checkpoint key names."""
    import torch.nn.functional as F
    from mojodiffusion_b200.models.kandinsky5 import Kandinsky5DiT, tiny_kandinsky5_config
    from mojodiffusion_b200.models.layers import timestep_embedding
    torch.manual_seed(2)
    cfg = tiny_kandinsky5_config()
    m = Kandinsky5DiT(cfg, torch.float32).init_weights(7)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    for k in ("text_embeddings.norm.bias", "pooled_text_embeddings.in_layer.weight", "time_embeddings.out_layer.bias",
              "visual_embeddings.in_layer.weight", "text_transformer_blocks.0.text_modulation.out_layer.weight",
              "visual_transformer_blocks.1.cross_attention.key_norm.weight", "visual_transformer_blocks.0.feed_forward.in_layer.weight",
              "out_layer.modulation.out_layer.bias", "out_layer.out_layer.weight"):
        assert k in sd, k
    assert "visual_transformer_blocks.0.feed_forward.in_layer.bias" not in sd
    B, Fr, Hh, Ww, T = 1, 2, 4, 6, 5
    D, H, Dh = cfg.model_dim, cfg.heads, cfg.head_dim
    z, text, pooled, t = torch.randn(B, cfg.in_visual_dim, Fr, Hh, Ww), torch.randn(B, T, cfg.in_text_dim), torch.randn(B, cfg.in_text_dim2), torch.tensor([417.0])
    got = m(z, text, pooled, t)
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, w: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * w
    ln = lambda v, n: F.layer_norm(v, (v.shape[-1],), sd[n + ".weight"], sd[n + ".bias"], cfg.eps)
    mod = lambda v, sc, sh: F.layer_norm(v, (D,), eps=cfg.eps) * (1 + sc[:, None]) + sh[:, None]

    def table(pos, axes):
        parts = [pos[:, a:a + 1] * torch.exp(-torch.log(torch.tensor(cfg.max_period)) * torch.arange(d // 2).float() / (d // 2))[None]
                 for a, d in enumerate(axes)]
        return torch.cat(parts, -1)

    def rope(v, ang):                                   # v [B, S, H, Dh], pairs (2i, 2i + 1)
        c, s = ang.cos()[None, :, None], ang.sin()[None, :, None]
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)

    def attn(p, xq, xkv, ang):
        q = rms(lin(xq, p + "to_query").reshape(B, -1, H, Dh), sd[p + "query_norm.weight"])
        k = rms(lin(xkv, p + "to_key").reshape(B, -1, H, Dh), sd[p + "key_norm.weight"])
        v = lin(xkv, p + "to_value").reshape(B, -1, H, Dh)
        if ang is not None:
            q, k = rope(q, ang), rope(k, ang)
        w_ = torch.softmax(torch.einsum("bqhd,bkhd->bhqk", q, k) / Dh ** 0.5, -1)
        return lin(torch.einsum("bhqk,bkhd->bqhd", w_, v).reshape(B, -1, D), p + "out_layer")

    te = lin(F.silu(lin(timestep_embedding(t, D, cfg.max_period, time_factor=1.0), "time_embeddings.in_layer")), "time_embeddings.out_layer")
    te = te + ln(lin(pooled, "pooled_text_embeddings.in_layer"), "pooled_text_embeddings.norm")
    txt = ln(lin(text, "text_embeddings.in_layer"), "text_embeddings.norm")
    tang = table(torch.arange(T).float()[:, None], [Dh])
    for i in range(cfg.num_text_blocks):
        p = f"text_transformer_blocks.{i}."
        c6 = lin(F.silu(te), p + "text_modulation.out_layer").chunk(6, -1)
        txt = txt + c6[2][:, None] * attn(p + "self_attention.", mod(txt, c6[1], c6[0]), mod(txt, c6[1], c6[0]), tang)
        txt = txt + c6[5][:, None] * lin(F.gelu(lin(mod(txt, c6[4], c6[3]), p + "feed_forward.in_layer")), p + "feed_forward.out_layer")
    f, h, w = Fr, Hh // 2, Ww // 2
    tok = z.reshape(B, -1, f, 1, h, 2, w, 2).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, f * h * w, -1)
    x = lin(tok, "visual_embeddings.in_layer")
    ids = torch.stack(torch.meshgrid(torch.arange(f), torch.arange(h), torch.arange(w), indexing="ij"), -1).reshape(-1, 3).float()
    vang = table(ids, cfg.axes_dim)
    for i in range(cfg.num_visual_blocks):
        p = f"visual_transformer_blocks.{i}."
        c9 = lin(F.silu(te), p + "visual_modulation.out_layer").chunk(9, -1)
        u = mod(x, c9[1], c9[0])
        x = x + c9[2][:, None] * attn(p + "self_attention.", u, u, vang)
        x = x + c9[5][:, None] * attn(p + "cross_attention.", mod(x, c9[4], c9[3]), txt, None)
        x = x + c9[8][:, None] * lin(F.gelu(lin(mod(x, c9[7], c9[6]), p + "feed_forward.in_layer")), p + "feed_forward.out_layer")
    om = lin(F.silu(te), "out_layer.modulation.out_layer")
    out = lin(mod(x, om[:, D:], om[:, :D]), "out_layer.out_layer")
    want = out.reshape(B, f, h, w, cfg.out_visual_dim, 1, 2, 2).permute(0, 4, 1, 5, 2, 6, 3, 7).reshape(B, cfg.out_visual_dim, Fr, Hh, Ww)
    assert got.shape == want.shape and (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_cosmos_predict25_matches_plain_torch_statement():
    """Cosmos-Predict2.5: equals a plain-torch statement (adaLN-LoRA modulation, NTK per-axis rotary bases, channel-slowest
    un-patchify, mask channels) and carries the published checkpoint key names; per-frame timesteps are accepted."""
    import torch.nn.functional as F
    from mojodiffusion_b200.models.cosmos import CosmosDiT, tiny_cosmos_config
    from mojodiffusion_b200.models.layers import timestep_embedding
    torch.manual_seed(3)
    cfg = tiny_cosmos_config()
    m = CosmosDiT(cfg, torch.float32).init_weights(9)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    for k in ("x_embedder.proj.1.weight", "crossattn_proj.0.bias", "t_embedder.1.linear_2.weight", "t_embedding_norm.weight",
              "blocks.0.adaln_modulation_self_attn.1.weight", "blocks.1.adaln_modulation_mlp.2.weight", "blocks.0.self_attn.q_norm.weight",
              "blocks.0.cross_attn.k_proj.weight", "blocks.1.mlp.layer2.weight", "final_layer.adaln_modulation.2.weight", "final_layer.linear.weight"):
        assert k in sd, k
    assert not any(k.endswith(".bias") and "crossattn_proj" not in k for k in sd)
    B, T, Hh, Ww, St = 1, 2, 4, 6, 5
    D, H, Dh = cfg.model_channels, cfg.heads, cfg.head_dim
    z, text, t = torch.randn(B, cfg.in_channels, T, Hh, Ww), torch.randn(B, St, cfg.text_in_dim), torch.tensor([[0.3, 0.7]])
    mask = (torch.rand(B, 1, T, Hh, Ww) > 0.5).float()
    got = m(z, text, t, cond_mask=mask)
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, w: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * w
    tp, hp, wp = T, Hh // 2, Ww // 2
    x_in = torch.cat((z, mask, torch.zeros(B, 1, T, Hh, Ww)), 1)
    tok = x_in.reshape(B, -1, tp, 1, hp, 2, wp, 2).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, tp, hp * wp, -1)
    x = lin(tok, "x_embedder.proj.1")                                            # [B, tp, hw, D]
    txt = lin(text, "crossattn_proj.0")
    sample = timestep_embedding(t.reshape(-1), D, 10000.0, time_factor=1.0).reshape(B, tp, 1, D)
    lora = lin(F.silu(lin(sample, "t_embedder.1.linear_1")), "t_embedder.1.linear_2")
    emb = rms(sample, sd["t_embedding_norm.weight"])
    dims = (Dh - 2 * (Dh // 6 * 2), Dh // 6 * 2, Dh // 6 * 2)
    ids = torch.stack(torch.meshgrid(torch.arange(tp), torch.arange(hp), torch.arange(wp), indexing="ij"), -1).reshape(-1, 3).float()
    ang = torch.cat([ids[:, a:a + 1] * ((10000.0 * r ** (d / (d - 2))) ** (-torch.arange(0, d, 2).float() / d))[None]
                     for a, (d, r) in enumerate(zip(dims, (1.0, 3.0, 3.0)))], -1)
    cosf, sinf = torch.cat((ang.cos(), ang.cos()), -1)[None, :, None], torch.cat((ang.sin(), ang.sin()), -1)[None, :, None]
    rot = lambda v: torch.cat((-v[..., Dh // 2:], v[..., :Dh // 2]), -1)

    def attn(p, xq, xkv, rope):
        q = rms(lin(xq, p + "q_proj").reshape(B, -1, H, Dh), sd[p + "q_norm.weight"])
        k = rms(lin(xkv, p + "k_proj").reshape(B, -1, H, Dh), sd[p + "k_norm.weight"])
        v = lin(xkv, p + "v_proj").reshape(B, -1, H, Dh)
        if rope:
            q, k = q * cosf + rot(q) * sinf, k * cosf + rot(k) * sinf
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
        return lin(o.reshape(B, -1, D), p + "output_proj")

    for i in range(cfg.depth):
        p = f"blocks.{i}."
        for sub in ("self_attn", "cross_attn", "mlp"):
            sh, sc, g = (lin(lin(F.silu(emb), p + f"adaln_modulation_{sub}.1"), p + f"adaln_modulation_{sub}.2") + lora).chunk(3, -1)
            u = F.layer_norm(x, (D,), eps=cfg.eps) * (1 + sc) + sh
            if sub == "self_attn":
                y = attn(p + "self_attn.", u.reshape(B, -1, D), u.reshape(B, -1, D), True)
            elif sub == "cross_attn":
                y = attn(p + "cross_attn.", u.reshape(B, -1, D), txt, False)
            else:
                y = lin(F.gelu(lin(u, p + "mlp.layer1")), p + "mlp.layer2").reshape(B, -1, D)
            x = x + g * y.reshape(B, tp, hp * wp, D)
    fm = lin(lin(F.silu(emb), "final_layer.adaln_modulation.1"), "final_layer.adaln_modulation.2") + lora[..., :2 * D]
    out = lin(F.layer_norm(x, (D,), eps=cfg.eps) * (1 + fm[..., D:]) + fm[..., :D], "final_layer.linear")
    want = out.reshape(B, tp, hp, wp, 2, 2, 1, cfg.out_channels).permute(0, 7, 1, 6, 2, 4, 3, 5).reshape(B, cfg.out_channels, T, Hh, Ww)
    assert got.shape == want.shape and (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_nucleus_moe_dit_matches_plain_torch_statement():
    """Nucleus-Image: expert-choice routing equals a loop statement (greedy top-C per sample and expert, ties to the lower
    token, per-token renormalisation times the route scale) and the whole model equals a plain-torch forward."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models.layers import timestep_embedding
    from mojodiffusion_b200.models.nucleus import NucleusDiT, _signed, tiny_nucleus_config
    from mojodiffusion_b200.ops import moe
    torch.manual_seed(4)
    # routing against loops, with a deliberate tie
    aff = torch.softmax(torch.randn(2, 3, 7), 1)
    aff[0, 1, 2] = aff[0, 1, 5]
    idx, gate = moe.expert_choice_route(aff, 3, 2.5)
    B, E, S, C = 2, 3, 7, 3
    picks = {}
    for b in range(B):
        for e in range(E):
            taken = []
            for _ in range(C):
                best = max((s for s in range(S) if s not in taken), key=lambda s: (float(aff[b, e, s]), -s))
                taken.append(best)
            picks[(b, e)] = taken
    tsum = torch.zeros(B * S)
    for (b, e), tk in picks.items():
        for s in tk:
            tsum[b * S + s] += aff[b, e, s]
    for e in range(E):
        for b in range(B):
            for c, s in enumerate(picks[(b, e)]):
                assert int(idx[e, b * C + c]) == b * S + s
                assert abs(float(gate[e, b * C + c]) - float(aff[b, e, s] / (tsum[b * S + s] + 1e-12) * 2.5)) < 1e-6
    assert [float(v) for v in _signed(5)] == [-3, -2, -1, 0, 1] and [float(v) for v in _signed(4)] == [-2, -1, 0, 1]

    cfg = tiny_nucleus_config()
    m = NucleusDiT(cfg, torch.float32).init_weights(11)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    f, h, w, St = 1, 4, 6, 5
    D, H, KV, Dh = cfg.hidden, cfg.heads, cfg.kv_heads, cfg.head_dim
    x_in, text, t = torch.randn(2, f * h * w, cfg.in_channels), torch.randn(2, St, cfg.joint_dim), torch.tensor([0.3, 0.8])
    got = m(x_in, text, t, (f, h, w))
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, wt: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * wt
    ln = lambda v: F.layer_norm(v, (D,), eps=cfg.eps)

    def angles(pos):
        return torch.cat([pos[:, a:a + 1] / (cfg.theta ** (torch.arange(d // 2).float() / (d // 2)))[None]
                          for a, d in enumerate(cfg.axes_dim)], -1)
    ipos = torch.stack(torch.meshgrid(torch.arange(f).float(), _signed(h), _signed(w), indexing="ij"), -1).reshape(-1, 3)
    tpos = (max(h // 2, w // 2) + torch.arange(St)).float()[:, None].expand(St, 3)
    iang, tang = angles(ipos), angles(tpos)

    def rope(v, ang):
        c, s = ang.cos()[None, :, None], ang.sin()[None, :, None]
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)

    def swiglu_ffn(v, p0, p2):
        gu = F.linear(v, sd[p0])
        inner = gu.shape[-1] // 2
        return F.linear(F.silu(gu[..., inner:]) * gu[..., :inner], sd[p2])

    x = lin(x_in, "img_in")
    enc = rms(text, sd["txt_norm.weight"])
    temb = rms(lin(F.silu(lin(timestep_embedding(t, D), "time_text_embed.timestep_embedder.linear_1")),
                   "time_text_embed.timestep_embedder.linear_2"), sd["time_text_embed.norm.weight"])
    for i in range(cfg.depth):
        p = f"transformer_blocks.{i}."
        sc1, g1, sc2, g2 = lin(F.silu(temb), p + "img_mod.1").chunk(4, -1)
        g1, g2 = torch.tanh(g1.clamp(-2, 2))[:, None], torch.tanh(g2.clamp(-2, 2))[:, None]
        ctx = lin(enc, p + "encoder_proj")
        u = ln(x) * (1 + sc1[:, None])
        q = rope(rms(lin(u, p + "attn.to_q").unflatten(-1, (H, Dh)), sd[p + "attn.norm_q.weight"]), iang)
        k = torch.cat((rope(rms(lin(u, p + "attn.to_k").unflatten(-1, (KV, Dh)), sd[p + "attn.norm_k.weight"]), iang),
                       rope(rms(lin(ctx, p + "attn.add_k_proj").unflatten(-1, (KV, Dh)), sd[p + "attn.norm_added_k.weight"]), tang)), 1)
        v = torch.cat((lin(u, p + "attn.to_v"), lin(ctx, p + "attn.add_v_proj")), 1).unflatten(-1, (KV, Dh))
        k, v = k.repeat_interleave(H // KV, 2), v.repeat_interleave(H // KV, 2)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(-2)
        x = x + g1 * lin(o, p + "attn.to_out.0")
        un = ln(x)
        u = un * (1 + sc2[:, None])
        if i < cfg.dense_layers:
            y = swiglu_ffn(u, p + "img_mlp.net.0.proj.weight", p + "img_mlp.net.2.weight")
        else:
            Bn, S = u.shape[:2]
            C = max(1, math.ceil(cfg.capacity_factor(i) * S / cfg.num_experts))
            scores = torch.softmax(F.linear(torch.cat((temb[:, None].expand(Bn, S, D), un), -1), sd[p + "img_mlp.gate.weight"]).float(), -1)
            scores = scores.to(torch.bfloat16).float()
            routed = torch.zeros(Bn * S, D)
            flat = u.reshape(Bn * S, D)
            top = torch.sort(scores.transpose(1, 2), dim=2, descending=True, stable=True).indices[:, :, :C]     # [B, E, C]
            tsum = torch.zeros(Bn * S)
            for b in range(Bn):
                for e in range(cfg.num_experts):
                    for s in top[b, e]:
                        tsum[b * S + int(s)] += scores[b, int(s), e]
            for b in range(Bn):
                for e in range(cfg.num_experts):
                    for s in top[b, e]:
                        tk = b * S + int(s)
                        gu = flat[tk] @ sd[p + "img_mlp.experts.gate_up_proj"][e]
                        inner = gu.shape[-1] // 2
                        eo = (F.silu(gu[:inner]) * gu[inner:]) @ sd[p + "img_mlp.experts.down_proj"][e]
                        routed[tk] += eo * (scores[b, int(s), e] / (tsum[tk] + 1e-12) * cfg.route_scale)
            y = swiglu_ffn(u, p + "img_mlp.shared_expert.net.0.proj.weight", p + "img_mlp.shared_expert.net.2.weight") + routed.reshape(Bn, S, D)
        x = x + g2 * y
    sc, sh = lin(F.silu(temb), "norm_out.linear").chunk(2, -1)
    want = F.linear(ln(x) * (1 + sc[:, None]) + sh[:, None], sd["proj_out.weight"])
    assert got.shape == want.shape and (got - want).abs().max() < 3e-4 * max(1.0, float(want.abs().max()))


def test_acestep_audio_dit_matches_plain_torch_statement():
    """ACE-Step: equals a plain-torch statement built on conv1d / conv_transpose1d, rotate-half rotary, grouped-query
    attention and a +-window band mask on the even layers (sequence longer than the window), odd length padded and cropped."""
    import torch.nn.functional as F
    from mojodiffusion_b200.models.acestep import AceStepDiT, tiny_acestep_config
    from mojodiffusion_b200.models.layers import timestep_embedding
    torch.manual_seed(5)
    cfg = tiny_acestep_config()
    m = AceStepDiT(cfg, torch.float32).init_weights(13)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() == 1 or "scale_shift_table" in n:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    B, T, L = 2, 21, 5
    D, H, KV, Dh = cfg.hidden, cfg.heads, cfg.kv_heads, cfg.head_dim
    x_t, ctx, cond = torch.randn(B, T, cfg.acoustic_dim), torch.randn(B, T, cfg.in_channels - cfg.acoustic_dim), torch.randn(B, L, D)
    t, r = torch.tensor([0.7, 0.2]), torch.tensor([0.5, 0.1])
    got = m(x_t, ctx, cond, t, r)
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, wt: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * wt

    def temb(tv, p):
        e = lin(F.silu(lin(timestep_embedding(tv, 256), p + ".linear_1")), p + ".linear_2")
        return e, lin(F.silu(e), p + ".time_proj").reshape(B, 6, D)
    e1, p1 = temb(t, "decoder.time_embed")
    e2, p2 = temb(t - r, "decoder.time_embed_r")
    te, tp = e1 + e2, p1 + p2
    xin = F.pad(torch.cat((ctx, x_t), -1), (0, 0, 0, 1))
    x = F.conv1d(xin.transpose(1, 2), sd["decoder.proj_in.1.weight"], sd["decoder.proj_in.1.bias"], stride=2).transpose(1, 2)
    S = x.shape[1]
    assert S == 11 and S > cfg.sliding_window
    enc = lin(cond, "decoder.condition_embedder")
    ang = torch.arange(S).float()[:, None] / (cfg.theta ** (torch.arange(0, Dh, 2).float() / Dh))[None]
    cosf, sinf = torch.cat((ang.cos(), ang.cos()), -1)[None, :, None], torch.cat((ang.sin(), ang.sin()), -1)[None, :, None]
    rot = lambda v: torch.cat((-v[..., Dh // 2:], v[..., :Dh // 2]), -1)
    idx = torch.arange(S)
    band = (idx[:, None] - idx[None]).abs() <= cfg.sliding_window

    def attn(p, xq, xkv, rope, mask):
        q = rms(lin(xq, p + ".q_proj").unflatten(-1, (H, Dh)), sd[p + ".q_norm.weight"])
        k = rms(lin(xkv, p + ".k_proj").unflatten(-1, (KV, Dh)), sd[p + ".k_norm.weight"])
        v = lin(xkv, p + ".v_proj").unflatten(-1, (KV, Dh))
        if rope:
            q, k = q * cosf + rot(q) * sinf, k * cosf + rot(k) * sinf
        k, v = k.repeat_interleave(H // KV, 2), v.repeat_interleave(H // KV, 2)
        s = torch.einsum("bqhd,bkhd->bhqk", q, k) / Dh ** 0.5
        if mask is not None:
            s = s.masked_fill(~mask, float("-inf"))
        return lin(torch.einsum("bhqk,bkhd->bqhd", torch.softmax(s, -1), v).flatten(-2), p + ".o_proj")

    for i in range(cfg.depth):
        p = f"decoder.layers.{i}."
        mod = sd[p + "scale_shift_table"] + tp
        sh1, sc1, g1, sh2, sc2, g2 = (mod[:, j:j + 1] for j in range(6))
        u = rms(x, sd[p + "self_attn_norm.weight"]) * (1 + sc1) + sh1
        x = x + g1 * attn(p + "self_attn", u, u, True, band if i % 2 == 0 else None)
        x = x + attn(p + "cross_attn", rms(x, sd[p + "cross_attn_norm.weight"]), enc, False, None)
        u = rms(x, sd[p + "mlp_norm.weight"]) * (1 + sc2) + sh2
        x = x + g2 * lin(F.silu(lin(u, p + "mlp.gate_proj")) * lin(u, p + "mlp.up_proj"), p + "mlp.down_proj")
    fm = sd["decoder.scale_shift_table"] + te[:, None]
    xo = rms(x, sd["decoder.norm_out.weight"]) * (1 + fm[:, 1:2]) + fm[:, 0:1]
    want = F.conv_transpose1d(xo.transpose(1, 2), sd["decoder.proj_out.1.weight"], sd["decoder.proj_out.1.bias"], stride=2).transpose(1, 2)[:, :T]
    assert got.shape == want.shape == (B, T, cfg.acoustic_dim) and (got - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_hidream_o1_spine_heads_mask_and_positions():
    """HiDream-O1: the text prefix is causal and the image rows see every key, the timestep embedding replaces the reserved
    token's embedding, positions follow the text-count / fix-point rule, and the forward equals a plain-torch statement of
    one layer stack built from the checkpoint-named tensors."""
    import torch.nn.functional as F
    from mojodiffusion_b200.models.hidream_o1 import HiDreamO1, build_mrope_positions, prefix_causal_mask, tiny_hidream_o1_config
    from mojodiffusion_b200.models.ideogram4 import mrope_table
    from mojodiffusion_b200.models.layers import timestep_embedding
    torch.manual_seed(6)
    cfg = tiny_hidream_o1_config()
    c = cfg.spine
    m = HiDreamO1(cfg, torch.float32).init_weights(17)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    for k in ("model.language_model.embed_tokens.weight", "model.language_model.layers.1.self_attn.k_norm.weight", "model.language_model.norm.weight",
              "model.x_embedder.proj1.weight", "model.x_embedder.proj2.bias", "model.t_embedder1.mlp.2.weight", "model.final_layer2.linear.bias"):
        assert k in sd, k
    assert "model.x_embedder.proj1.bias" not in sd
    ids = [1, 2, cfg.tms_token_id, 3, cfg.vision_start_token_id]
    L, ph, pw = 6, 2, 3
    pos = build_mrope_positions(ids + [cfg.image_token_id] * L, cfg.image_token_id, ph, pw, 10)
    assert pos[:4].tolist() == [[i] * 3 for i in range(4)] and pos[4].tolist() == [10, 10, 10] and pos[9].tolist() == [10, 11, 12]
    assert build_mrope_positions([1, 2, 3], cfg.image_token_id, 1, 1, 5).tolist() == [[0] * 3, [1] * 3, [2] * 3]
    mk = prefix_causal_mask(4, 2)[0, 0]
    assert mk.tolist() == [[0, -1e4, -1e4, -1e4], [0, 0, -1e4, -1e4], [0, 0, 0, 0], [0, 0, 0, 0]]
    assert prefix_causal_mask(3, 0, torch.tensor([1, 0, 1]))[0, 0, :, 1].tolist() == [-1e4] * 3
    patches = torch.randn(1, L, cfg.patch_dim)
    S, ar = len(ids) + L, len(ids)
    out = m(ids, patches, pos, ar, 0.4)
    # causality of the prefix: changing the last text token leaves earlier text rows alone but moves the image rows
    ids2 = list(ids)
    ids2[-1] = 7
    out2 = m(ids2, patches, pos, ar, 0.4)
    assert torch.allclose(out[:, :ar - 1], out2[:, :ar - 1], atol=1e-6) and (out[:, ar:] - out2[:, ar:]).abs().max() > 1e-5
    # the timestep reaches the output only through the reserved token's row and what attends to it
    out3 = m(ids, patches, pos, ar, 0.9)
    assert torch.allclose(out[:, :2], out3[:, :2], atol=1e-6) and (out[:, 2] - out3[:, 2]).abs().max() > 1e-6
    # plain-torch statement
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, w: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + c.rms_norm_eps) * w
    H, KV, Dh = c.num_attention_heads, c.num_key_value_heads, c.head_dim
    x = sd["model.language_model.embed_tokens.weight"][torch.tensor(ids)][None].clone()
    x[0, 2] = lin(F.silu(lin(timestep_embedding(torch.tensor([0.4]), cfg.timestep_freq_dim), "model.t_embedder1.mlp.0")), "model.t_embedder1.mlp.2")[0]
    x = torch.cat((x, lin(lin(patches, "model.x_embedder.proj1"), "model.x_embedder.proj2")), 1)
    cs, sn = mrope_table(pos, Dh, cfg.mrope_section, c.rope_theta)
    cosf, sinf = torch.cat((cs, cs), -1)[None, :, None], torch.cat((sn, sn), -1)[None, :, None]
    rot = lambda v: torch.cat((-v[..., Dh // 2:], v[..., :Dh // 2]), -1)
    i = torch.arange(S)
    allow = (i[None] <= i[:, None]) | (i[:, None] >= ar)
    for li in range(c.num_hidden_layers):
        p = f"model.language_model.layers.{li}."
        hN = rms(x, sd[p + "input_layernorm.weight"])
        q = rms(lin(hN, p + "self_attn.q_proj").unflatten(-1, (H, Dh)), sd[p + "self_attn.q_norm.weight"])
        k = rms(lin(hN, p + "self_attn.k_proj").unflatten(-1, (KV, Dh)), sd[p + "self_attn.k_norm.weight"])
        v = lin(hN, p + "self_attn.v_proj").unflatten(-1, (KV, Dh))
        q, k = q * cosf + rot(q) * sinf, k * cosf + rot(k) * sinf
        k, v = k.repeat_interleave(H // KV, 2), v.repeat_interleave(H // KV, 2)
        sc = torch.einsum("bqhd,bkhd->bhqk", q, k) / Dh ** 0.5 + torch.where(allow, 0.0, -1e4)
        x = x + lin(torch.einsum("bhqk,bkhd->bqhd", torch.softmax(sc, -1), v).flatten(-2), p + "self_attn.o_proj")
        hN = rms(x, sd[p + "post_attention_layernorm.weight"])
        x = x + lin(F.silu(lin(hN, p + "mlp.gate_proj")) * lin(hN, p + "mlp.up_proj"), p + "mlp.down_proj")
    want = lin(rms(x, sd["model.language_model.norm.weight"]), "model.final_layer2.linear")
    assert (out - want).abs().max() < 2e-4 * max(1.0, float(want.abs().max()))


def test_krea2_single_stream_dit_matches_plain_torch_statement():
    """Krea-2: three-axis rotary table against the complex-rotation statement (float64), patchify round trip, and the
    whole model (text fusion over layers then tokens, shared modulation vector + per-block offsets, grouped-query gated
    attention, SwiGLU, last layer on the time vector) against a plain-torch forward written from the state dict."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models import krea2 as K
    torch.manual_seed(9)
    cfg = K.tiny_krea2_config()
    assert K.Krea2Config().rope_axes == (32, 48, 48) and K.swiglu_width(6144, 4) == 16384 and cfg.head_dim == 32

    lat = torch.randn(2, cfg.channels, 6, 8)
    tok = K.patchify(lat, 2)
    assert tok.shape == (2, 12, cfg.channels * 4)
    assert torch.equal(tok[1, 1 * 4 + 2].reshape(cfg.channels, 2, 2), lat[1, :, 2:4, 4:6])
    assert torch.equal(K.unpatchify(tok, 3, 4, 2), lat)

    pos = K.krea2_positions(3, 3, 4)
    assert pos.shape == (15, 3) and float(pos[:3].abs().sum()) == 0 and pos[3 + 1 * 4 + 2].tolist() == [0.0, 1.0, 2.0]
    big = torch.tensor([[4000.0, 37.0, 63.0]])
    cos, sin = K.krea2_rope_table(big, (32, 48, 48), 1.0e3)
    want = torch.cat([big[:, a:a + 1].double() / (1.0e3 ** (torch.arange(0, d, 2).double() / d)) for a, d in enumerate((32, 48, 48))], -1)
    assert cos.shape == (1, 64) and (cos.double() - want.cos()).abs().max() < 1e-6 and (sin.double() - want.sin()).abs().max() < 1e-6

    m = K.Krea2DiT(cfg, torch.float32).init_weights(5)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(".scale") or n.endswith(".lin"):
                p.add_(torch.randn_like(p) * 0.2)
    sd = m.state_dict()
    assert {"first.weight", "tmlp.0.bias", "tmlp.2.weight", "tproj.1.weight", "txtfusion.projector.weight", "txtmlp.0.scale",
            "txtmlp.1.weight", "txtmlp.3.bias", "blocks.0.mod.lin", "blocks.1.attn.qknorm.knorm.scale", "blocks.0.attn.gate.weight",
            "blocks.0.mlp.down.weight", "txtfusion.layerwise_blocks.1.attn.wq.weight", "txtfusion.refiner_blocks.0.postnorm.scale",
            "last.norm.scale", "last.modulation.lin", "last.linear.bias"} <= set(sd)
    B, Lt, gh, gw = 2, 5, 3, 4
    img = torch.randn(B, gh * gw, cfg.patch_dim)
    context = torch.randn(B, Lt, cfg.txtlayers, cfg.txtdim)
    t = torch.tensor([0.25, 0.9])
    pos = K.krea2_positions(Lt, gh, gw)
    got = m(img, context, t, pos)
    assert got.shape == (B, gh * gw, cfg.patch_dim)

    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    norm = lambda v, n: F.rms_norm(v, (v.shape[-1],), weight=sd[n + ".scale"] + 1.0, eps=1e-5)
    gelu = lambda v: F.gelu(v, approximate="tanh")

    def attn(v, p, heads, kvheads, ang=None):
        b, s, d = v.shape
        dh = d // heads
        q = norm(lin(v, p + ".wq").reshape(b, s, heads, dh), p + ".qknorm.qnorm").transpose(1, 2)
        k = norm(lin(v, p + ".wk").reshape(b, s, kvheads, dh), p + ".qknorm.knorm").transpose(1, 2)
        vv = lin(v, p + ".wv").reshape(b, s, kvheads, dh).transpose(1, 2)
        if ang is not None:
            rot = torch.polar(torch.ones_like(ang), ang)[None, None]                  # [1, 1, S, dh / 2] complex
            q = torch.view_as_real(torch.view_as_complex(q.reshape(b, heads, s, dh // 2, 2).contiguous()) * rot).flatten(-2)
            k = torch.view_as_real(torch.view_as_complex(k.reshape(b, kvheads, s, dh // 2, 2).contiguous()) * rot).flatten(-2)
        o = F.scaled_dot_product_attention(q, k, vv, enable_gqa=kvheads != heads).transpose(1, 2).reshape(b, s, d)
        return lin(o * torch.sigmoid(lin(v, p + ".gate")), p + ".wo")

    swiglu = lambda v, p: lin(F.silu(lin(v, p + ".gate")) * lin(v, p + ".up"), p + ".down")

    def fusion_block(v, p):
        v = v + attn(norm(v, p + ".prenorm"), p + ".attn", cfg.txtheads, cfg.txtkvheads)
        return v + swiglu(norm(v, p + ".postnorm"), p + ".mlp")

    half = cfg.tdim // 2
    args = (t * 1000.0)[:, None] * torch.exp(-math.log(1.0e4) * torch.arange(half).float() / half)[None]
    tv = lin(gelu(lin(torch.cat((args.cos(), args.sin()), -1), "tmlp.0")), "tmlp.2")
    vec = lin(gelu(tv), "tproj.1")
    c = context.reshape(B * Lt, cfg.txtlayers, cfg.txtdim)
    for i in range(2):
        c = fusion_block(c, f"txtfusion.layerwise_blocks.{i}")
    c = F.linear(c.transpose(1, 2), sd["txtfusion.projector.weight"]).reshape(B, Lt, cfg.txtdim)
    for i in range(2):
        c = fusion_block(c, f"txtfusion.refiner_blocks.{i}")
    c = lin(gelu(lin(norm(c, "txtmlp.0"), "txtmlp.1")), "txtmlp.3")
    x = torch.cat((c, lin(img, "first")), 1)
    ang = torch.cat([pos[:, a:a + 1] / (cfg.theta ** (torch.arange(0, d, 2).float() / d))[None] for a, d in enumerate(cfg.rope_axes)], -1)
    for i in range(cfg.layers):
        p = f"blocks.{i}"
        s1, b1, g1, s2, b2, g2 = (vec + sd[p + ".mod.lin"])[:, None].chunk(6, -1)
        x = x + g1 * attn((1 + s1) * norm(x, p + ".prenorm") + b1, p + ".attn", cfg.heads, cfg.kvheads, ang)
        x = x + g2 * swiglu((1 + s2) * norm(x, p + ".postnorm") + b2, p + ".mlp")
    sc, sh = (tv[:, None] + sd["last.modulation.lin"][None]).chunk(2, 1)
    want = lin((1 + sc) * norm(x, "last.norm") + sh, "last.linear")[:, Lt:]
    assert F.cosine_similarity(got.flatten(), want.flatten(), 0) > 0.99999 and (got - want).abs().max() < 2e-4 * want.abs().max() + 1e-5

    # sampler: one step without guidance equals latent + (t1 - t0) * v; with guidance the two velocities combine as v_c + s (v_c - v_u)
    from mojodiffusion_b200.sampling.family_schedules import krea2_packed_seq_len, krea2_timesteps
    ctx1, ctx0 = context[:1], torch.randn(1, 3, cfg.txtlayers, cfg.txtdim)
    start = torch.randn(1, cfg.channels, 2 * gh, 2 * gw)
    ts = krea2_timesteps(krea2_packed_seq_len(16 * gh, 16 * gw), 1)
    out = K.krea2_sample(m, ctx1, ctx0, 16 * gh, 16 * gw, steps=1, cfg_scale=2.0, latent=start)
    tt = torch.tensor([ts[0]])
    vc = m(K.patchify(start), ctx1, tt, K.krea2_positions(Lt, gh, gw))
    vu = m(K.patchify(start), ctx0, tt, K.krea2_positions(3, gh, gw))
    assert torch.allclose(out, start + (ts[1] - ts[0]) * K.unpatchify(vc + 2.0 * (vc - vu), gh, gw), atol=1e-5)


def test_zimage_l2p_pixel_trunk_and_local_decoder_match_plain_torch_statement():
    """Z-Image L2P: pixel patch order, sigma table, the U-Net pixel head against NCHW torch convolutions, and the whole model
    against a plain-torch forward in the reference's caption-first token order with interleaved rotary pairs."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models import zimage_l2p as Z
    torch.manual_seed(12)
    full = Z.zimage_l2p_config()
    assert full.in_channels == 16 * 16 * 3 and full.hidden == 3840 and full.depth == 30 and not full.final_layer
    sig = Z.l2p_sigmas(30, 3.0)
    assert len(sig) == 31 and sig[0] == 1.0 and sig[-1] == 0.0 and abs(sig[15] - 3 * 0.5 / 2.0) < 1e-12
    px = torch.randn(1, 3, 8, 12)
    tok = Z.patchify_pixels(px, 4)
    assert tok.shape == (1, 6, 48) and torch.equal(tok[0, 1 * 3 + 2].reshape(4, 4, 3), px[0, :, 4:8, 8:12].permute(1, 2, 0))

    cfg = Z.tiny_zimage_l2p_config()
    m = Z.ZImageL2P(cfg, decoder_channels=(8, 16, 24, 32), dtype=torch.float32).init_weights(3)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() == 1 or n.endswith("pad_token"):
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    assert {"all_x_embedder.16-1.weight", "cap_embedder.1.bias", "t_embedder.mlp.0.weight", "noise_refiner.0.adaLN_modulation.0.weight",
            "layers.1.attention.norm_q.weight", "local_decoder.enc1.0.weight", "local_decoder.bottleneck.0.bias",
            "local_decoder.up4.1.weight", "local_decoder.dec1.0.bias", "local_decoder.out_conv.weight"} <= set(sd)
    assert not any(k.startswith("all_final_layer") for k in sd) and not any(k.startswith("context_refiner.0.adaLN") for k in sd)
    assert sum(1 for k in sd if k.startswith("local_decoder.")) == 28
    B, H, W, Sc = 2, 32, 48, 5
    pixels, cap, sigma = torch.randn(B, 3, H, W), torch.randn(B, Sc, cfg.cap_dim), torch.tensor([0.8, 0.35])
    got = m(pixels, cap, sigma)
    assert got.shape == (B, 3, H, W)

    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, n: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.norm_eps) * sd[n + ".weight"]
    gh, gw, D, Hh, Dh = H // 16, W // 16, cfg.hidden, cfg.heads, cfg.head_dim
    pos = torch.zeros(Sc + gh * gw, 3)
    pos[:Sc, 0] = torch.arange(1, Sc + 1).float()
    pos[Sc:, 0] = Sc + 1
    pos[Sc:, 1] = torch.arange(gh).float().repeat_interleave(gw)
    pos[Sc:, 2] = torch.arange(gw).float().repeat(gh)
    ang = torch.cat([pos[:, a:a + 1] / (cfg.theta ** (torch.arange(d // 2).float() / (d // 2)))[None] for a, d in enumerate(cfg.axes_dim)], -1)

    def rope(v, a):
        c, s = a.cos()[None, :, None], a.sin()[None, :, None]
        x0, x1 = v[..., 0::2], v[..., 1::2]
        return torch.stack((x0 * c - x1 * s, x0 * s + x1 * c), -1).flatten(-2)

    def block(v, p, a, c=None):
        b, s, _ = v.shape
        if c is not None:
            sm, gm, sf, gf = lin(c, p + ".adaLN_modulation.0")[:, None].chunk(4, -1)
        h = rms(v, p + ".attention_norm1") * ((1 + sm) if c is not None else 1.0)
        q = rope(rms(lin(h, p + ".attention.to_q").reshape(b, s, Hh, Dh), p + ".attention.norm_q"), a).transpose(1, 2)
        k = rope(rms(lin(h, p + ".attention.to_k").reshape(b, s, Hh, Dh), p + ".attention.norm_k"), a).transpose(1, 2)
        vv = lin(h, p + ".attention.to_v").reshape(b, s, Hh, Dh).transpose(1, 2)
        o = rms(lin(F.scaled_dot_product_attention(q, k, vv).transpose(1, 2).reshape(b, s, D), p + ".attention.to_out.0"), p + ".attention_norm2")
        v = v + (torch.tanh(gm) * o if c is not None else o)
        h = rms(v, p + ".ffn_norm1") * ((1 + sf) if c is not None else 1.0)
        o = rms(lin(F.silu(lin(h, p + ".feed_forward.w1")) * lin(h, p + ".feed_forward.w3"), p + ".feed_forward.w2"), p + ".ffn_norm2")
        return v + (torch.tanh(gf) * o if c is not None else o)

    half = 128
    targ = ((1.0 - sigma) * 1000.0)[:, None] * torch.exp(-math.log(10000.0) * torch.arange(half).float() / half)[None]
    c = lin(F.silu(lin(torch.cat((targ.cos(), targ.sin()), -1), "t_embedder.mlp.0")), "t_embedder.mlp.2")
    x = lin(Z.patchify_pixels(pixels, 16), "all_x_embedder.16-1")
    y = lin(rms(cap, "cap_embedder.0"), "cap_embedder.1")
    y = block(y, "context_refiner.0", ang[:Sc])
    x = block(x, "noise_refiner.0", ang[Sc:], c)
    j = torch.cat((y, x), 1)
    for i in range(cfg.depth):
        j = block(j, f"layers.{i}", ang, c)
    feat = j[:, Sc:].reshape(B, gh, gw, D).permute(0, 3, 1, 2)

    conv = lambda v, n, pad: F.conv2d(v, sd[n + ".weight"].permute(0, 3, 1, 2), sd[n + ".bias"], padding=pad)
    ld = "local_decoder."
    e1 = F.silu(conv(pixels, ld + "enc1.0", 1))
    e2 = F.silu(conv(F.max_pool2d(e1, 2), ld + "enc2.0", 1))
    e3 = F.silu(conv(F.max_pool2d(e2, 2), ld + "enc3.0", 1))
    e4 = F.silu(conv(F.max_pool2d(e3, 2), ld + "enc4.0", 1))
    h = F.silu(conv(torch.cat((F.max_pool2d(e4, 2), feat), 1), ld + "bottleneck.0", 0))
    for lvl, skip in ((4, e4), (3, e3), (2, e2), (1, e1)):
        h = conv(F.interpolate(h, scale_factor=2, mode="nearest"), ld + f"up{lvl}.1", 1)
        h = F.silu(conv(torch.cat((h, skip), 1), ld + f"dec{lvl}.0", 1))
    want = -conv(h, ld + "out_conv", 0)
    assert F.cosine_similarity(got.flatten(), want.flatten(), 0) > 0.99999 and (got - want).abs().max() < 2e-4 * want.abs().max() + 1e-5

    # checkpoint layout of the convolutions and one guided Euler step
    raw = {k: (v.permute(0, 3, 1, 2).contiguous() if k.startswith(ld) and v.dim() == 4 else v) for k, v in sd.items()}
    assert all(torch.equal(v, sd[k]) for k, v in Z.remap_l2p_keys(raw).items())
    x0 = torch.randn(1, 3, H, W)
    out = Z.l2p_sample(m, cap[:1], cap[1:, :3], H, W, steps=2, cfg_scale=2.0, shift=3.0, x=x0)
    s2 = Z.l2p_sigmas(2, 3.0)
    xx = x0
    for i in range(2):
        sg = torch.tensor([s2[i]])
        pc, pu = m(xx, cap[:1], sg), m(xx, cap[1:, :3], sg)
        xx = xx + (s2[i + 1] - s2[i]) * (pu + 2.0 * (pc - pu))
    assert torch.allclose(out, xx, atol=1e-5)


def test_lens_double_stream_dit_matches_plain_torch_statement():
    """Lens: tensor inventory of the full architecture (1264 tensors, the checkpoint's names and shapes), rotary angles of image
    and text tokens, the text plan, and the tiny model against a plain-torch forward (weighted RMS pre-norms, fused qkv,
    SwiGLU, four normalised text layers)."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models import lens as Ls
    torch.manual_seed(21)
    assert Ls.lens_text_plan() == (415, 4511) and Ls.lens_text_plan(353) == (256, 4352)
    full = Ls.LensDiT(Ls.LensConfig(), torch.float32, "meta")
    shapes = {k: tuple(v.shape) for k, v in full.state_dict().items()}
    assert len(shapes) == 1264
    for k, s in {"img_in.weight": (1536, 128), "txt_in.weight": (1536, 11520), "txt_norm.3.weight": (2880,),
                 "transformer_blocks.0.img_mod.1.weight": (9216, 1536), "transformer_blocks.0.txt_norm2.weight": (1536,),
                 "transformer_blocks.47.attn.img_qkv.bias": (4608,), "transformer_blocks.0.attn.norm_added_k.weight": (64,),
                 "transformer_blocks.0.attn.to_add_out.bias": (1536,), "transformer_blocks.0.img_mlp.w1.weight": (4096, 1536),
                 "transformer_blocks.0.txt_mlp.w2.weight": (1536, 4096)}.items():
        assert shapes[k] == s, k
    assert "transformer_blocks.0.img_mlp.w1.bias" not in shapes

    # rotary angles: image token (y, x) of a 64 x 64 grid and text token i, per frequency pair
    ids = Ls.LensDiT.make_ids(64, 64, 8)
    cos, _ = __import__("mojodiffusion_b200").ops.rope_table(ids, (8, 28, 28), 1.0e4)
    tok = 5 * 64 + 40
    for pair, want in ((2, 0.0), (4 + 3, (5 - 32) / 1.0e4 ** (6 / 28.0)), (18 + 5, (40 - 32) / 1.0e4 ** (10 / 28.0))):
        assert abs(float(cos[tok, pair]) - math.cos(want)) < 1e-5
    for pair, want in ((1, (32 + 3) / 1.0e4 ** (2 / 8.0)), (4 + 2, (32 + 3) / 1.0e4 ** (4 / 28.0)), (18, 35.0)):
        assert abs(float(cos[4096 + 3, pair]) - math.cos(want)) < 1e-5

    cfg = Ls.tiny_lens_config()
    m = Ls.LensDiT(cfg, torch.float32).init_weights(2)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    B, gh, gw, St = 2, 4, 6, 5
    D, H, Dh = cfg.hidden, cfg.heads, cfg.head_dim
    img, layers, t = torch.randn(B, gh * gw, cfg.in_channels), torch.randn(B, St, 4, cfg.text_hidden), torch.tensor([0.2, 0.7])
    got = m(img, layers, t, (gh, gw))
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, n, eps=1e-6: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps) * sd[n + ".weight"]
    args = (t * 1000.0)[:, None] * torch.exp(-math.log(1.0e4) * torch.arange(128).float() / 128)[None]
    temb = F.silu(lin(F.silu(lin(torch.cat((args.cos(), args.sin()), -1), "time_text_embed.timestep_embedder.linear_1")),
                      "time_text_embed.timestep_embedder.linear_2"))
    x = lin(img, "img_in")
    y = lin(torch.cat([rms(layers[:, :, j], f"txt_norm.{j}", 1e-5) for j in range(4)], -1), "txt_in")
    pos = torch.zeros(gh * gw + St, 3)
    pos[:gh * gw, 1] = (torch.arange(gh).float() - gh // 2).repeat_interleave(gw)
    pos[:gh * gw, 2] = (torch.arange(gw).float() - gw // 2).repeat(gh)
    pos[gh * gw:] = (max(gh, gw) // 2 + torch.arange(St).float())[:, None]
    ang = torch.cat([pos[:, a:a + 1] / (1.0e4 ** (torch.arange(0, d, 2).float() / d))[None] for a, d in enumerate(cfg.axes_dim)], -1)

    def rope(v):
        c, s = ang.cos()[None, :, None], ang.sin()[None, :, None]
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack((a * c - b * s, a * s + b * c), -1).flatten(-2)

    for i in range(cfg.depth):
        p = f"transformer_blocks.{i}."
        mi, mt = lin(temb, p + "img_mod.1")[:, None].chunk(6, -1), lin(temb, p + "txt_mod.1")[:, None].chunk(6, -1)
        qi = lin(rms(x, p + "img_norm1") * (1 + mi[1]) + mi[0], p + "attn.img_qkv").reshape(B, -1, 3, H, Dh)
        qt = lin(rms(y, p + "txt_norm1") * (1 + mt[1]) + mt[0], p + "attn.txt_qkv").reshape(B, -1, 3, H, Dh)
        q = rope(torch.cat((rms(qi[:, :, 0], p + "attn.norm_q"), rms(qt[:, :, 0], p + "attn.norm_added_q")), 1))
        k = rope(torch.cat((rms(qi[:, :, 1], p + "attn.norm_k"), rms(qt[:, :, 1], p + "attn.norm_added_k")), 1))
        v = torch.cat((qi[:, :, 2], qt[:, :, 2]), 1)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).reshape(B, -1, D)
        x = x + mi[2] * lin(o[:, :gh * gw], p + "attn.to_out.0")
        y = y + mt[2] * lin(o[:, gh * gw:], p + "attn.to_add_out")
        ffn = lambda v_, n: lin(F.silu(lin(v_, n + ".w1")) * lin(v_, n + ".w3"), n + ".w2")
        x = x + mi[5] * ffn(rms(x, p + "img_norm2") * (1 + mi[4]) + mi[3], p + "img_mlp")
        y = y + mt[5] * ffn(rms(y, p + "txt_norm2") * (1 + mt[4]) + mt[3], p + "txt_mlp")
    sc, sh = lin(temb, "norm_out.linear")[:, None].chunk(2, -1)
    want = lin(F.layer_norm(x, (D,), eps=1e-6) * (1 + sc) + sh, "proj_out")
    assert F.cosine_similarity(got.flatten(), want.flatten(), 0) > 0.99999 and (got - want).abs().max() < 2e-4 * want.abs().max() + 1e-5


def test_lance_t2v_two_expert_spine_matches_plain_torch_statement():
    """Lance T2V: sequence / position builder, mask, full-width three-axis rotary table, and the model against a plain-torch
    forward written as "run every row through the text weights, then overwrite the generated rows with the generation
    weights' result"."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models import lance as La
    torch.manual_seed(31)
    full = La.LanceConfig()
    inp = La.build_lance_input(full, [11, 12, 13], 2, 2, 3)
    assert inp.full_ids[:5] == (full.bos_token_id, 11, 12, 13, full.eos_token_id) and inp.full_ids[5] == full.start_of_image_id
    assert inp.text_split_len == 5 and inp.gen_start == 6 and inp.gen_len == 12 and inp.full_ids[-1] == full.end_of_image_id
    assert inp.t_pos[:6] == tuple(range(6)) and (inp.t_pos[6 + 7], inp.h_pos[6 + 7], inp.w_pos[6 + 7]) == (6 + 2, 6 + 0, 6 + 1)
    assert inp.latent_pos_ids[7] == 1 * 64 * 64 + 0 * 64 + 1 and inp.t_pos[-1] == inp.h_pos[-1] == inp.w_pos[-1] == 6 + 2 + 1
    mk = La.lance_mask(5, 3)[0, 0]
    assert mk.tolist() == [[0, -1e4, -1e4, -1e4, -1e4], [0, 0, -1e4, -1e4, -1e4], [0, 0, 0, -1e4, -1e4], [0] * 5, [0] * 5]
    cos, sin = La.lance_rope_table(inp, 128, 1.0e6, (16, 24, 24))
    row = 6 + 7
    for d, axis_pos in ((5, inp.t_pos[row]), (31, inp.t_pos[row]), (32, inp.h_pos[row]), (70, inp.h_pos[row]), (79, inp.h_pos[row]),
                        (80, inp.w_pos[row]), (127, inp.w_pos[row])):
        want = axis_pos * math.exp(-math.log(1.0e6) * (d % 64) / 64)
        assert abs(float(cos[row, d]) - math.cos(want)) < 1e-5 and abs(float(sin[row, d]) - math.sin(want)) < 1e-5

    cfg = La.tiny_lance_config()
    m = La.LanceT2V(cfg, torch.float32).init_weights(8)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() == 1 or n.endswith("pos_embed"):
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    for k in ("language_model.model.embed_tokens.weight", "language_model.model.norm_moe_gen.weight", "vae2llm.bias", "llm2vae.weight",
              "time_embedder.mlp.2.bias", "latent_pos_embed.pos_embed", "language_model.model.layers.1.self_attn.q_proj_moe_gen.bias",
              "language_model.model.layers.0.self_attn.k_norm_moe_gen.weight", "language_model.model.layers.0.mlp_moe_gen.down_proj.weight",
              "language_model.model.layers.0.post_attention_layernorm_moe_gen.weight", "language_model.model.layers.0.self_attn.o_proj.weight"):
        assert k in sd, k
    assert "language_model.model.layers.0.self_attn.o_proj.bias" not in sd
    inp = La.build_lance_input(cfg, [3, 4, 5, 6], 2, 2, 3)
    x_t, t = torch.randn(inp.gen_len, cfg.patch_latent_dim), torch.tensor([0.37])
    got = m(inp, x_t, t)
    assert got.shape == (inp.gen_len, cfg.patch_latent_dim)

    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, n: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * sd[n + ".weight"]
    S, g0, g1 = len(inp.full_ids), inp.gen_start, inp.gen_start + inp.gen_len
    H, KV, Dh = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim

    def span(all_rows, gen_rows):
        out = all_rows.clone()
        out[:, g0:g1] = gen_rows
        return out

    half = cfg.timestep_dim // 2
    args = t[:, None] * torch.exp(-math.log(1.0e4) * torch.arange(half).float() / half)[None]
    temb = lin(F.silu(lin(torch.cat((args.cos(), args.sin()), -1), "time_embedder.mlp.0")), "time_embedder.mlp.2")
    h = sd["language_model.model.embed_tokens.weight"][list(inp.full_ids)][None]
    h = span(h, lin(x_t[None], "vae2llm") + temb[:, None] + sd["latent_pos_embed.pos_embed"][list(inp.latent_pos_ids)][None])
    cos, sin = La.lance_rope_table(inp, Dh, cfg.rope_theta, cfg.mrope)
    rot = lambda v: v * cos[None, :, None] + torch.cat((-v[..., Dh // 2:], v[..., :Dh // 2]), -1) * sin[None, :, None]
    mask = La.lance_mask(S, inp.text_split_len)
    for i in range(cfg.num_layers):
        p = f"language_model.model.layers.{i}."
        n1 = span(rms(h, p + "input_layernorm"), rms(h[:, g0:g1], p + "input_layernorm_moe_gen"))
        q, k, v = (span(lin(n1, p + f"self_attn.{w}_proj"), lin(n1[:, g0:g1], p + f"self_attn.{w}_proj_moe_gen")) for w in "qkv")
        q, k, v = q.reshape(1, S, H, Dh), k.reshape(1, S, KV, Dh), v.reshape(1, S, KV, Dh)
        q, k = rms(q, p + "self_attn.q_norm"), rms(k, p + "self_attn.k_norm")
        q = span(q, rms(q[:, g0:g1], p + "self_attn.q_norm_moe_gen"))
        k = span(k, rms(k[:, g0:g1], p + "self_attn.k_norm_moe_gen"))
        q, k = rot(q), rot(k)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask, enable_gqa=True)
        o = o.transpose(1, 2).reshape(1, S, H * Dh)
        h = h + span(lin(o, p + "self_attn.o_proj"), lin(o[:, g0:g1], p + "self_attn.o_proj_moe_gen"))
        ffn = lambda v_, n: lin(F.silu(lin(v_, n + ".gate_proj")) * lin(v_, n + ".up_proj"), n + ".down_proj")
        h = h + span(ffn(rms(h, p + "post_attention_layernorm"), p + "mlp"),
                     ffn(rms(h[:, g0:g1], p + "post_attention_layernorm_moe_gen"), p + "mlp_moe_gen"))
    want = lin(rms(h[:, g0:g1], "language_model.model.norm_moe_gen"), "llm2vae")[0]
    assert F.cosine_similarity(got.flatten(), want.flatten(), 0) > 0.99999 and (got - want).abs().max() < 2e-4 * want.abs().max() + 1e-5
    # the single-norm variant differs, and the text prefix is causal: a later text token does not move... the generated rows see all text
    assert (m(inp, x_t, t, renorm_gen=False) - got).abs().max() > 1e-4
    inp2 = La.build_lance_input(cfg, [3, 4, 5, 7], 2, 2, 3)
    assert (m(inp2, x_t, t) - got).abs().max() > 1e-5


def test_magihuman_three_modality_dit_matches_plain_torch_statement():
    """MagiHuman: tensor inventory of the 15 B architecture (331 tensors), SwiGLU7 / GELU7, the Fourier rotary table, the model
    against a plain-torch forward that picks every token's weight set by a modality index, and the split super-resolution
    checkpoint layout mapped onto the fused one."""
    import torch.nn.functional as F
    from mojodiffusion_b200.models import magihuman as M
    torch.manual_seed(41)
    full = M.MagiHumanDiT(M.MagiHumanConfig(), torch.float32, "meta")
    shapes = {k: tuple(v.shape) for k, v in full.state_dict().items()}
    assert len(shapes) == 331
    for k, s in {"adapter.rope.bands": (16,), "adapter.text_embedder.weight": (5120, 3584), "block.layers.4.attention.linear_qkv.weight": (7208, 5120),
                 "block.layers.0.attention.linear_qkv.weight": (3 * 7208, 5120), "block.layers.0.mlp.up_gate_proj.weight": (3 * 20480, 5120),
                 "block.layers.36.mlp.up_gate_proj.weight": (3 * 27304, 5120), "block.layers.20.mlp.down_proj.weight": (5120, 13652),
                 "block.layers.39.attention.q_norm.weight": (3 * 128,), "final_linear_audio.weight": (64, 5120)}.items():
        assert shapes[k] == s, k
    x = torch.tensor([[8.0, -9.0, -1.0, 0.5]])
    assert torch.allclose(M.swiglu7(x), torch.tensor([[7.0 * torch.sigmoid(torch.tensor(1.702 * 7.0)) * (-7.0 + 1.0),
                                                       -1.0 * torch.sigmoid(torch.tensor(-1.702)) * 1.5]]))
    assert torch.allclose(M.gelu7(torch.tensor([9.0, -2.0])), torch.tensor([7.0, -2.0]) * torch.sigmoid(1.702 * torch.tensor([7.0, -2.0])))
    coords = torch.tensor([[3.0, 2.0, 5.0, 4.0, 6.0, 8.0, 4.0, 12.0, 16.0]])
    bands = torch.tensor([1.0, 0.1])
    cos, sin = M.fourier_rope(coords, bands)
    cx = [3.0 * (3.0 / 3.0), (2.0 - 2.5) * (11.0 / 5.0), (5.0 - 3.5) * (15.0 / 7.0)]
    want = torch.tensor([c * b for c in cx for b in (1.0, 0.1)], dtype=torch.float64)
    assert cos.shape == (1, 6) and torch.allclose(cos[0].double(), want.cos(), atol=1e-6) and torch.allclose(sin[0].double(), want.sin(), atol=1e-6)

    cfg = M.tiny_magihuman_config()
    m = M.MagiHumanDiT(cfg, torch.float32).init_weights(4)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() == 1 and "bands" not in n:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    V, A, T = 6, 3, 4
    L = V + A + T
    video, audio, text = torch.randn(V, cfg.video_in), torch.randn(A, cfg.audio_in), torch.randn(T, cfg.text_in)
    coords = torch.cat((torch.stack(torch.meshgrid(torch.arange(1.0), torch.arange(2.0), torch.arange(3.0), indexing="ij"), -1).reshape(V, 3),
                        torch.stack((torch.arange(A).float(), torch.zeros(A), torch.zeros(A)), 1),
                        torch.stack((torch.arange(T).float(), torch.zeros(T), torch.zeros(T)), 1)), 0)
    coords = torch.cat((coords, torch.tensor([[1.0, 2.0, 3.0, 1.0, 4.0, 6.0]]).expand(L, 6)), 1)
    got = m(video, audio, text, coords)
    assert got.shape == (L, cfg.video_in) and float(got[V + A:].abs().sum()) == 0 and float(got[V:V + A, cfg.audio_in:].abs().sum()) == 0

    mod = torch.tensor([0] * V + [1] * A + [2] * T)
    H, KV, Dh, D = cfg.num_heads_q, cfg.num_heads_kv, cfg.head_dim, cfg.hidden_size
    x = torch.cat((F.linear(video, sd["adapter.video_embedder.weight"], sd["adapter.video_embedder.bias"]),
                   F.linear(audio, sd["adapter.audio_embedder.weight"], sd["adapter.audio_embedder.bias"]),
                   F.linear(text, sd["adapter.text_embedder.weight"], sd["adapter.text_embedder.bias"])), 0)
    cos, sin = M.fourier_rope(coords, sd["adapter.rope.bands"])

    def per_token_linear(v, w, sets):          # v [L, in]; w [sets * out, in]
        w3 = w.reshape(sets, -1, w.shape[-1])
        return torch.einsum("li,loi->lo", v, w3[mod if sets == 3 else torch.zeros_like(mod)])

    def per_token_norm(v, w, sets):            # v [L, ..., dim]; w [sets * dim]
        gain = (w.reshape(sets, -1) + 1.0)[mod if sets == 3 else torch.zeros_like(mod)]
        gain = gain.reshape(L, *([1] * (v.dim() - 2)), -1)
        return v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * gain

    def rope(v):
        r = cfg.rope_dim
        a, b = v[..., :r // 2], v[..., r // 2:r]
        c, s = cos[:, None], sin[:, None]
        return torch.cat((a * c - b * s, b * c + a * s, v[..., r:]), -1)

    for i in range(cfg.num_layers):
        p = f"block.layers.{i}."
        sets = 3 if i in cfg.mm_layers else 1
        qkv = per_token_linear(per_token_norm(x, sd[p + "attention.pre_norm.weight"], sets), sd[p + "attention.linear_qkv.weight"], sets)
        q, k, v, g = qkv.split((H * Dh, KV * Dh, KV * Dh, H), -1)
        q = rope(per_token_norm(q.reshape(L, H, Dh), sd[p + "attention.q_norm.weight"], sets)).transpose(0, 1)
        k = rope(per_token_norm(k.reshape(L, KV, Dh), sd[p + "attention.k_norm.weight"], sets)).transpose(0, 1)
        o = F.scaled_dot_product_attention(q[None], k[None], v.reshape(L, KV, Dh).transpose(0, 1)[None], enable_gqa=True)[0].transpose(0, 1)
        o = (o * torch.sigmoid(g)[..., None]).reshape(L, H * Dh)
        x = x + per_token_linear(o, sd[p + "attention.linear_proj.weight"], sets)
        up = per_token_linear(per_token_norm(x, sd[p + "mlp.pre_norm.weight"], sets), sd[p + "mlp.up_gate_proj.weight"], sets)
        act = M.gelu7(up) if i in cfg.gelu7_layers else M.swiglu7(up)
        x = x + per_token_linear(act, sd[p + "mlp.down_proj.weight"], sets)
    nrm = lambda v, w: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_eps) * (w + 1.0)
    want_v = F.linear(nrm(x[:V], sd["final_norm_video.weight"]), sd["final_linear_video.weight"])
    want_a = F.linear(nrm(x[V:V + A], sd["final_norm_audio.weight"]), sd["final_linear_audio.weight"])
    assert F.cosine_similarity(got[:V].flatten(), want_v.flatten(), 0) > 0.99999 and (got[:V] - want_v).abs().max() < 2e-4 * want_v.abs().max() + 1e-5
    assert (got[V:V + A, :cfg.audio_in] - want_a).abs().max() < 2e-4 * want_a.abs().max() + 1e-5

    # super-resolution layout: split the fused tensors the way that checkpoint stores them, then map back
    split = {}
    for k, v in sd.items():
        if k.endswith("attention.linear_qkv.weight") or (".mlp." in k and "pre_norm" not in k) or k.endswith("attention.linear_proj.weight"):
            i = int(k.split(".")[2])
            sets = 3 if i in cfg.mm_layers else 1
            base = k[:-len(".weight")]
            chunks = v.reshape(sets, -1, v.shape[-1])
            for s in range(sets):
                suffix = ("_" + M.MODALITIES[s]) if sets == 3 else ""
                if k.endswith("linear_qkv.weight"):
                    for name, part in zip("qkvg", chunks[s].split((H * Dh, KV * Dh, KV * Dh, H), 0)):
                        split[base[:-len("linear_qkv")] + f"linear_{name}{suffix}.weight"] = part
                elif sets == 3:
                    split[base + suffix + ".weight"] = chunks[s]
                else:
                    split[k] = v
        else:
            split[k] = v
    assert "block.layers.1.attention.linear_q.weight" in split and "block.layers.0.mlp.down_proj_text.weight" in split
    back = M.remap_magihuman_sr_keys(split, cfg)
    assert set(back) == set(sd) and all(torch.equal(back[k], sd[k]) for k in sd)
    # distilled sampler step
    xs, vs, ns = torch.randn(4), torch.randn(4), torch.randn(4)
    assert torch.allclose(M.distilled_step(xs, vs, ns, 0.8, 0.5), 0.5 * ns + 0.5 * (xs - 0.8 * vs))


def test_sensenova_u1_two_weight_set_pixel_model_matches_plain_torch_statement():
    """SenseNova-U1: tensor inventory of the text-to-image part (26 tensors per layer + 23 shared), patch orders, noise scale, time
    table, and prompt pass + image pass + head against a plain-torch forward over ONE joint sequence with an explicit mask
    (prompt rows causal, image rows see everything), which must equal the cached two-pass form."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models import sensenova_u1 as S
    torch.manual_seed(51)
    full = S.SenseNovaU1(S.SenseNovaU1Config(), torch.float32, "meta")
    shapes = {k: tuple(v.shape) for k, v in full.state_dict().items()}
    assert len(shapes) == 26 * 42 + 3 + 4 + 4 + 4 + 4 and S.SenseNovaU1Config().fm_head_out_dim == 3072
    for k, s in {"language_model.model.layers.0.self_attn.q_norm.weight": (64,), "language_model.model.layers.41.self_attn.k_norm_hw_mot_gen.weight": (64,),
                 "language_model.model.layers.3.self_attn.k_proj_mot_gen.weight": (1024, 4096), "language_model.model.norm_mot_gen.weight": (4096,),
                 "fm_modules.vision_model_mot_gen.embeddings.patch_embedding.weight": (1024, 3, 16, 16),
                 "fm_modules.vision_model_mot_gen.embeddings.dense_embedding.weight": (4096, 1024, 2, 2),
                 "fm_modules.noise_scale_embedder.mlp.0.weight": (4096, 256), "fm_modules.fm_head.2.weight": (3072, 4096)}.items():
        assert shapes[k] == s, k
    assert abs(full.noise_scale(16, 16) - 1.0) < 1e-6 and abs(full.noise_scale(64, 64) - 4.0) < 1e-6 and full.noise_scale(256, 256) == 8.0
    ts = S.time_schedule(4, 3.0)
    assert ts[0] == 0.0 and ts[-1] == 1.0 and abs(ts[2] - (1 - 3 * 0.5 / 2.0)) < 1e-12
    img = torch.randn(1, 3, 8, 12)
    pc, pl = S.patchify(img, 4, True), S.patchify(img, 4, False)
    assert torch.equal(pc[0, 4].reshape(3, 4, 4), img[0, :, 4:8, 4:8]) and torch.equal(pl[0, 4].reshape(4, 4, 3), img[0, :, 4:8, 4:8].permute(1, 2, 0))
    assert torch.equal(S.unpatchify(pl, 4, 8, 12), img)

    cfg = S.tiny_sensenova_u1_config()
    m = S.SenseNovaU1(cfg, torch.float32).init_weights(6)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    ids = [5, 9, 2, 7, 11]
    Hh, Ww = 16, 24
    gh, gw, th, tw = Hh // 4, Ww // 4, Hh // 8, Ww // 8
    x_img, t = torch.randn(1, 3, Hh, Ww), 0.3
    cache = m.forward_und(ids)
    got = m.predict_clean(x_img, t, cache, len(ids))
    assert got.shape == (1, th * tw, cfg.fm_head_out_dim)

    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, n: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * sd[n + ".weight"]
    gelu = lambda v: F.gelu(v, approximate="tanh")
    H, KV, Dh, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden_size
    # image tokens
    px = S.patchify(x_img, 4, True)[0]
    f = gelu(F.linear(px, sd["fm_modules.vision_model_mot_gen.embeddings.patch_embedding.weight"].flatten(1),
                      sd["fm_modules.vision_model_mot_gen.embeddings.patch_embedding.bias"]))
    vh = cfg.vision_hidden_size

    def pair_rot(v, pos, dim):
        ang = pos.float()[:, None] / (1.0e4 ** (torch.arange(0, dim, 2).float() / dim))[None]
        return torch.view_as_real(torch.view_as_complex(v.reshape(v.shape[0], -1, 2).contiguous()) * torch.polar(torch.ones_like(ang), ang)).flatten(1)

    n = torch.arange(gh * gw)
    f = torch.cat((pair_rot(f[:, :vh // 2], n % gw, vh // 2), pair_rot(f[:, vh // 2:], n // gw, vh // 2)), -1)
    f = f.reshape(th, 2, tw, 2, vh).permute(0, 2, 4, 1, 3).reshape(th * tw, vh * 4)
    e = F.linear(f, sd["fm_modules.vision_model_mot_gen.embeddings.dense_embedding.weight"].flatten(1),
                 sd["fm_modules.vision_model_mot_gen.embeddings.dense_embedding.bias"])

    def scalar(v, name):
        args = torch.tensor([v])[:, None] * torch.exp(-math.log(1.0e4) * torch.arange(128).float() / 128)[None]
        return lin(F.silu(lin(torch.cat((args.cos(), args.sin()), -1), name + ".mlp.0")), name + ".mlp.2")

    e = e + scalar(t, "fm_modules.timestep_embedder") + scalar(m.noise_scale(gh, gw) / 8.0, "fm_modules.noise_scale_embedder")
    # one joint sequence: prompt rows on the base weights, image rows on the generation weights
    P, L = len(ids), th * tw
    pos = torch.zeros(P + L, 3)
    pos[:P, 0] = torch.arange(P).float()
    pos[P:, 0] = P
    pos[P:, 1] = (torch.arange(L) // tw).float()
    pos[P:, 2] = (torch.arange(L) % tw).float()
    x = torch.cat((sd["language_model.model.embed_tokens.weight"][ids], e), 0)[None]
    mask = torch.ones(P + L, P + L, dtype=torch.bool).tril()
    mask[P:] = True

    def rot(v, p_, dim, theta):                # half-split, v [1, S, heads, dim]
        ang = p_[:, None] / (theta ** (torch.arange(0, dim, 2).float() / dim))[None]
        c_, s_ = ang.cos()[None, :, None], ang.sin()[None, :, None]
        a_, b_ = v.chunk(2, -1)
        return torch.cat((a_ * c_ - b_ * s_, b_ * c_ + a_ * s_), -1)

    def two(fn, v):                            # fn(rows, suffix)
        return torch.cat((fn(v[:, :P], ""), fn(v[:, P:], "_mot_gen")), 1)

    for i in range(cfg.num_layers):
        p = f"language_model.model.layers.{i}."
        h = two(lambda r, s: rms(r, p + "input_layernorm" + s), x)

        def qk(which, heads):
            raw = two(lambda r, s: lin(r, p + f"self_attn.{which}_proj" + s), h).reshape(1, P + L, heads, Dh)
            vt = two(lambda r, s: rms(r[..., :Dh // 2], p + f"self_attn.{which}_norm" + s), raw)
            vhw = two(lambda r, s: rms(r[..., Dh // 2:], p + f"self_attn.{which}_norm_hw" + s), raw)
            return torch.cat((rot(vt, pos[:, 0], Dh // 2, cfg.rope_theta), rot(vhw[..., :Dh // 4], pos[:, 1], Dh // 4, 1.0e4),
                              rot(vhw[..., Dh // 4:], pos[:, 2], Dh // 4, 1.0e4)), -1)

        q, k = qk("q", H), qk("k", KV)
        v = two(lambda r, s: lin(r, p + "self_attn.v_proj" + s), h).reshape(1, P + L, KV, Dh)
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask, enable_gqa=True)
        o = o.transpose(1, 2).reshape(1, P + L, H * Dh)
        x = x + two(lambda r, s: lin(r, p + "self_attn.o_proj" + s), o)
        h2 = two(lambda r, s: rms(r, p + "post_attention_layernorm" + s), x)
        x = x + two(lambda r, s: lin(F.silu(lin(r, p + f"mlp{s}.gate_proj")) * lin(r, p + f"mlp{s}.up_proj"), p + f"mlp{s}.down_proj"), h2)
    want = lin(gelu(lin(rms(x[:, P:], "language_model.model.norm_mot_gen"), "fm_modules.fm_head.0")), "fm_modules.fm_head.2")
    assert F.cosine_similarity(got.flatten(), want.flatten(), 0) > 0.99999 and (got - want).abs().max() < 2e-4 * want.abs().max() + 1e-5

    # one guided Euler step of the sampler
    out = m.sample(ids, [5, 9], Hh, Ww, steps=1, cfg_scale=2.0, shift=3.0, noise=x_img)
    z = S.patchify(x_img * m.noise_scale(gh, gw), 8, False)
    vc = (m.predict_clean(x_img * m.noise_scale(gh, gw), 0.0, cache, 5) - z) / 1.0
    vu = (m.predict_clean(x_img * m.noise_scale(gh, gw), 0.0, m.forward_und([5, 9]), 2) - z) / 1.0
    assert torch.allclose(out, S.unpatchify(z + 1.0 * (vu + 2.0 * (vc - vu)), 8, Hh, Ww) * 0.5 + 0.5, atol=1e-5)


def test_boogu_double_then_single_stream_dit_matches_plain_torch_statement():
    """Boogu-Image: checkpoint names of the full architecture, patch order, positions, and the tiny model against a plain-torch
    forward (norm-zero modulation chunks, tanh gates, joint attention with per-stream projections plus the image self-attention,
    feed-forward input built from norm2's output with norm1's scale and norm2's chunk-1 shift)."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models import boogu as Bg
    torch.manual_seed(61)
    full = Bg.BooguDiT(Bg.BooguConfig(), torch.float32, "meta")
    shapes = {k: tuple(v.shape) for k, v in full.state_dict().items()}
    for k, s in {"x_embedder.weight": (3360, 64), "time_caption_embed.timestep_embedder.linear_1.weight": (1024, 256),
                 "time_caption_embed.caption_embedder.0.weight": (4096,), "time_caption_embed.caption_embedder.1.weight": (3360, 4096),
                 "context_refiner.1.norm1.weight": (3360,), "noise_refiner.0.norm1.linear.weight": (4 * 3360, 1024),
                 "single_stream_layers.31.attn.to_k.weight": (840, 3360), "single_stream_layers.0.attn.norm_q.weight": (120,),
                 "single_stream_layers.0.feed_forward.linear_3.weight": (13568, 3360),
                 "double_stream_layers.7.img_instruct_attn.processor.instruct_to_v.weight": (840, 3360),
                 "double_stream_layers.0.img_instruct_attn.processor.img_out.weight": (3360, 3360),
                 "double_stream_layers.0.img_instruct_attn.to_out.0.weight": (3360, 3360), "double_stream_layers.0.img_norm3.linear.bias": (4 * 3360,),
                 "double_stream_layers.0.img_self_attn.to_out.0.weight": (3360, 3360), "double_stream_layers.0.instruct_ffn_norm2.weight": (3360,),
                 "norm_out.linear_1.weight": (3360, 1024), "norm_out.linear_2.bias": (64,)}.items():
        assert shapes[k] == s, k
    assert not any(k.endswith("to_q.bias") or k.endswith("linear_1.bias") and "feed_forward" in k for k in shapes)
    lat = torch.randn(1, 4, 4, 6)
    tok = Bg.boogu_patchify(lat)
    assert torch.equal(tok[0, 1 * 3 + 2].reshape(2, 2, 4), lat[0, :, 2:4, 4:6].permute(1, 2, 0)) and torch.equal(Bg.boogu_unpatchify(tok, 2, 3), lat)
    pos = Bg.boogu_positions(3, 2, 4)
    assert pos[2].tolist() == [2.0, 2.0, 2.0] and pos[3 + 1 * 4 + 2].tolist() == [3.0, 1.0, 2.0]

    cfg = Bg.tiny_boogu_config()
    m = Bg.BooguDiT(cfg, torch.float32).init_weights(9)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() == 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    B, Hh, Ww, Lc = 2, 4, 6, 5
    h, w = Hh // 2, Ww // 2
    latent, ins_in, t = torch.randn(B, cfg.in_channels, Hh, Ww), torch.randn(B, Lc, cfg.instruction_dim), torch.tensor([0.15, 0.8])
    got = m(latent, ins_in, t)
    assert got.shape == latent.shape

    D, H, KV, Dh = cfg.hidden, cfg.heads, cfg.kv_heads, cfg.head_dim
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, n: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.eps) * sd[n + ".weight"]
    args = (t * 1000.0)[:, None] * torch.exp(-math.log(1.0e4) * torch.arange(128).float() / 128)[None]
    temb = lin(F.silu(lin(torch.cat((args.cos(), args.sin()), -1), "time_caption_embed.timestep_embedder.linear_1")),
               "time_caption_embed.timestep_embedder.linear_2")
    st = F.silu(temb)
    cap = lin(rms(ins_in, "time_caption_embed.caption_embedder.0"), "time_caption_embed.caption_embedder.1")
    pos = Bg.boogu_positions(Lc, h, w)
    ang = torch.cat([pos[:, a:a + 1] / (1.0e4 ** (torch.arange(0, d, 2).float() / d))[None] for a, d in enumerate(cfg.axes_dim)], -1)

    def rope(v, a):
        rot = torch.polar(torch.ones_like(a), a)[None, :, None]
        return torch.view_as_real(torch.view_as_complex(v.reshape(*v.shape[:-1], -1, 2).contiguous()) * rot).flatten(-2)

    def sdpa(q, k, v):
        return F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), enable_gqa=True).transpose(1, 2).flatten(-2)

    def self_attn(v_, p, a):
        q = rope(rms(lin(v_, p + ".to_q").unflatten(-1, (H, Dh)), p + ".norm_q"), a)
        k = rope(rms(lin(v_, p + ".to_k").unflatten(-1, (KV, Dh)), p + ".norm_k"), a)
        return lin(sdpa(q, k, lin(v_, p + ".to_v").unflatten(-1, (KV, Dh))), p + ".to_out.0")

    ffn = lambda v_, p: lin(F.silu(lin(v_, p + ".linear_1")) * lin(v_, p + ".linear_3"), p + ".linear_2")
    zero = lambda v_, p: (lambda e: (rms(v_, p + ".norm") * (1 + e[0]), e[1], e[2], e[3]))(lin(st, p + ".linear")[:, None].chunk(4, -1))

    def block(v_, p, a, mod):
        if not mod:
            v_ = v_ + rms(self_attn(rms(v_, p + ".norm1"), p + ".attn", a), p + ".norm2")
            return v_ + rms(ffn(rms(v_, p + ".ffn_norm1"), p + ".feed_forward"), p + ".ffn_norm2")
        hn, g1, s2, g2 = zero(v_, p + ".norm1")
        v_ = v_ + torch.tanh(g1) * rms(self_attn(hn, p + ".attn", a), p + ".norm2")
        return v_ + torch.tanh(g2) * rms(ffn(rms(v_, p + ".ffn_norm1") * (1 + s2), p + ".feed_forward"), p + ".ffn_norm2")

    cap = block(cap, "context_refiner.0", ang[:Lc], False)
    x = block(lin(Bg.boogu_patchify(latent), "x_embedder"), "noise_refiner.0", ang[Lc:], True)
    for i in range(cfg.n_double):
        p = f"double_stream_layers.{i}."
        jp = p + "img_instruct_attn.processor."
        i1, ig_msa, is_mlp, ig_mlp = zero(x, p + "img_norm1")
        i2, i_shift, _, _ = zero(x, p + "img_norm2")
        i3, ig_self, _, _ = zero(x, p + "img_norm3")
        t1, tg_msa, ts_mlp, tg_mlp = zero(cap, p + "instruct_norm1")
        t2, t_shift, _, _ = zero(cap, p + "instruct_norm2")
        q = torch.cat((lin(t1, jp + "instruct_to_q"), lin(i1, jp + "img_to_q")), 1).unflatten(-1, (H, Dh))
        k = torch.cat((lin(t1, jp + "instruct_to_k"), lin(i1, jp + "img_to_k")), 1).unflatten(-1, (KV, Dh))
        v = torch.cat((lin(t1, jp + "instruct_to_v"), lin(i1, jp + "img_to_v")), 1).unflatten(-1, (KV, Dh))
        o = sdpa(rope(rms(q, p + "img_instruct_attn.norm_q"), ang), rope(rms(k, p + "img_instruct_attn.norm_k"), ang), v)
        o = lin(torch.cat((lin(o[:, :Lc], jp + "instruct_out"), lin(o[:, Lc:], jp + "img_out")), 1), p + "img_instruct_attn.to_out.0")
        a_self = self_attn(i3, p + "img_self_attn", ang[Lc:])
        x = x + torch.tanh(ig_msa) * rms(o[:, Lc:], p + "img_attn_norm")
        x = x + torch.tanh(ig_self) * rms(a_self, p + "img_self_attn_norm")
        x = x + torch.tanh(ig_mlp) * rms(ffn(rms((1 + is_mlp) * i2 + i_shift, p + "img_ffn_norm1"), p + "img_feed_forward"), p + "img_ffn_norm2")
        cap = cap + torch.tanh(tg_msa) * rms(o[:, :Lc], p + "instruct_attn_norm")
        cap = cap + torch.tanh(tg_mlp) * rms(ffn(rms((1 + ts_mlp) * t2 + t_shift, p + "instruct_ffn_norm1"), p + "instruct_feed_forward"),
                                              p + "instruct_ffn_norm2")
    joint = torch.cat((cap, x), 1)
    for i in range(cfg.n_single):
        joint = block(joint, f"single_stream_layers.{i}", ang, True)
    y = F.layer_norm(joint, (D,), eps=1e-6) * (1 + lin(st, "norm_out.linear_1"))[:, None]
    want = Bg.boogu_unpatchify(lin(y, "norm_out.linear_2")[:, Lc:], h, w)
    assert F.cosine_similarity(got.flatten(), want.flatten(), 0) > 0.99999 and (got - want).abs().max() < 2e-4 * want.abs().max() + 1e-5


def test_nava_audio_video_dit_matches_plain_torch_statement():
    """NAVA: checkpoint names of the full architecture, the joint rotary table (video three axes, audio one position on 44
    columns), the fp8 + prefix key mapping, and the tiny model against a plain-torch forward with per-stream weights in the
    double blocks."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models import nava as Nv
    torch.manual_seed(71)
    full = Nv.NavaDiT(Nv.NavaConfig(), torch.float32, "meta")
    shapes = {k: tuple(v.shape) for k, v in full.state_dict().items()}
    for k, s in {"patch_embedding.weight": (3072, 48, 1, 2, 2), "patch_embedding_audio.0.weight": (3072, 128, 7), "patch_embedding_audio.0.bias": (3072,),
                 "patch_embedding_audio.2.w1.weight": (8192, 3072, 7), "patch_embedding_audio.2.w2.weight": (3072, 8192, 7),
                 "text_embedding.0.weight": (3072, 4096), "time_projection.1.weight": (18432, 3072),
                 "double_blocks.9.self_attn.q_audio.weight": (3072, 3072), "double_blocks.0.cross_attn.norm_k_audio.weight": (3072,),
                 "double_blocks.0.modulation_audio.modulation": (1, 6, 3072), "double_blocks.0.modulation.modulation": (1, 6, 3072),
                 "double_blocks.0.norm3.bias": (3072,), "double_blocks.0.ffn.0.weight": (14336, 3072),
                 "single_blocks.19.cross_attn.o.bias": (3072,), "single_blocks.0.modulation": (1, 6, 3072),
                 "head.head.weight": (192, 3072), "head.modulation": (1, 2, 3072), "head_audio.head.weight": (128, 3072)}.items():
        assert shapes[k] == s, k
    assert "patch_embedding_audio.2.w1.bias" not in shapes and "single_blocks.0.self_attn.q_audio.weight" not in shapes
    cos, sin = Nv.nava_rope_table(5, 8, 8, 34, Nv.NavaConfig())
    assert cos.shape == (354, 64)
    tok = 2 * 64 + 3 * 8 + 5
    for pair, want in ((0, 2.0), (21, 2.0 / 1.0e4 ** (42 / 44.0)), (22 + 4, 3.0 / 1.0e4 ** (8 / 42.0)), (43 + 20, 5.0 / 1.0e4 ** (40 / 42.0))):
        assert abs(float(cos[tok, pair]) - math.cos(want)) < 1e-5
    a7 = 7 * 0.24
    assert abs(float(sin[320 + 7, 3]) - math.sin(a7 / 1.0e4 ** (6 / 44.0))) < 1e-5 and float(cos[320 + 7, 22]) == 1.0 and float(sin[320 + 7, 63]) == 0.0

    cfg = Nv.tiny_nava_config()
    m = Nv.NavaDiT(cfg, torch.float32).init_weights(3)
    with torch.no_grad():
        g = torch.Generator().manual_seed(5)
        for n, p in m.named_parameters():
            if p.dim() == 1:
                p.add_(torch.randn(p.shape, generator=g) * 0.1)
            if p.dim() == 3 and "patch_embedding_audio" in n:
                p.copy_(torch.randn(p.shape, generator=g) / math.sqrt(p.shape[1] * p.shape[2]))
    sd = m.state_dict()
    B, Fr, Hh, Ww, Na, Lt = 1, 2, 4, 6, 5, 7
    video, audio, text, t = torch.randn(B, cfg.in_dim, Fr, Hh, Ww), torch.randn(B, Na, cfg.audio_dim), torch.randn(B, Lt, cfg.text_dim), torch.tensor([0.45])
    got_v, got_a = m(video, audio, text, t)
    assert got_v.shape == video.shape and got_a.shape == audio.shape

    D, H = cfg.dim, cfg.heads
    Dh = D // H
    f, h, w = Fr, Hh // 2, Ww // 2
    V = f * h * w
    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, n: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * sd[n + ".weight"]
    ln = lambda v: F.layer_norm(v, (D,), eps=1e-6)
    gelu = lambda v: F.gelu(v, approximate="tanh")
    tokv = video.reshape(B, cfg.in_dim, f, 1, h, 2, w, 2).permute(0, 2, 4, 6, 1, 3, 5, 7).reshape(B, V, -1)       # (c, pt, ph, pw) per token
    xv = F.linear(tokv, sd["patch_embedding.weight"].flatten(1), sd["patch_embedding.bias"])
    c1 = lambda v, n, b=None: F.conv1d(v.transpose(1, 2), sd[n + ".weight"], sd.get(n + ".bias"), padding=3).transpose(1, 2)
    ha = F.silu(c1(audio, "patch_embedding_audio.0"))
    xa = c1(F.silu(c1(ha, "patch_embedding_audio.2.w1")) * c1(ha, "patch_embedding_audio.2.w3"), "patch_embedding_audio.2.w2")
    ctx = lin(gelu(lin(torch.cat((text, torch.zeros(B, cfg.text_len - Lt, cfg.text_dim)), 1), "text_embedding.0")), "text_embedding.2")
    half = cfg.freq_dim // 2
    args = (t * 1000.0)[:, None] * torch.exp(-math.log(1.0e4) * torch.arange(half).float() / half)[None]
    e = lin(F.silu(lin(torch.cat((args.cos(), args.sin()), -1), "time_embedding.0")), "time_embedding.2")
    e0 = lin(F.silu(e), "time_projection.1").reshape(B, 6, D)
    vpos = torch.stack(torch.meshgrid(torch.arange(f).float(), torch.arange(h).float(), torch.arange(w).float(), indexing="ij"), -1).reshape(V, 3)
    vang = torch.cat([vpos[:, a:a + 1] / (1.0e4 ** (torch.arange(0, d, 2).float() / d))[None] for a, d in enumerate(cfg.axes_dim)], -1)
    aang = (torch.arange(Na).float() * 0.24)[:, None] / (1.0e4 ** (torch.arange(0, cfg.audio_rope_dim, 2).float() / cfg.audio_rope_dim))[None]

    def rope(v, ang, width):                       # v [B, S, H, Dh]; rotate the first ``width`` columns in interleaved pairs
        r = v[..., :width]
        rot = torch.polar(torch.ones_like(ang), ang)[None, :, None]
        r = torch.view_as_real(torch.view_as_complex(r.reshape(*r.shape[:-1], -1, 2).contiguous()) * rot).flatten(-2)
        return torch.cat((r, v[..., width:]), -1)

    sdpa = lambda q, k, v: F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(-2)
    heads = lambda v: v.unflatten(-1, (H, Dh))

    def cross(xs, p, sfx):
        q = heads(rms(lin(ln(xs) * sd[p + "norm3.weight"] + sd[p + "norm3.bias"], p + "cross_attn.q" + sfx), p + "cross_attn.norm_q" + sfx))
        k = heads(rms(lin(ctx, p + "cross_attn.k" + sfx), p + "cross_attn.norm_k" + sfx))
        return xs + lin(sdpa(q, k, heads(lin(ctx, p + "cross_attn.v" + sfx))), p + "cross_attn.o" + sfx)

    xv_, xa_ = xv, xa
    for i in range(cfg.double_depth):
        p = f"double_blocks.{i}."
        ev = (sd[p + "modulation.modulation"] + e0)[:, :, None]
        ea = (sd[p + "modulation_audio.modulation"] + e0)[:, :, None]
        nv, na = ln(xv_) * (1 + ev[:, 1]) + ev[:, 0], ln(xa_) * (1 + ea[:, 1]) + ea[:, 0]
        qv = rope(heads(rms(lin(nv, p + "self_attn.q"), p + "self_attn.norm_q")), vang, Dh)
        kv = rope(heads(rms(lin(nv, p + "self_attn.k"), p + "self_attn.norm_k")), vang, Dh)
        qa = rope(heads(rms(lin(na, p + "self_attn.q_audio"), p + "self_attn.norm_q_audio")), aang, cfg.audio_rope_dim)
        ka = rope(heads(rms(lin(na, p + "self_attn.k_audio"), p + "self_attn.norm_k_audio")), aang, cfg.audio_rope_dim)
        o = sdpa(torch.cat((qv, qa), 1), torch.cat((kv, ka), 1), torch.cat((heads(lin(nv, p + "self_attn.v")), heads(lin(na, p + "self_attn.v_audio"))), 1))
        xv_ = xv_ + lin(o[:, :V], p + "self_attn.o") * ev[:, 2]
        xa_ = xa_ + lin(o[:, V:], p + "self_attn.o_audio") * ea[:, 2]
        xv_, xa_ = cross(xv_, p, ""), cross(xa_, p, "_audio")
        xv_ = xv_ + lin(gelu(lin(ln(xv_) * (1 + ev[:, 4]) + ev[:, 3], p + "ffn.0")), p + "ffn.2") * ev[:, 5]
        xa_ = xa_ + lin(gelu(lin(ln(xa_) * (1 + ea[:, 4]) + ea[:, 3], p + "ffn.0")), p + "ffn.2") * ea[:, 5]
    x = torch.cat((xv_, xa_), 1)
    for i in range(cfg.depth):
        p = f"single_blocks.{i}."
        em = (sd[p + "modulation"] + e0)[:, :, None]
        n1 = ln(x) * (1 + em[:, 1]) + em[:, 0]
        q, k = heads(rms(lin(n1, p + "self_attn.q"), p + "self_attn.norm_q")), heads(rms(lin(n1, p + "self_attn.k"), p + "self_attn.norm_k"))
        q = torch.cat((rope(q[:, :V], vang, Dh), rope(q[:, V:], aang, cfg.audio_rope_dim)), 1)
        k = torch.cat((rope(k[:, :V], vang, Dh), rope(k[:, V:], aang, cfg.audio_rope_dim)), 1)
        x = x + lin(sdpa(q, k, heads(lin(n1, p + "self_attn.v"))), p + "self_attn.o") * em[:, 2]
        x = cross(x, p, "")
        x = x + lin(gelu(lin(ln(x) * (1 + em[:, 4]) + em[:, 3], p + "ffn.0")), p + "ffn.2") * em[:, 5]
    hv = (sd["head.modulation"] + e[:, None])[:, :, None]
    ha_ = (sd["head_audio.modulation"] + e[:, None])[:, :, None]
    want_v = lin(ln(x[:, :V]) * (1 + hv[:, 1]) + hv[:, 0], "head.head")
    want_v = want_v.reshape(B, f, h, w, 1, 2, 2, cfg.out_dim).permute(0, 7, 1, 4, 2, 5, 3, 6).reshape(video.shape)
    want_a = lin(ln(x[:, V:]) * (1 + ha_[:, 1]) + ha_[:, 0], "head_audio.head")
    for got, want in ((got_v, want_v), (got_a, want_a)):
        assert F.cosine_similarity(got.flatten(), want.flatten(), 0) > 0.99999 and (got - want).abs().max() < 2e-4 * want.abs().max() + 1e-5
    # per-modality attention in the double blocks changes the result; the checkpoint mapping strips the prefix and dequantises fp8 rows
    cfg0 = Nv.tiny_nava_config()
    cfg0.depth = 0
    m0 = Nv.NavaDiT(cfg0, torch.float32).init_weights(3)
    assert (m0(video, audio, text, t, masking_modality=True)[0] - m0(video, audio, text, t)[0]).abs().max() > 1e-6
    wq = torch.randn(4, 8).clamp(-2, 2).to(torch.float8_e4m3fn)
    raw = {"backbone.double_blocks.0.ffn.0.weight": wq, "backbone.double_blocks.0.ffn.0.weight_scale": torch.tensor([0.5, 1.0, 2.0, 4.0]),
           "backbone.double_blocks.0.ffn.0.bias": torch.ones(4), "other.key": torch.zeros(1)}
    mapped = Nv.remap_nava_keys(raw, torch.float32)
    assert set(mapped) == {"double_blocks.0.ffn.0.weight", "double_blocks.0.ffn.0.bias"}
    assert torch.equal(mapped["double_blocks.0.ffn.0.weight"], wq.float() * torch.tensor([0.5, 1.0, 2.0, 4.0])[:, None])


def test_pid_pixel_super_resolution_net_matches_plain_torch_statement():
    """PiD: checkpoint names of the released configuration, the max-period-10 timestep sinusoid, the NTK 2-D rotary table and the
    sin / cos pixel positions against their formulas, and the tiny net against a plain-torch forward (latent branch with gated
    injection every second block, dual-stream MMDiT blocks, per-pixel modulated PiT blocks, fold to the image)."""
    import math
    import torch.nn.functional as F
    from mojodiffusion_b200.models import pid as P
    torch.manual_seed(81)
    full = P.PidNet(P.PidConfig(), torch.float32, "meta")
    shapes = {k: tuple(v.shape) for k, v in full.state_dict().items()}
    for k, s in {"s_embedder.proj.weight": (1536, 768), "t_embedder.mlp.0.weight": (1536, 256), "y_embedder.proj.weight": (1536, 2304),
                 "y_embedder.norm.weight": (1536,), "y_pos_embedding": (1, 300, 1536), "lq_proj.latent_proj.0.weight": (512, 3, 3, 16),
                 "lq_proj.latent_proj.6.block.5.bias": (512,), "lq_proj.latent_proj.3.block.0.weight": (512,), "lq_proj.output_heads.6.weight": (1536, 512),
                 "lq_proj.gate_modules.0.content_proj.weight": (1536, 3072), "lq_proj.gate_modules.6.log_alpha": (),
                 "patch_blocks.13.adaLN_modulation_txt.0.weight": (9216, 1536), "patch_blocks.0.attn.qkv_y.weight": (4608, 1536),
                 "patch_blocks.0.attn.k_norm_x.weight": (64,), "patch_blocks.0.attn.proj_y.bias": (1536,), "patch_blocks.0.mlp_x.w3.weight": (4096, 1536),
                 "pixel_embedder.proj.weight": (16, 3), "pixel_blocks.1.adaLN_modulation.0.weight": (6 * 16 * 256, 1536),
                 "pixel_blocks.0.compress_to_attn.weight": (1152, 4096), "pixel_blocks.0.expand_from_attn.bias": (4096,),
                 "pixel_blocks.0.attn.qkv.weight": (3456, 1152), "pixel_blocks.0.attn.q_norm.weight": (72,), "pixel_blocks.0.mlp.fc1.weight": (64, 16),
                 "final_layer.norm.weight": (16,), "final_layer.linear.weight": (3, 16)}.items():
        assert shapes[k] == s, k
    assert len([k for k in shapes if k.startswith("lq_proj.output_heads.")]) == 14 and "patch_blocks.0.attn.qkv_x.bias" not in shapes
    e = P.pid_timestep_embedding(torch.tensor([0.7]), 8)
    assert torch.allclose(e[0, :4], torch.cos(0.7 * torch.exp(-math.log(10.0) * torch.arange(4).float() / 4))) and torch.allclose(e[0, 4:], torch.sin(0.7 * torch.exp(-math.log(10.0) * torch.arange(4).float() / 4)))
    cos, sin = P.ntk_rope_2d(64, 8, 16, 64, 64)
    th_h, th_w = 1.0e4 * (8 / 64) ** (32 / 30), 1.0e4 * (16 / 64) ** (32 / 30)
    pos = 3 * 16 + 5
    assert abs(float(cos[pos, 2 * 4]) - math.cos(16.0 * 5 / 15 / th_w ** (16 / 64))) < 1e-5 and abs(float(sin[pos, 2 * 4 + 1]) - math.sin(16.0 * 3 / 7 / th_h ** (16 / 64))) < 1e-5
    pp = P.sincos_pos_2d(16, 4, 6)
    om = 1.0 / 10000.0 ** (torch.arange(4).float() / 4)
    assert torch.allclose(pp[2 * 6 + 5], torch.cat(((5 * om).sin(), (5 * om).cos(), (2 * om).sin(), (2 * om).cos())), atol=1e-6)

    cfg = P.tiny_pid_config()
    m = P.PidNet(cfg, torch.float32).init_weights(7)
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() <= 1:
                p.add_(torch.randn_like(p) * 0.1)
    sd = m.state_dict()
    B, H, W, Lt, sigma = 2, 8, 12, 5, 0.3
    ps, D, G, hd = cfg.patch_size, cfg.hidden, cfg.groups, cfg.head_dim
    ph, pw = H // ps, W // ps
    L, P2, Cp = ph * pw, ps * ps, cfg.pixel_dim
    x, t, cap, lat = torch.randn(B, 3, H, W), torch.tensor([0.2, 0.9]), torch.randn(B, Lt, cfg.txt_dim), torch.randn(B, cfg.lq_channels, 1, 3)
    got = m(x, t, cap, lat, sigma)
    assert got.shape == x.shape

    lin = lambda v, n: F.linear(v, sd[n + ".weight"], sd.get(n + ".bias"))
    rms = lambda v, n: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6) * sd[n + ".weight"]
    conv = lambda v, n: F.conv2d(v, sd[n + ".weight"].permute(0, 3, 1, 2), sd[n + ".bias"], padding=1)
    h = conv(F.silu(conv(F.interpolate(lat, size=(ph, pw), mode="nearest"), "lq_proj.latent_proj.0")), "lq_proj.latent_proj.2")
    for i in range(3, 7):
        p = f"lq_proj.latent_proj.{i}.block."
        r = conv(F.silu(F.group_norm(h, 4, sd[p + "0.weight"], sd[p + "0.bias"], 1e-5)), p + "2")
        h = h + conv(F.silu(F.group_norm(r, 4, sd[p + "3.weight"], sd[p + "3.bias"], 1e-5)), p + "5")
    lq_tok = h.flatten(2).transpose(1, 2)
    s = lin(F.unfold(x, ps, stride=ps).transpose(1, 2), "s_embedder.proj")
    t_emb = lin(F.silu(lin(P.pid_timestep_embedding(t, cfg.freq_dim), "t_embedder.mlp.0")), "t_embedder.mlp.2")
    cond = F.silu(t_emb)[:, None]
    y = rms(lin(cap, "y_embedder.proj"), "y_embedder.norm") + sd["y_pos_embedding"][:, :Lt]

    def rope(v, table):                      # v [B, N, heads, d]
        rot = torch.complex(table[0], table[1])[None, :, None]
        return torch.view_as_real(torch.view_as_complex(v.reshape(*v.shape[:-1], -1, 2).contiguous()) * rot).flatten(-2)

    sdpa = lambda q, k, v: F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(-2)
    img_rope, txt_rope = P.ntk_rope_2d(hd, ph, pw, cfg.rope_ref, cfg.rope_ref), P.text_rope_1d(Lt, hd)
    for i in range(cfg.patch_depth):
        if i % 2 == 0:
            g = f"lq_proj.gate_modules.{i // 2}."
            lqf = lin(lq_tok, f"lq_proj.output_heads.{i // 2}")
            s = s + torch.sigmoid(lin(torch.cat((s, lqf), -1), g + "content_proj") - torch.exp(sd[g + "log_alpha"]) * sigma) * lqf
        p = f"patch_blocks.{i}."
        mx, my = lin(cond, p + "adaLN_modulation_img.0").chunk(6, -1), lin(cond, p + "adaLN_modulation_txt.0").chunk(6, -1)
        qx, kx, vx = lin((1 + mx[1]) * rms(s, p + "norm_x1") + mx[0], p + "attn.qkv_x").reshape(B, L, 3, G, hd).unbind(2)
        qy, ky, vy = lin((1 + my[1]) * rms(y, p + "norm_y1") + my[0], p + "attn.qkv_y").reshape(B, Lt, 3, G, hd).unbind(2)
        q = torch.cat((rope(rms(qy, p + "attn.q_norm_y"), txt_rope), rope(rms(qx, p + "attn.q_norm_x"), img_rope)), 1)
        k = torch.cat((rope(rms(ky, p + "attn.k_norm_y"), txt_rope), rope(rms(kx, p + "attn.k_norm_x"), img_rope)), 1)
        o = sdpa(q, k, torch.cat((vy, vx), 1))
        s = s + mx[2] * lin(o[:, Lt:], p + "attn.proj_x")
        y = y + my[2] * lin(o[:, :Lt], p + "attn.proj_y")
        ffn = lambda v_, n: lin(F.silu(lin(v_, n + ".w1")) * lin(v_, n + ".w3"), n + ".w2")
        s = s + mx[5] * ffn((1 + mx[4]) * rms(s, p + "norm_x2") + mx[3], p + "mlp_x")
        y = y + my[5] * ffn((1 + my[4]) * rms(y, p + "norm_y2") + my[3], p + "mlp_y")
    s_cond = F.silu(s + t_emb[:, None]).reshape(B * L, D)
    px = lin(x.permute(0, 2, 3, 1), "pixel_embedder.proj") + P.sincos_pos_2d(Cp, H, W).reshape(1, H, W, Cp)
    px = F.unfold(px.permute(0, 3, 1, 2), ps, stride=ps).reshape(B, Cp, P2, L).permute(0, 3, 2, 1).reshape(B * L, P2, Cp)
    pix_rope = P.ntk_rope_2d(cfg.pixel_attn // cfg.pixel_groups, ph, pw, cfg.rope_ref, cfg.rope_ref)
    for j in range(cfg.pixel_depth):
        p = f"pixel_blocks.{j}."
        sh1, sc1, g1, sh2, sc2, g2 = lin(s_cond, p + "adaLN_modulation.0").reshape(B * L, P2, 6 * Cp).chunk(6, -1)
        hcomp = lin((rms(px, p + "norm1") * (1 + sc1) + sh1).reshape(B * L, P2 * Cp), p + "compress_to_attn").reshape(B, L, -1)
        q, k, v = lin(hcomp, p + "attn.qkv").reshape(B, L, 3, cfg.pixel_groups, -1).unbind(2)
        a = lin(sdpa(rope(rms(q, p + "attn.q_norm"), pix_rope), rope(rms(k, p + "attn.k_norm"), pix_rope), v), p + "attn.proj")
        px = px + g1 * lin(a.reshape(B * L, -1), p + "expand_from_attn").reshape(B * L, P2, Cp)
        px = px + g2 * lin(F.gelu(lin(rms(px, p + "norm2") * (1 + sc2) + sh2, p + "mlp.fc1")), p + "mlp.fc2")
    out = lin(rms(px, "final_layer.norm"), "final_layer.linear").reshape(B, L, P2, 3).permute(0, 3, 2, 1).reshape(B, 3 * P2, L)
    want = F.fold(out, (H, W), ps, stride=ps)
    assert F.cosine_similarity(got.flatten(), want.flatten(), 0) > 0.99999 and (got - want).abs().max() < 2e-4 * want.abs().max() + 1e-5
    raw = {k: (v.permute(0, 3, 1, 2).contiguous() if v.dim() == 4 else v) for k, v in sd.items()}
    assert all(torch.equal(v, sd[k]) for k, v in P.remap_pid_keys(raw).items())
