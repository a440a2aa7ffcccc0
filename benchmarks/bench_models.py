#!/usr/bin/env python
"""Per-model-family step timing on one GPU at the real architecture sizes (random-init weights, synthetic inputs).

Each row is one denoise iteration (model forward + sampler update, no_grad, bf16 unless noted) or one training step,
device-timed with CUDA events after warm-up; every step streams far more weight bytes than the L2 holds. Counterpart of
the reference's per-model sampler smokes and trainer step reports (serenitymojo/docs/MODEL_RENDER_CAMPAIGN_2026-06-15.md,
BEAT_FLAME_SCOREBOARD_2026-06-10.md), which time the same loops on its hardware.

    python benchmarks/bench_models.py [--only ltx2,ltx2_fp8,ltx2_mxfp8,ltx2_vae,qwen,zimage,zimage_train,klein,klein_train,sdxl,sdxl_train,vae] [--tiny] [--json out.json]
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojodiffusion_b200 import ops  # noqa: E402
from mojodiffusion_b200.ops import native  # noqa: E402


def timed(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def nparams(m):
    return sum(p.numel() for p in m.parameters()) + sum(b.numel() for b in m.buffers())


def bench_ltx2(dev, tiny, steps, warmup, fp8, block_scaled=False):
    """LTX-2-shaped 48-layer video DiT, 6144 latent tokens (8 frames x 24 x 32), 256 context tokens, Euler update."""
    from mojodiffusion_b200.models.video_dit import VideoDiT, ltx2_config, tiny_video_dit_config
    cfg = tiny_video_dit_config() if tiny else ltx2_config()
    grid = (2, 4, 8) if tiny else (8, 24, 32)
    S = grid[0] * grid[1] * grid[2]
    m = VideoDiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    if fp8:
        m.to_fp8(0 if tiny else 4, None if tiny else 46, block_scaled=block_scaled)
    x = torch.randn(1, S, cfg.in_channels, device=dev)
    xb = x.to(torch.bfloat16)
    ctx = torch.randn(1, 16 if tiny else 256, cfg.context_dim, device=dev, dtype=torch.bfloat16)
    t = torch.full((1,), 0.7, device=dev)

    def step():
        with torch.no_grad():
            v = m(xb, ctx, t, grid)
            ops.cfg_euler(x, v, None, dt=-0.025, mode=0, x_bf16=xb)

    ms = timed(step, steps, warmup)
    return {"model": cfg.name + ((" mxfp8 (block-scaled) blocks 4-46" if block_scaled else " fp8 blocks 4-46") if fp8 else " bf16"), "params_b": nparams(m) / 1e9, "tokens": S,
            "metric": "denoise it/s", "ms_per_step": ms, "value": 1000.0 / ms}


def bench_qwen(dev, tiny, steps, warmup):
    """Qwen-Image-shaped 60-layer MMDiT (20 B parameters), 1024^2 = 4096 image tokens + 512 text tokens."""
    from mojodiffusion_b200.models.qwen_image import QwenImageDiT, qwen_image_config, tiny_qwen_image_config
    cfg = tiny_qwen_image_config() if tiny else qwen_image_config()
    hw, S_txt = ((8, 8), 16) if tiny else ((64, 64), 512)
    m = QwenImageDiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    x = torch.randn(1, hw[0] * hw[1], cfg.in_channels, device=dev)
    xb = x.to(torch.bfloat16)
    txt = torch.randn(1, S_txt, cfg.context_dim, device=dev, dtype=torch.bfloat16)
    t = torch.full((1,), 0.7, device=dev)

    def step():
        with torch.no_grad():
            v = m(xb, txt, t, hw)
            ops.cfg_euler(x, v, None, dt=-0.03, mode=0, x_bf16=xb)

    ms = timed(step, steps, warmup)
    return {"model": cfg.name, "params_b": nparams(m) / 1e9, "tokens": hw[0] * hw[1] + S_txt, "metric": "denoise it/s",
            "ms_per_step": ms, "value": 1000.0 / ms}


def bench_zimage(dev, tiny, steps, warmup, train):
    """Z-Image-shaped 6 B single-stream DiT: 1024^2 denoise (CFG: two forwards per step), or a 512^2 LoRA r16 step."""
    from mojodiffusion_b200.models.single_dit import SingleStreamDiT, tiny_single_dit_config, zimage_config
    cfg = tiny_single_dit_config() if tiny else zimage_config()
    side = 8 if tiny else (32 if train else 64)
    S_cap = 16 if tiny else 128
    m = SingleStreamDiT(cfg, torch.bfloat16, dev).init_weights(0)
    x = torch.randn(1, side * side, cfg.in_channels, device=dev)
    cap = torch.randn(1, S_cap, cfg.cap_dim, device=dev, dtype=torch.bfloat16)
    t = torch.full((1,), 0.6, device=dev)
    if not train:
        m.eval()
        xb = x.to(torch.bfloat16)
        neg = torch.randn_like(cap)

        def step():
            with torch.no_grad():
                vc = m(xb, cap, t, (side, side))
                vu = m(xb, neg, t, (side, side))
                ops.cfg_euler(x, vc, vu, dt=-0.03, s=3.5, mode=1, x_bf16=xb)

        ms = timed(step, steps, warmup)
        return {"model": cfg.name + " CFG 3.5 (2 forwards/step)", "params_b": nparams(m) / 1e9, "tokens": side * side + S_cap,
                "metric": "denoise it/s", "ms_per_step": ms, "value": 1000.0 / ms}
    from mojodiffusion_b200.training import lora as L
    from mojodiffusion_b200.training.optim import FusedAdamW
    from mojodiffusion_b200.models.layers import Linear
    names = {n: n for n, mod in m.named_modules() if n.startswith("layers.") and isinstance(mod, Linear) and "adaLN" not in n}
    slots = L.inject_lora_by_name(m, names, rank=16, alpha=16.0)
    params = L.lora_parameters(slots)
    opt = FusedAdamW(params, lr=1e-4, max_grad_norm=1.0)
    m.gradient_checkpointing = True
    m.train()
    eps = torch.randn_like(x)

    def step():
        opt.zero_grad(set_to_none=True)
        xt, target = ops.flow_match(x, eps, t)
        pred = m(xt.to(torch.bfloat16), cap, t, (side, side))
        loss = ops.mse_loss(pred, target)
        loss.backward()
        opt.step()

    ms = timed(step, steps, warmup)
    return {"model": cfg.name + f" LoRA r16 ({len(slots)} adapters), {side * 16}^2, grad ckpt", "params_b": nparams(m) / 1e9,
            "tokens": side * side + S_cap, "metric": "train samples/s", "ms_per_step": ms, "value": 1000.0 / ms}


def bench_krea2(dev, tiny, steps, warmup):
    """Krea-2-shaped 12 B single-stream MMDiT: 1024^2 denoise with guidance (two forwards per step; 114 and 5 text tokens of
    twelve stacked encoder layers each, as in the reference's sample run)."""
    import dataclasses
    from mojodiffusion_b200.models.krea2 import Krea2Config, Krea2DiT, krea2_positions, tiny_krea2_config
    cfg = dataclasses.replace(tiny_krea2_config(), features=256, txtdim=128) if tiny else Krea2Config()
    g = 8 if tiny else 64
    lt_c, lt_u = (16, 8) if tiny else (114, 5)
    m = Krea2DiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    x = torch.randn(1, g * g, cfg.patch_dim, device=dev)
    xb = x.to(torch.bfloat16)
    ctx_c = torch.randn(1, lt_c, cfg.txtlayers, cfg.txtdim, device=dev, dtype=torch.bfloat16)
    ctx_u = torch.randn(1, lt_u, cfg.txtlayers, cfg.txtdim, device=dev, dtype=torch.bfloat16)
    pos_c, pos_u = krea2_positions(lt_c, g, g, dev), krea2_positions(lt_u, g, g, dev)
    t = torch.full((1,), 0.6, device=dev)

    def step():
        with torch.no_grad():
            vc = m(xb, ctx_c, t, pos_c)
            vu = m(xb, ctx_u, t, pos_u)
            ops.cfg_euler(x, vc, vu, dt=-0.03, s=4.5, mode=2, x_bf16=xb)          # v_c + 4.5 (v_c - v_u)

    ms = timed(step, steps, warmup)
    return {"model": cfg.name + " guidance 4.5 (2 forwards/step)", "params_b": nparams(m) / 1e9, "tokens": g * g + lt_c,
            "metric": "denoise it/s", "ms_per_step": ms, "value": 1000.0 / ms}


def bench_krea2_train(dev, tiny, steps, warmup):
    """Krea-2-shaped 12.8 B model, LoRA r16 on the eight projections of every single-stream block (the reference's surface),
    512^2 (1024 image + 114 text tokens), batch 1, per-block recompute, AdamW."""
    import dataclasses
    from mojodiffusion_b200.models.krea2 import Krea2Config, Krea2DiT, krea2_positions, tiny_krea2_config
    from mojodiffusion_b200.training import lora as L
    from mojodiffusion_b200.training.optim import FusedAdamW
    cfg = dataclasses.replace(tiny_krea2_config(), features=256, txtdim=128) if tiny else Krea2Config()
    g, lt = (8, 16) if tiny else (32, 114)
    m = Krea2DiT(cfg, torch.bfloat16, dev).init_weights(0)
    slots = L.inject_krea2_lora(m, rank=16, alpha=16.0)
    opt = FusedAdamW(L.lora_parameters(slots), lr=1e-4, max_grad_norm=1.0)
    m.gradient_checkpointing = True
    m.train()
    x0, eps = torch.randn(1, g * g, cfg.patch_dim, device=dev), torch.randn(1, g * g, cfg.patch_dim, device=dev)
    ctx = torch.randn(1, lt, cfg.txtlayers, cfg.txtdim, device=dev, dtype=torch.bfloat16)
    pos = krea2_positions(lt, g, g, dev)
    t = torch.full((1,), 0.6, device=dev)

    def step():
        opt.zero_grad(set_to_none=True)
        xt, target = ops.flow_match(x0, eps, t)
        ops.mse_loss(m(xt.to(torch.bfloat16), ctx, t, pos), target).backward()
        opt.step()

    ms = timed(step, steps, warmup)
    return {"model": cfg.name + f" LoRA r16 ({len(slots)} adapters), {g * 16}^2, grad ckpt", "params_b": nparams(m) / 1e9,
            "tokens": g * g + lt, "metric": "train samples/s", "ms_per_step": ms, "value": 1000.0 / ms}


def _row(name, m, tokens, ms, what="denoise it/s"):
    return {"model": name, "params_b": nparams(m) / 1e9, "tokens": tokens, "metric": what, "ms_per_step": ms, "value": 1000.0 / ms}


def bench_lens(dev, tiny, steps, warmup):
    """Lens-shaped 48-block double-stream DiT (width 1536, 24 x 64), 1024^2 (4096 image + 415 text tokens), guidance."""
    from mojodiffusion_b200.models.lens import LensConfig, LensDiT, tiny_lens_config
    cfg = tiny_lens_config() if tiny else LensConfig()
    g, lt = (8, 16) if tiny else (64, 415)
    m = LensDiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    x = torch.randn(1, g * g, cfg.in_channels, device=dev)
    xb = x.to(torch.bfloat16)
    tc, tu = (torch.randn(1, lt, cfg.text_layers, cfg.text_hidden, device=dev, dtype=torch.bfloat16) for _ in range(2))
    t = torch.full((1,), 0.6, device=dev)

    def step():
        with torch.no_grad():
            ops.cfg_euler(x, m(xb, tc, t, (g, g)), m(xb, tu, t, (g, g)), dt=-0.03, s=5.0, mode=1, x_bf16=xb)

    return _row(cfg.name + " guidance 5 (2 forwards/step)", m, g * g + lt, timed(step, steps, warmup))


def bench_ideogram4(dev, tiny, steps, warmup):
    """Ideogram-4-shaped 34-block single-stream DiT (width 4608, 18 heads of 256: attention on the library kernel), 1024^2:
    4096 image + 512 text positions in one sequence, one forward per step."""
    from mojodiffusion_b200.models.ideogram4 import IND_IMAGE, IND_TEXT, Ideogram4Config, Ideogram4DiT, tiny_ideogram4_config
    cfg = tiny_ideogram4_config() if tiny else Ideogram4Config()
    g, lt = (8, 16) if tiny else (64, 512)
    L = lt + g * g
    m = Ideogram4DiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    x = torch.randn(1, L, cfg.in_channels, device=dev, dtype=torch.bfloat16)
    llm = torch.randn(1, L, cfg.llm_dim, device=dev, dtype=torch.bfloat16)
    ind = torch.tensor([[IND_TEXT] * lt + [IND_IMAGE] * (g * g)], device=dev)
    pos = torch.zeros(L, 3)
    pos[:lt, 0] = torch.arange(lt).float()
    pos[lt:, 1] = torch.arange(g).float().repeat_interleave(g)
    pos[lt:, 2] = torch.arange(g).float().repeat(g)
    pos = pos.to(dev)
    t = torch.full((1,), 0.6, device=dev)

    def step():
        with torch.no_grad():
            m(x, llm, t, ind, pos)

    return _row(cfg.name + " (1 forward/step)", m, L, timed(step, steps, warmup))


def bench_more(dev, tiny, steps, warmup, which):
    """One forward per step of a family that has no packed fast path, at its real size (``which``: hunyuan15, kandinsky5, cosmos,
    wan_vace, nucleus, acestep, hidream_o1). Video grids hold 6144 tokens, image grids 4096."""
    bf = torch.bfloat16
    rn = lambda *sh, dtype=bf: torch.randn(*sh, device=dev, dtype=dtype)
    t = torch.full((1,), 0.6, device=dev)
    if which == "hunyuan15":
        from mojodiffusion_b200.models.hunyuan15 import Hunyuan15Config, Hunyuan15DiT, tiny_hunyuan15_config
        cfg = tiny_hunyuan15_config() if tiny else Hunyuan15Config()
        m = Hunyuan15DiT(cfg, bf, dev).init_weights(0).eval()
        f, h, w = (2, 4, 8) if tiny else (4, 32, 48)
        args, tokens = (rn(1, cfg.in_channels, f, h, w), rn(1, 16 if tiny else 256, cfg.hidden), t), f * h * w
    elif which == "kandinsky5":
        from mojodiffusion_b200.models.kandinsky5 import Kandinsky5Config, Kandinsky5DiT, tiny_kandinsky5_config
        cfg = tiny_kandinsky5_config() if tiny else Kandinsky5Config()
        m = Kandinsky5DiT(cfg, bf, dev).init_weights(0).eval()
        f, h, w = (2, 8, 8) if tiny else (4, 64, 96)
        args, tokens = (rn(1, cfg.in_visual_dim, f, h, w), rn(1, 16 if tiny else 256, cfg.in_text_dim), rn(1, cfg.in_text_dim2),
                        torch.full((1,), 417.0, device=dev)), f * (h // 2) * (w // 2)
    elif which == "cosmos":
        from mojodiffusion_b200.models.cosmos import CosmosConfig, CosmosDiT, tiny_cosmos_config
        cfg = tiny_cosmos_config() if tiny else CosmosConfig()
        m = CosmosDiT(cfg, bf, dev).init_weights(0).eval()
        f, h, w = (2, 8, 8) if tiny else (4, 64, 96)
        args, tokens = (rn(1, cfg.in_channels, f, h, w), rn(1, 16 if tiny else 512, cfg.text_in_dim), t), f * (h // 2) * (w // 2)
    elif which == "wan_vace":
        from mojodiffusion_b200.models.wan import WanVaceDiT, tiny_wan_vace_config, wan21_vace_14b_config
        cfg = tiny_wan_vace_config() if tiny else wan21_vace_14b_config()
        m = WanVaceDiT(cfg, bf, dev).init_weights(0).eval()
        f, h, w = (2, 8, 8) if tiny else (4, 64, 96)
        ctl = rn(1, cfg.vace_in_dim, f, h, w)
        args, tokens = (rn(1, cfg.in_dim, f, h, w), rn(1, 16 if tiny else 512, cfg.text_dim), t), f * (h // 2) * (w // 2)
        fwd = lambda: m(*args, control=ctl)
    elif which == "nucleus":
        from mojodiffusion_b200.models.nucleus import NucleusConfig, NucleusDiT, tiny_nucleus_config
        cfg = tiny_nucleus_config() if tiny else NucleusConfig()
        m = NucleusDiT(cfg, bf, dev).init_weights(0).eval()
        g = 8 if tiny else 64
        args, tokens = (rn(1, g * g, cfg.in_channels), rn(1, 16 if tiny else 256, cfg.joint_dim), t), g * g
        fwd = lambda: m(*args, grid=(1, g, g))
    elif which == "acestep":
        import dataclasses
        from mojodiffusion_b200.models.acestep import AceStepConfig, AceStepDiT, tiny_acestep_config
        cfg = dataclasses.replace(tiny_acestep_config(), hidden=256, head_dim=64) if tiny else AceStepConfig()
        m = AceStepDiT(cfg, bf, dev).init_weights(0).eval()
        T = 32 if tiny else 3000                                                  # 2 minutes of audio at 25 latent frames / s
        args, tokens = (rn(1, T, cfg.acoustic_dim), rn(1, T, cfg.in_channels - cfg.acoustic_dim), rn(1, 8 if tiny else 256, cfg.hidden), t,
                        torch.full((1,), 0.2, device=dev)), T // cfg.patch
    else:
        import dataclasses
        from mojodiffusion_b200.models.hidream_o1 import HiDreamO1, HiDreamO1Config, build_mrope_positions, tiny_hidream_o1_config
        cfg = tiny_hidream_o1_config() if tiny else HiDreamO1Config()
        if tiny:
            cfg = dataclasses.replace(cfg, spine=dataclasses.replace(cfg.spine, hidden_size=256, head_dim=64))
        m = HiDreamO1(cfg, bf, dev).init_weights(0).eval()
        g, lt = (4, 5) if tiny else (32, 64)
        ids = [1] * (lt - 2) + [cfg.tms_token_id, cfg.vision_start_token_id]
        pos = build_mrope_positions(ids + [cfg.image_token_id] * (g * g), cfg.image_token_id, g, g, lt + 8)
        patches = rn(1, g * g, cfg.patch_dim)
        tokens = g * g + lt
        fwd = lambda: m(ids, patches, pos, lt, 0.4)
    if which not in ("wan_vace", "nucleus", "hidream_o1"):
        fwd = lambda: m(*args)

    def step():
        with torch.no_grad():
            fwd()

    return _row(getattr(cfg, "name", which) + " (1 forward/step)", m, tokens, timed(step, steps, warmup))


def bench_boogu(dev, tiny, steps, warmup):
    """Boogu-Image-shaped DiT (width 3360, 28 / 7 heads of 120; 2 + 2 refiner, 8 double, 32 single blocks), 1024^2, guidance."""
    from mojodiffusion_b200.models.boogu import BooguConfig, BooguDiT, tiny_boogu_config
    cfg = tiny_boogu_config() if tiny else BooguConfig()
    side, lt = (16, 16) if tiny else (128, 256)
    m = BooguDiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    x = torch.randn(1, cfg.in_channels, side, side, device=dev)
    tc, tu = (torch.randn(1, lt, cfg.instruction_dim, device=dev, dtype=torch.bfloat16) for _ in range(2))
    t = torch.full((1,), 0.6, device=dev)

    def step():
        with torch.no_grad():
            vc, vu = m(x, tc, t), m(x, tu, t)
            x.add_((vu + 4.0 * (vc - vu)).float(), alpha=-0.03)

    return _row(cfg.name + " guidance 4 (2 forwards/step)", m, (side // 2) ** 2 + lt, timed(step, steps, warmup))


def bench_magihuman(dev, tiny, steps, warmup):
    """MagiHuman-shaped 15 B DiT: 4096 video + 64 audio + 64 text tokens in one stream, one forward per (distilled) step."""
    import dataclasses
    from mojodiffusion_b200.models.magihuman import MagiHumanConfig, MagiHumanDiT, tiny_magihuman_config
    cfg = dataclasses.replace(tiny_magihuman_config(), hidden_size=256, head_dim=64, rope_dim=48, rope_bands=8) if tiny else MagiHumanConfig()
    f, h, w = (2, 4, 4) if tiny else (4, 32, 32)
    V, A, T = f * h * w, (8 if tiny else 64), (8 if tiny else 64)
    m = MagiHumanDiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    coords = torch.cat((torch.stack(torch.meshgrid(torch.arange(float(f)), torch.arange(float(h)), torch.arange(float(w)), indexing="ij"), -1).reshape(V, 3),
                        torch.stack((torch.arange(A + T).float(), torch.zeros(A + T), torch.zeros(A + T)), 1)), 0)
    coords = torch.cat((coords, torch.tensor([[float(f), float(h), float(w), float(f), float(h), float(w)]]).expand(V + A + T, 6)), 1).to(dev)
    xv, xa, xt = (torch.randn(n, d, device=dev, dtype=torch.bfloat16) for n, d in ((V, cfg.video_in), (A, cfg.audio_in), (T, cfg.text_in)))

    def step():
        m(xv, xa, xt, coords)

    return _row(cfg.name + " (1 forward/step)", m, V + A + T, timed(step, steps, warmup))


def bench_sensenova(dev, tiny, steps, warmup):
    """SenseNova-U1-shaped 8 B (two weight sets) pixel model, 1024^2: 1024 image tokens over a cached 64-token prompt, guidance."""
    import dataclasses
    from mojodiffusion_b200.models.sensenova_u1 import SenseNovaU1, SenseNovaU1Config, tiny_sensenova_u1_config
    cfg = dataclasses.replace(tiny_sensenova_u1_config(), head_dim=64) if tiny else SenseNovaU1Config()
    side, lt = (32, 8) if tiny else (1024, 64)
    m = SenseNovaU1(cfg, torch.bfloat16, dev).init_weights(0).eval()
    ids_c, ids_u = list(range(1, lt + 1)), list(range(1, 9))
    cc, cu = m.forward_und(ids_c), m.forward_und(ids_u)
    img = torch.randn(1, 3, side, side, device=dev, dtype=torch.bfloat16)

    def step():
        m.predict_clean(img, 0.4, cc, len(ids_c))
        m.predict_clean(img, 0.4, cu, len(ids_u))

    return _row(cfg.name + " guidance (2 image passes/step, prompt cached)", m, (side // (cfg.patch_size * cfg.merge_size)) ** 2 + lt, timed(step, steps, warmup))


def bench_nava(dev, tiny, steps, warmup):
    """NAVA-shaped audio + video DiT (10 double + 20 joint Wan blocks, width 3072), 832 x 480 x 17 frames: 1950 video + 34 audio tokens."""
    from mojodiffusion_b200.models.nava import NavaConfig, NavaDiT, tiny_nava_config
    cfg = tiny_nava_config() if tiny else NavaConfig()
    F_, Hh, Ww, Na, Lt = (2, 8, 8, 6, 8) if tiny else (5, 30, 52, 34, 64)
    m = NavaDiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    v, a = torch.randn(1, cfg.in_dim, F_, Hh, Ww, device=dev), torch.randn(1, Na, cfg.audio_dim, device=dev)
    tc, tu = (torch.randn(1, Lt, cfg.text_dim, device=dev, dtype=torch.bfloat16) for _ in range(2))
    t = torch.full((1,), 0.5, device=dev)

    def step():
        m(v, a, tc, t)
        m(v, a, tu, t)

    return _row(cfg.name + " guidance (2 forwards/step)", m, F_ * (Hh // 2) * (Ww // 2) + Na, timed(step, steps, warmup))


def bench_pid(dev, tiny, steps, warmup):
    """PiD super-resolution decoder at 1024^2 output (4096 patches, 64-token caption), one forward per distilled step."""
    from mojodiffusion_b200.models.pid import PidConfig, PidNet, tiny_pid_config
    cfg = tiny_pid_config() if tiny else PidConfig()
    side, lt = (32, 8) if tiny else (1024, 64)
    m = PidNet(cfg, torch.bfloat16, dev).init_weights(0).eval()
    x = torch.randn(1, 3, side, side, device=dev)
    cap = torch.randn(1, lt, cfg.txt_dim, device=dev, dtype=torch.bfloat16)
    lat = torch.randn(1, cfg.lq_channels, side // 32, side // 32, device=dev)
    t = torch.full((1,), 0.7, device=dev)

    def step():
        m(x, t, cap, lat, 0.0)

    return _row(cfg.name + " (1 forward/step)", m, (side // cfg.patch_size) ** 2 + lt, timed(step, steps, warmup))


def bench_klein(dev, tiny, steps, warmup, train):
    """FLUX.2 Klein-9B-shaped MMDiT: 1024^2 denoise (4096 + 512 tokens), or the reference's headline training case:
    LoRA r16 on every block projection, 512^2 (1024 image + 512 text tokens = 1536), batch 1, gradient checkpointing."""
    from mojodiffusion_b200.models.flux2 import Flux2DiT, klein_9b_config, tiny_flux2_config
    cfg = tiny_flux2_config() if tiny else klein_9b_config()
    side = 8 if tiny else (32 if train else 64)
    S_txt = 16 if tiny else 512
    m = Flux2DiT(cfg, torch.bfloat16, dev).init_weights(0)
    x = torch.randn(1, side * side, cfg.in_channels, device=dev)
    txt = torch.randn(1, S_txt, cfg.context_dim, device=dev, dtype=torch.bfloat16)
    t = torch.full((1,), 0.6, device=dev)
    if not train:
        m.eval()
        xb = x.to(torch.bfloat16)

        def step():
            with torch.no_grad():
                v = m(xb, txt, t, (side, side))
                ops.cfg_euler(x, v, None, dt=-0.03, mode=0, x_bf16=xb)

        ms = timed(step, steps, warmup)
        return {"model": cfg.name, "params_b": nparams(m) / 1e9, "tokens": side * side + S_txt, "metric": "denoise it/s",
                "ms_per_step": ms, "value": 1000.0 / ms}
    from mojodiffusion_b200.training import lora as L
    from mojodiffusion_b200.training.optim import FusedAdamW
    slots = L.inject_lora_by_name(m, {n: n for n in m.lora_target_names()}, rank=16, alpha=16.0)
    params = L.lora_parameters(slots)
    opt = FusedAdamW(params, lr=1e-4, max_grad_norm=1.0)
    m.gradient_checkpointing = True
    m.train()
    eps = torch.randn_like(x)

    def step():
        opt.zero_grad(set_to_none=True)
        xt, target = ops.flow_match(x, eps, t)
        loss = ops.mse_loss(m(xt.to(torch.bfloat16), txt, t, (side, side)), target)
        loss.backward()
        opt.step()

    ms = timed(step, steps, warmup)
    return {"model": cfg.name + f" LoRA r16 ({len(slots)} adapters), 512^2, S=1536, batch 1, grad ckpt",
            "params_b": nparams(m) / 1e9, "tokens": side * side + S_txt, "metric": "train samples/s", "ms_per_step": ms,
            "value": 1000.0 / ms}


def bench_sdxl(dev, tiny, steps, warmup):
    """SDXL UNet, 1024^2 (128 x 128 latent), eps-prediction Euler step with CFG (batch of 2 = cond + uncond)."""
    from mojodiffusion_b200.models.unet import UNet, sdxl_config, tiny_unet_config
    cfg = tiny_unet_config() if tiny else sdxl_config()
    side = 16 if tiny else 128
    m = UNet(cfg, torch.bfloat16, dev).init_weights(0).eval()
    x = torch.randn(2, cfg.in_channels, side, side, device=dev)
    ctx = torch.randn(2, 77, cfg.context_dim, device=dev, dtype=torch.bfloat16)
    y = torch.randn(2, cfg.adm_in_channels, device=dev, dtype=torch.bfloat16)
    ts = torch.full((2,), 500.0, device=dev)

    def step():
        with torch.no_grad():
            eps = m(x.to(torch.bfloat16), ts, ctx, y).float()
            e = eps[1:] + 7.0 * (eps[:1] - eps[1:])
            x.add_(e.expand_as(x), alpha=-0.01)

    ms = timed(step, steps, warmup)
    return {"model": cfg.name, "params_b": nparams(m) / 1e9, "tokens": side * side,
            "metric": "denoise it/s (CFG, cond+uncond batched)", "ms_per_step": ms, "value": 1000.0 / ms}


def bench_vae(dev, tiny, steps, warmup):
    """FLUX VAE decode of one 1024^2 image (128 x 128 x 16 latent)."""
    from mojodiffusion_b200.models.vae import AutoencoderKL, flux_vae_config, tiny_vae_config
    cfg = tiny_vae_config() if tiny else flux_vae_config()
    side = 16 if tiny else 128
    m = AutoencoderKL(cfg, torch.bfloat16, dev, with_encoder=False).init_weights(0).eval()
    z = torch.randn(1, cfg.z_channels, side, side, device=dev)

    def step():
        with torch.no_grad():
            m.decode(z)

    ms = timed(step, steps, warmup)
    return {"model": "flux-vae decode" if not tiny else "tiny-vae decode", "params_b": nparams(m) / 1e9,
            "tokens": side * side, "metric": "images/s", "ms_per_step": ms, "value": 1000.0 / ms}


def bench_ltx2_vae(dev, tiny, steps, warmup):
    """LTX-2 video VAE decode of a 768 x 512, 121-frame clip (latent 128 x 16 x 16 x 24)."""
    from mojodiffusion_b200.models.video_vae import VideoVAE, ltx2_vae_config, tiny_video_vae_config
    cfg = tiny_video_vae_config() if tiny else ltx2_vae_config()
    shape = (1, cfg.latent_channels, 2, 4, 4) if tiny else (1, cfg.latent_channels, 16, 16, 24)
    m = VideoVAE(cfg, torch.bfloat16, dev).init_weights(0).eval()
    z = torch.randn(*shape, device=dev)
    out = {}

    def step():
        with torch.no_grad():
            out["v"] = m.decode(z)

    ms = timed(step, steps, warmup)
    v = out["v"]
    return {"model": cfg.name + " decode", "params_b": nparams(m) / 1e9, "tokens": int(z.numel() // z.shape[1]), "frames": int(v.shape[2]),
            "height": int(v.shape[3]), "width": int(v.shape[4]), "metric": "clips/s", "ms_per_step": ms, "value": 1000.0 / ms}


def bench_sdxl_train(dev, tiny, steps, warmup):
    """SDXL UNet LoRA (rank 16) train step at 1024^2 (128 x 128 latent, batch 1): eps target over the DDPM grid, forward +
    backward on the package's convolution / GroupNorm / attention / GEMM kernels, fused AdamW on the adapters."""
    from mojodiffusion_b200.models.unet import UNet, sdxl_config, tiny_unet_config
    from mojodiffusion_b200.training import lora as L
    from mojodiffusion_b200.training.optim import FusedAdamW
    cfg = tiny_unet_config() if tiny else sdxl_config()
    side = 16 if tiny else 128
    m = UNet(cfg, torch.bfloat16, dev).init_weights(0)
    slots = L.inject_sdxl_lora(m, rank=4 if tiny else 16, alpha=16.0)
    params = L.lora_parameters(slots)
    opt = FusedAdamW(params, lr=1e-4, max_grad_norm=1.0)
    x0 = torch.randn(1, cfg.in_channels, side, side, device=dev)
    ctx = torch.randn(1, 77, cfg.context_dim, device=dev, dtype=torch.bfloat16)
    y = torch.randn(1, cfg.adm_in_channels, device=dev, dtype=torch.bfloat16)
    ts = torch.full((1,), 500.0, device=dev)
    calls = {"n": 0}
    orig = torch.nn.functional.conv2d

    def spy(*a, **k):
        calls["n"] += 1
        return orig(*a, **k)
    torch.nn.functional.conv2d = spy

    def step():
        noise = torch.randn_like(x0)
        xt = (0.7 * x0 + 0.714 * noise).to(torch.bfloat16)
        opt.zero_grad(set_to_none=True)
        loss = (m(xt, ts, ctx, y).float() - noise).square().mean()
        loss.backward()
        opt.step()

    try:
        ms = timed(step, steps, warmup)
    finally:
        torch.nn.functional.conv2d = orig
    return {"model": cfg.name + " LoRA r16 train", "params_b": nparams(m) / 1e9, "tokens": side * side, "metric": "samples/s",
            "library_conv_calls": calls["n"], "ms_per_step": ms, "value": 1000.0 / ms}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="ltx2,ltx2_fp8,qwen,zimage,zimage_train,klein,klein_train,sdxl,vae")
    ap.add_argument("--tiny", action="store_true", help="tiny architectures (seconds; for checking the script)")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    native.load(True)
    table = {
        "ltx2": lambda: bench_ltx2(dev, args.tiny, args.steps, args.warmup, False),
        "ltx2_fp8": lambda: bench_ltx2(dev, args.tiny, args.steps, args.warmup, True),
        "qwen": lambda: bench_qwen(dev, args.tiny, args.steps, args.warmup),
        "zimage": lambda: bench_zimage(dev, args.tiny, args.steps, args.warmup, False),
        "zimage_train": lambda: bench_zimage(dev, args.tiny, args.steps, args.warmup, True),
        "klein": lambda: bench_klein(dev, args.tiny, args.steps, args.warmup, False),
        "klein_train": lambda: bench_klein(dev, args.tiny, args.steps, args.warmup, True),
        "sdxl": lambda: bench_sdxl(dev, args.tiny, args.steps, args.warmup),
        "vae": lambda: bench_vae(dev, args.tiny, args.steps, args.warmup),
        "ltx2_mxfp8": lambda: bench_ltx2(dev, args.tiny, args.steps, args.warmup, True, True),
        "ltx2_vae": lambda: bench_ltx2_vae(dev, args.tiny, args.steps, args.warmup),
        "sdxl_train": lambda: bench_sdxl_train(dev, args.tiny, args.steps, args.warmup),
        "krea2": lambda: bench_krea2(dev, args.tiny, args.steps, args.warmup),
        "krea2_train": lambda: bench_krea2_train(dev, args.tiny, args.steps, args.warmup),
        "lens": lambda: bench_lens(dev, args.tiny, args.steps, args.warmup),
        "boogu": lambda: bench_boogu(dev, args.tiny, args.steps, args.warmup),
        **{k: (lambda k=k: bench_more(dev, args.tiny, args.steps, args.warmup, k))
           for k in ("hunyuan15", "kandinsky5", "cosmos", "wan_vace", "nucleus", "acestep", "hidream_o1")},
        "ideogram4": lambda: bench_ideogram4(dev, args.tiny, args.steps, args.warmup),
        "magihuman": lambda: bench_magihuman(dev, args.tiny, args.steps, args.warmup),
        "sensenova": lambda: bench_sensenova(dev, args.tiny, args.steps, args.warmup),
        "nava": lambda: bench_nava(dev, args.tiny, args.steps, args.warmup),
        "pid": lambda: bench_pid(dev, args.tiny, args.steps, args.warmup),
    }
    rows = []
    for name in args.only.split(","):
        t0 = time.time()
        row = table[name]()
        native.check_status()
        row["case"] = name
        row["peak_gib"] = torch.cuda.max_memory_allocated() / 2 ** 30
        row["wall_s_incl_init"] = time.time() - t0
        rows.append(row)
        print(json.dumps(row), flush=True)
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
    if args.json:
        json.dump(rows, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
