"""CPU tests for the training extras: loss levers, optimizer family, LyCORIS adapters, EMA schedule, buckets, features,
dataset cache, full-finetune state contract, progress line, board, cadence / resume loop."""
import io
import math
import os
import sqlite3

import pytest
import torch

from mojodiffusion_b200.io.config import TrainConfig
from mojodiffusion_b200.training import buckets, features, full_finetune, loop, losses, lycoris, optim_extra
from mojodiffusion_b200.training.board import BoardWriter
from mojodiffusion_b200.training.dataset import BatchLoader, LatentCache, write_sample
from mojodiffusion_b200.training.ema import EMA, ema_decay_at_step
from mojodiffusion_b200.training.optim import FusedAdamW
from mojodiffusion_b200.training.progress import ProgressDisplay, format_hms


def test_loss_levers_defaults_and_weights():
    torch.manual_seed(0)
    p, t = torch.randn(4, 8, 16), torch.randn(4, 8, 16)
    base = torch.nn.functional.mse_loss(p, t)
    assert torch.allclose(losses.diffusion_loss(p, t), base, atol=1e-6)
    assert torch.allclose(losses.diffusion_loss(p, t, loss_fn="huber", huber_delta=1.0),
                          torch.nn.functional.huber_loss(p, t, delta=1.0), atol=1e-6)
    assert torch.allclose(losses.diffusion_loss(p, t, loss_fn="smooth_l1", smooth_l1_beta=0.5),
                          torch.nn.functional.smooth_l1_loss(p, t, beta=0.5), atol=1e-6)
    sig = torch.tensor([0.1, 0.5, 0.9, 0.5])
    snr = ((1 - sig) / sig) ** 2
    w = losses.min_snr_weight(sig, 5.0)
    assert torch.allclose(w, torch.minimum(snr, torch.tensor(5.0)) / (snr + 1))
    assert torch.allclose(losses.debiased_weight(sig), 1 / torch.sqrt(snr + 1))
    per = ((p - t) ** 2).reshape(4, -1).mean(1)
    assert torch.allclose(losses.diffusion_loss(p, t, sigma=sig, min_snr_gamma=5.0), (per * w).mean(), atol=1e-6)
    mask = torch.zeros(4, 8, 1)
    mask[:, :4] = 1
    exp = ((p - t) ** 2)[:, :4].reshape(4, -1).mean(1).mean()
    assert torch.allclose(losses.diffusion_loss(p, t, mask=mask), exp, atol=1e-6)


@pytest.mark.parametrize("name", ["ADAMW", "ADAMW_8BIT", "LION", "STABLEADAMW", "ADAFACTOR", "PRODIGY",
                                  "SCHEDULE_FREE_ADAMW", "SGD"])
def test_optimizer_family_descends(name):
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(8, 8))
    tgt = torch.randn(8, 8)
    opt = optim_extra.create_optimizer(name, [w], 1.0 if name == "PRODIGY" else 1e-2)
    first = None
    for _ in range(60):
        opt.zero_grad()
        loss = ((w - tgt) ** 2).mean()
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
    assert loss.item() < first * 0.8
    with pytest.raises(ValueError):
        optim_extra.create_optimizer("NOPE", [w], 1e-3)


def test_lion_and_8bit_match_formulas():
    w = torch.nn.Parameter(torch.tensor([1.0, -2.0, 3.0]))
    w.grad = torch.tensor([0.5, -0.1, 0.0])
    optim_extra.Lion([w], lr=0.1, betas=(0.9, 0.99), weight_decay=0.0).step()
    assert torch.allclose(w.detach(), torch.tensor([0.9, -1.9, 3.0]))
    code = optim_extra.dynamic_map(True)
    assert code.numel() == 256 and bool((code[1:] >= code[:-1]).all()) and code.max() == 1.0
    x = torch.randn(1000) * 0.02
    q, a = optim_extra.quantize_blockwise(x, code)
    y = optim_extra.dequantize_blockwise(q, a, code, x.shape)
    assert q.dtype == torch.uint8 and a.numel() == 4
    assert float((x - y).abs().max() / x.abs().max()) < 0.02
    # 8-bit AdamW tracks fp32 AdamW closely over a few steps
    torch.manual_seed(1)
    p0 = torch.randn(512)
    a8, a32 = torch.nn.Parameter(p0.clone()), torch.nn.Parameter(p0.clone())
    o8, o32 = optim_extra.AdamW8bit([a8], 1e-2), FusedAdamW([a32], 1e-2)
    for i in range(5):
        g = torch.randn(512, generator=torch.Generator().manual_seed(i))
        a8.grad, a32.grad = g.clone(), g.clone()
        o8.step()
        o32.step()
    assert float((a8 - a32).detach().abs().max()) < 5e-3


@pytest.mark.parametrize("algo,kw", [("loha", dict(rank=4, alpha=4)), ("lokr", dict(rank=2, alpha=2, factor=4)),
                                     ("lokr", dict(rank=1, alpha=1, factor=2, decompose_both=True)), ("full", {}),
                                     ("dora", dict(rank=4, alpha=4)), ("oft", dict(block=4)), ("boft", dict(block=4))])
def test_lycoris_identity_at_init_and_grad_coverage(algo, kw):
    torch.manual_seed(0)
    W, x = torch.randn(16, 12), torch.randn(5, 12)
    if algo == "dora":
        kw = dict(kw, base_weight=W)
    ad = lycoris.ALGOS[algo](16, 12, **kw)
    assert float((ad.effective_weight(W) - W).abs().max()) < 1e-6
    opt = torch.optim.SGD(ad.parameters(), lr=0.05)
    for _ in range(2):
        opt.zero_grad()
        (x @ ad.effective_weight(W).T).pow(2).sum().backward()
        opt.step()
    cov = features.GradCoverage().check(ad.named_parameters(), step=1)
    assert cov.ok, (cov.dead, cov.nonfinite)
    if algo in ("oft", "boft"):
        We = ad.effective_weight(W)
        assert torch.allclose(We.T @ We, W.T @ W, atol=1e-4)      # rotation of the output axis keeps W^T W
    keys = ad.state_tensors("p")
    assert "p.alpha" in keys or algo == "full"


def test_lycoris_formulas_and_keys():
    torch.manual_seed(0)
    l = lycoris.LoHa(6, 4, rank=2, alpha=1.0)
    with torch.no_grad():
        l.hada_w2_a.normal_()
    exp = (l.hada_w1_a @ l.hada_w1_b) * (l.hada_w2_a @ l.hada_w2_b) * 0.5
    assert torch.allclose(l.delta_weight(), exp)
    assert set(k.split(".", 1)[1] for k in l.state_tensors("m")) == {"hada_w1_a", "hada_w1_b", "hada_w2_a", "hada_w2_b", "alpha"}
    k = lycoris.LoKr(8, 6, rank=8, alpha=8, factor=2)
    assert not k.w2_factored and k.scale == 1.0 and "m.lokr_w2" in k.state_tensors("m")
    with torch.no_grad():
        k.lokr_w2.normal_()
    d = k.delta_weight()
    w1, w2 = k.lokr_w1, k.lokr_w2
    assert abs(float(d[1 * w2.shape[0] + 2, 1 * w2.shape[1] + 1] - w1[1, 1] * w2[2, 1])) < 1e-6
    assert lycoris.factorization(3072, -1) == (48, 64) and lycoris.factorization(3072, 16) == (16, 192)
    t = lycoris.TuckerConv(8, 4, k=3, rank=2)
    assert t.delta_weight().shape == (8, 4, 3, 3)
    assert set(x.split(".", 1)[1] for x in t.state_tensors("m")) == {"lora_down.weight", "lora_mid.weight", "lora_up.weight", "alpha"}
    b = lycoris.BOFT(32, 4, block=4)
    assert b.boft_m == bin(8 - 1).count("1") + 1 and b.oft_blocks.shape == (4, 8, 4, 4)
    dora = lycoris.DoRA(6, 4, rank=2, base_weight=torch.randn(6, 4))
    assert dora.dora_scale.dtype == torch.float32 and "m.dora_scale" in dora.state_tensors("m")


def test_lycoris_inject_save_load(tmp_path):
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.GELU(), torch.nn.Linear(16, 8))
    x = torch.randn(3, 8)
    y0 = net(x)
    ads = lycoris.inject_lycoris(net, "loha", rank=2, alpha=2)
    assert len(ads) == 2 and torch.allclose(net(x), y0, atol=1e-5)
    for a in ads.values():
        with torch.no_grad():
            a.hada_w2_a.normal_(0, 0.1)
    y1 = net(x)
    assert not torch.allclose(y1, y0, atol=1e-4)
    sd = lycoris.lycoris_state_dict(ads)
    assert all(v.dtype in (torch.bfloat16, torch.float32) for v in sd.values())
    for a in ads.values():
        with torch.no_grad():
            a.hada_w2_a.zero_()
    lycoris.load_lycoris_state_dict(ads, sd)
    assert torch.allclose(net(x), y1, atol=2e-2)


def test_ema_schedule_and_update():
    assert ema_decay_at_step(5, update_after_step=5) == 0.0
    v = ema_decay_at_step(15, 5, inv_gamma=2.0, power=0.75, min_decay=0.0, max_decay=0.9999)
    assert abs(v - (1 - (1 + 10 / 2.0) ** -0.75)) < 1e-9
    assert ema_decay_at_step(10 ** 9, 0, 1.0, 1.0, 0.0, 0.999) == 0.999
    p = torch.nn.Parameter(torch.tensor([2.0]))
    e = EMA([p], decay=0.999)
    e.shadow[0].fill_(1.0)
    e.update(1)
    assert abs(float(e.shadow[0]) - 1.001) < 1e-6
    with e.swap_in():
        assert abs(float(p) - 1.001) < 1e-6
    assert float(p) == 2.0


def test_aspect_buckets():
    assert buckets.round_to_multiple(1000.0, 64) == 1024 and buckets.pixel_resolution(1.0, 64) == 1024
    bs = buckets.generate_aspect_buckets(1.0, 64)
    dims = {(b.width, b.height) for b in bs}
    assert (1024, 1024) in dims and all(w % 64 == 0 and h % 64 == 0 for w, h in dims)
    for b in bs:
        assert abs(b.width * b.height - 1024 * 1024) / (1024 * 1024) < 0.15
    a = buckets.assign_aspect_bucket(4000, 3000, 1.0, 64)
    assert a.aspect == 1.33 and a.target_w > a.target_h
    assert a.inter_w >= a.target_w and a.inter_h >= a.target_h
    assert a.crop_x == (a.inter_w - a.target_w) // 2 and a.crop_y == (a.inter_h - a.target_h) // 2
    s = buckets.assign_aspect_bucket(512, 512, 1.0, 64)
    assert (s.target_w, s.target_h) == (1024, 1024) and s.crop_x == 0


def test_features_default_off_and_math():
    g = torch.Generator().manual_seed(0)
    n = torch.randn(2, 16, 8)
    st = g.get_state()
    assert features.apply_offset_noise(n, 0.0, 1.0, g) is n and features.apply_input_perturbation(n, 0.0, g) is n
    assert features.apply_multires_noise(n, 0) is n and not features.should_drop_caption(0.0, g)
    assert torch.equal(st, g.get_state())                       # nothing drawn while everything is off
    o = features.apply_offset_noise(n, 0.1, 1.0, g)
    d = o - n
    assert torch.allclose(d[:, 0], d[:, 5]) and not torch.allclose(d[0, 0], d[1, 0])   # per (sample, channel)
    m = features.apply_multires_noise(torch.randn(1, 4, 16, 16), 3, 0.3, g)
    assert abs(float(m.std()) - 1.0) < 1e-3
    t = torch.tensor([0.2, 0.8])
    assert torch.equal(features.apply_timestep_bias(t), t)
    assert torch.allclose(features.apply_timestep_bias(t, 1.0, "later", 0.5), t + 0.5 * (1 - t))
    assert torch.allclose(features.apply_timestep_bias(t, 1.0, "earlier", 0.25), t * 0.75)
    assert torch.allclose(features.apply_timestep_bias(t, 1.0, "range", 0, 0.2, 0.6), 0.2 + t * 0.4)
    acc = features.GradAccumulator(3)
    assert [acc.tick() for _ in range(6)] == [False, False, True, False, False, True] and abs(acc.loss_scale - 1 / 3) < 1e-9
    assert features.drop_caption(torch.ones(1, 2, 3), None, 1.0, g).abs().sum() == 0


def _make_cache(d, n=6):
    for i in range(n):
        h = 4 if i % 3 else 6
        write_sample(os.path.join(d, f"s{i:03d}.safetensors"), torch.full((1, 16, h, 4), float(i)).bfloat16(),
                     torch.full((1, 8, 32), float(i)).bfloat16(), torch.ones(1, 8))


def test_dataset_cache_and_loader(tmp_path):
    d = str(tmp_path)
    _make_cache(d)
    cache = LatentCache(d)
    assert len(cache) == 6 and len(cache.buckets()) == 2
    ld = BatchLoader(cache, 2, seed=3, pin=False)
    b0 = ld.batches_for_epoch(0)
    assert b0 == ld.batches_for_epoch(0) and all(len(b) == 2 for b in b0) and len(b0) == 3
    for b in b0:
        assert len({cache.keys[i] for i in b}) == 1          # same-shape batches only
    seen = 0
    for got in ld.epoch(0):                                  # staging buffers are reused: consume each batch in turn
        assert got["latent"].shape[0] == 2 and got["latent"].dtype == torch.bfloat16
        assert [float(x) for x in got["latent"][:, 0, 0, 0]] == [float(i) for i in got["indices"]]
        seen += 1
    assert seen == 3
    assert len(list(ld.epoch(0, skip=2))) == 1
    r0 = BatchLoader(cache, 2, seed=3, rank=0, world=2, pin=False).batches_for_epoch(0)
    r1 = BatchLoader(cache, 2, seed=3, rank=1, world=2, pin=False).batches_for_epoch(0)
    assert len(r0) == len(r1) == 1 and not set(map(tuple, r0)) & set(map(tuple, r1))
    with pytest.raises(FileNotFoundError):
        LatentCache(str(tmp_path / "nope")) if (tmp_path / "nope").mkdir() is None else None


def test_full_finetune_state_contract(tmp_path):
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(4, 6), torch.nn.Linear(6, 2)).bfloat16()
    inv, opt = full_finetune.prepare_full_finetune(net, 1e-2)
    x = torch.randn(3, 4).bfloat16()
    for _ in range(2):
        opt.zero_grad(set_to_none=True)
        net(x).float().pow(2).mean().backward()
        opt.step()
    assert opt.masters[0].dtype == torch.float32
    assert torch.equal(opt.masters[0].bfloat16(), inv[0][1].detach())
    sp, mp = str(tmp_path / "state.safetensors"), str(tmp_path / "model.safetensors")
    full_finetune.save_state(sp, inv, opt, t_step=2, accum_count=0)
    full_finetune.save_model_tensors(mp, inv)
    from mojodiffusion_b200.io.safetensors_io import SafeTensors, load_safetensors
    st = SafeTensors(sp)
    keys = st.keys()
    st.close()
    n = len(inv)
    assert keys[:n] == [f"param.{i}" for i in range(n)] and keys[n] == "adam_m.0" and keys[n + 1] == "adam_v.0"
    assert keys[3 * n] == "__meta__" and full_finetune.MANIFEST_KEY in keys
    assert all(v.dtype == torch.bfloat16 for v in load_safetensors(mp).values())
    net2 = torch.nn.Sequential(torch.nn.Linear(4, 6), torch.nn.Linear(6, 2)).bfloat16()
    inv2, opt2 = full_finetune.prepare_full_finetune(net2, 1e-2)
    assert full_finetune.load_state(sp, inv2, opt2) == (2, 0)
    assert torch.equal(opt2.masters[1], opt.masters[1]) and torch.equal(opt2.m[2], opt.m[2]) and opt2.step_count == 2
    with pytest.raises(ValueError):
        full_finetune.load_state(sp, list(reversed(inv2)), opt2)


def test_progress_line():
    assert format_hms(3725) == "1:02:05"
    clock = iter([0.0, 2.0, 4.0]).__next__
    buf = io.StringIO()
    d = ProgressDisplay("Flux", 10, 2, stream=buf, clock=clock)
    s = d.update(1, 1, 0.12345, 1.5)
    assert s == "[Flux] step 1/10 | epoch 1/2 | loss 0.1235 | grad_norm 1.5000 | 2.0s/step | elapsed 0:00:02 | ETA 0:00:18"
    assert buf.getvalue().startswith("\r[Flux]")


def test_board_roundtrip(tmp_path):
    from mojodiffusion_b200.io.png import save_png
    b = BoardWriter(str(tmp_path), "sess-1", resume_step=0, name="flux-lora")
    b.log_hparams({"lr": 1e-4})
    b.log_train_step(1, 0.5, 1.2, 1e-4, 0.25)
    b.log_train_step(1, 0.4, 1.2, 1e-4, 0.25)           # same step: replaced, not duplicated
    b.log_text("prompt", 1, "a cat")
    b.log_trace(1, "forward", 12.5)
    png = str(tmp_path / "x.png")
    save_png(png, torch.zeros(8, 12, 3, dtype=torch.uint8))
    key = b.log_image_png("samples/0", 1, 0, png)
    b.close()
    assert os.path.isfile(tmp_path / "blobs" / key)
    db = sqlite3.connect(str(tmp_path / "board.db"))
    assert db.execute("SELECT value FROM scalars WHERE tag='loss/train' AND step=1").fetchall() == [(0.4,)]
    assert db.execute("SELECT COUNT(*) FROM scalars").fetchone()[0] == 5
    assert db.execute("SELECT status FROM sessions").fetchone()[0] == "complete"
    assert db.execute("SELECT width, height FROM artifacts").fetchone() == (12, 8)
    tables = {r[0] for r in db.execute("SELECT name FROM sqlite_master WHERE type='table'")}
    assert {"metadata", "sessions", "scalars", "tensors", "artifacts", "text_events", "trace_events", "eval_results",
            "hparam_metrics", "plugin_data", "custom_scalar_layouts", "pr_curves", "audio", "graphs", "embeddings",
            "meshes"} <= tables


def test_cadence_names_and_resume(tmp_path):
    p = loop.TrainProgress(120, 3, 7, 28)
    assert loop.step_save_path("/w", "lora_", "2026-01-01_00-00-00", p).endswith("/save/lora_2026-01-01_00-00-00-save-120-3-7.safetensors")
    assert loop.backup_path("/w", "T", p) == "/w/backup/T-backup-120-3-7"
    assert loop.training_sample_leaf("x", "T", p) == "xT-training-sample-120-3-7"
    with pytest.raises(ValueError):
        loop.model_file_extension("GGUF")
    cfg = TrainConfig(save_every=4, sample_every=3, save_skip_first=5, max_steps=10, batch_size=2)
    cad = loop.Cadence(cfg)
    saves, samples = [], []
    for s in range(0, 13):
        d = cad.decide(loop.TrainProgress(s, 0, s, 0))
        saves += [s] if d.save else []
        samples += [s] if d.sample else []
    assert saves == [8, 12] and samples == [0, 3, 6, 9, 12]

    # a tiny run: linear regression "model", 2 epochs of 3 batches, then resume to the same final state
    def make(ws, resume):
        torch.manual_seed(0)
        w = torch.nn.Parameter(torch.zeros(4))
        opt = FusedAdamW([w], 1e-1)
        cfg = TrainConfig(workspace_dir=ws, output_model_destination="final.safetensors", save_every=2, sample_every=0,
                          max_steps=6, batch_size=2, learning_rate=1e-1, continue_last_backup=resume, model_type="flux")

        class L:
            def steps_per_epoch(self):
                return 3

            def epoch(self, e, skip=0):
                for i in range(skip, 3):
                    yield torch.full((4,), float(e * 3 + i + 1))

        def step_fn(batch, lr):
            opt.zero_grad(set_to_none=True)
            loss = ((w - batch) ** 2).mean()
            loss.backward()
            opt.step(lr=lr)
            return loss.detach(), 0.0

        run = loop.TrainRun(cfg, L(), step_fn, lambda: {"w": w.detach().clone()},
                            lambda: {"m": opt.m[0], "v": opt.v[0], "step": torch.tensor([opt.step_count])},
                            lambda sd: w.data.copy_(sd["w"]),
                            lambda sd: (opt.set_moments(w, sd["m"], sd["v"]), setattr(opt, "step_count", int(sd["step"][0]))),
                            timestamp="T", display=False, backup_after=4, backup_after_unit="STEP")
        return run, w

    ws = str(tmp_path / "ws")
    run, w_full = make(ws, False)
    run.run()
    assert run.progress.global_step == 6 and run.progress.epoch == 2 and run.progress.epoch_step == 0
    assert sorted(os.listdir(os.path.join(ws, "save"))) == ["T-save-2-0-2.safetensors", "T-save-4-1-1.safetensors", "T-save-6-1-3.safetensors"]
    assert os.path.isfile(os.path.join(ws, "backup", "T-backup-4-1-1", "meta.json"))
    # remove the final backup so the resume starts from step 4, then finish and compare
    import shutil
    shutil.rmtree(os.path.join(ws, "backup", "T-backup-6-2-0"))
    run2, w_res = make(ws, True)
    assert run2.resume_if_requested() and run2.progress.global_step == 4 and run2.progress.epoch_step == 1
    run2.run()
    assert torch.allclose(w_res, w_full, atol=1e-6)
    os.remove(os.path.join(ws, "backup", "T-backup-4-1-1", "optimizer", "optimizer.safetensors"))
    shutil.rmtree(os.path.join(ws, "backup", "T-backup-6-2-0"))
    with pytest.raises(FileNotFoundError):
        loop.read_backup(os.path.join(ws, "backup", "T-backup-4-1-1"))


def test_lora_key_schemes_of_the_other_families(tmp_path):
    """Klein (diffusers-style names over fused BFL weights), Qwen-Image, Z-Image and LTX-2 adapter inventories; the PEFT
    file of each has exactly <prefix>.lora_A.weight / .lora_B.weight per adapter, and a zero-initialised up matrix leaves
    the model output unchanged."""
    import torch
    from mojodiffusion_b200.io.safetensors_io import SafeTensors
    from mojodiffusion_b200.models.flux2 import Flux2DiT, tiny_flux2_config
    from mojodiffusion_b200.models.qwen_image import QwenImageDiT, tiny_qwen_image_config
    from mojodiffusion_b200.models.single_dit import SingleStreamDiT, tiny_single_dit_config
    from mojodiffusion_b200.models.video_dit import VideoDiT, tiny_video_dit_config
    from mojodiffusion_b200.training import lora as L

    g = torch.Generator().manual_seed(0)
    cfg = tiny_flux2_config()
    m = Flux2DiT(cfg, torch.float32, "cpu").init_weights(0)
    img, txt, t = torch.randn(1, 16, cfg.in_channels, generator=g), torch.randn(1, 4, cfg.context_dim, generator=g), torch.tensor([0.5])
    with torch.no_grad():
        base = m(img, txt, t, (4, 4))
    slots = L.inject_klein_lora(m, rank=4, alpha=4.0)
    assert [s.key for s in slots] == L.klein_lora_prefixes(cfg.depth_double, cfg.depth_single)
    assert len(slots) == 12 * cfg.depth_double + 2 * cfg.depth_single
    q = next(s for s in slots if s.key.endswith("transformer_blocks.0.attn.to_k"))
    assert (q.row0, q.row1) == (cfg.hidden, 2 * cfg.hidden) and tuple(q.up.shape) == (cfg.hidden, 4)
    with torch.no_grad():
        assert torch.allclose(m(img, txt, t, (4, 4)), base, atol=1e-6)
    path = tmp_path / "klein.safetensors"
    L.save_lora(str(path), slots, layout="peft")
    keys = set(SafeTensors(str(path)).keys())
    assert keys == {f"{p}.lora_{ab}.weight" for p in L.klein_lora_prefixes(cfg.depth_double, cfg.depth_single) for ab in "AB"}

    qm = QwenImageDiT(tiny_qwen_image_config(), torch.float32, "cpu").init_weights(0)
    qs = L.inject_qwen_lora(qm, rank=4)
    assert len(qs) == 12 * len(qm.transformer_blocks)
    assert qs[4].key == "transformer.transformer_blocks.0.img_mlp.net.0.proj" and qs[-1].key.endswith("txt_mlp.net.2")

    zm = SingleStreamDiT(tiny_single_dit_config(), torch.float32, "cpu").init_weights(0)
    zs = L.inject_zimage_lora(zm, rank=4)
    assert len(zs) == 7 * len(zm.layers) and all(s.key.startswith("layers.") for s in zs)
    zr = L.inject_zimage_lora(SingleStreamDiT(tiny_single_dit_config(), torch.float32, "cpu"), rank=4, refiners=True)
    assert len(zr) == 7 * (len(zm.layers) + len(zm.noise_refiner) + len(zm.context_refiner))
    assert L.zimage_kohya_name("layers.3.attention.to_out.0") == "lora_unet_layers_3_attention_to_out_0"
    from mojodiffusion_b200.models.single_dit import zimage_config
    with torch.device("meta"):
        full = SingleStreamDiT(zimage_config(), torch.float32, "meta")
        assert len(L.inject_zimage_lora(full, rank=16)) == 210

    vm = VideoDiT(tiny_video_dit_config(), torch.float32, "cpu").init_weights(0)
    vs = L.inject_ltx2_lora(vm, rank=4)
    assert len(vs) == 10 * len(vm.transformer_blocks)
    assert vs[0].key == "diffusion_model.transformer_blocks.0.attn1.to_q" and vs[9].key == "diffusion_model.transformer_blocks.0.ff.net.2"


def test_epoch_unit_cadence_fires_at_epoch_boundaries(tmp_path):
    """save_every = 1 EPOCH over two short epochs writes one file per finished epoch (the decision is taken right after
    the epoch counter advances, where epoch_step == 0), and the hooks around rank-0-only actions are called."""
    import torch
    from mojodiffusion_b200.io.config import TrainConfig
    from mojodiffusion_b200.training.loop import TrainRun

    class Loader:
        def steps_per_epoch(self):
            return 3

        def epoch(self, epoch, skip=0):
            for i in range(skip, 3):
                yield i

    cfg = TrainConfig()
    cfg.workspace_dir = str(tmp_path)
    cfg.save_every, cfg.save_every_unit = 1, "EPOCH"
    cfg.sample_after_unit, cfg.sample_every, cfg.sample_after = "NEVER", 0, 0
    cfg.output_model_destination = ""
    w = {"a": torch.zeros(2)}
    calls = {"pre": 0, "bar": 0}
    run = TrainRun(cfg, Loader(), lambda b, lr: (torch.tensor(1.0), torch.tensor(0.5)), lambda: w, lambda: {"m": torch.zeros(2)},
                   lambda sd: None, lambda sd: None, display=False,
                   pre_save_fn=lambda: calls.__setitem__("pre", calls["pre"] + 1),
                   barrier_fn=lambda: calls.__setitem__("bar", calls["bar"] + 1), loss_sync_every=2)
    p = run.run(max_steps=6)
    assert p.global_step == 6 and p.epoch == 2
    names = sorted(os.path.basename(s) for s in run.saved)
    assert len(names) == 2 and names[0].endswith("-save-3-1-0.safetensors") and names[1].endswith("-save-6-2-0.safetensors"), names
    assert calls["pre"] == 3 and calls["bar"] == 3          # two epoch saves + the final backup
    assert len(run.losses) == 3                              # read back every second step only


def test_automagic3_update_vote_and_stochastic_rounding():
    import math
    import torch
    from mojodiffusion_b200.training.optim_extra import Automagic3, create_optimizer
    torch.manual_seed(0)
    # factored update of one step against the loop statement
    p = torch.nn.Parameter(torch.zeros(3, 4))
    g = torch.randn(3, 4)
    p.grad = g.clone()
    opt = Automagic3([p], lr=1e-3, beta2=0.9, eps=1e-30, clip=1.0)
    opt.step()
    row = 0.1 * ((g * g).mean(1) + 1e-30)
    col = 0.1 * ((g * g).mean(0) + 1e-30)
    upd = torch.zeros(3, 4)
    for i in range(3):
        for j in range(4):
            upd[i, j] = (row[i] / row.mean()) ** -0.5 * col[j] ** -0.5 * g[i, j]
    upd = (upd / max(float(upd.square().mean().sqrt()) / 1.0, 1.0)).clamp(-1, 1)
    assert torch.allclose(p.detach(), -1e-3 * upd, atol=1e-7)
    # vote: abstains for H steps, then constant-sign gradients multiply the rate by e per step, alternating ones divide
    q = torch.nn.Parameter(torch.zeros(6))
    o2 = Automagic3([q], lr=1e-4, history=4)
    rates = []
    for _ in range(7):
        q.grad = torch.ones(6)
        o2.step()
        rates.append(o2.lr)
    assert rates[:3] == [1e-4] * 3 and all(abs(rates[i + 1] / rates[i] - math.e) < 1e-9 for i in range(3, 6))
    o3 = Automagic3([torch.nn.Parameter(torch.zeros(6))], lr=1e-4, history=4)
    r3 = []
    for k in range(7):
        o3.params[0].grad = torch.full((6,), 1.0 if k % 2 == 0 else -1.0)
        o3.step()
        r3.append(o3.lr)
    assert r3[:3] == [1e-4] * 3 and abs(r3[4] / r3[3] - math.exp(-1)) < 1e-9
    # mixed histories neither raise nor lower
    o4 = Automagic3([torch.nn.Parameter(torch.zeros(2))], lr=1e-4, history=4)
    for sgn in (1, 1, -1, -1, 1, 1):
        o4.params[0].grad = torch.full((2,), float(sgn))
        o4.step()
    assert o4.lr == 1e-4
    # bf16 weights keep moving at a step far below one bf16 ulp (unbiased stochastic rounding)
    w = torch.nn.Parameter(torch.full((4096,), 0.1, dtype=torch.bfloat16))
    o5 = Automagic3([w], lr=1e-5, history=64)
    for _ in range(50):
        w.grad = torch.ones(4096, dtype=torch.bfloat16)
        o5.step()
    moved = 0.1 - float(w.detach().float().mean())
    assert 0.6 * 50e-5 < moved < 1.4 * 50e-5            # expected 50 steps x 1e-5 x |update| = 1
    assert isinstance(create_optimizer("automagic3", [torch.nn.Parameter(torch.zeros(2))], 1e-6), Automagic3)
