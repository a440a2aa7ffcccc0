"""Public entry points on the tiny architectures (CPU): train CLI (LoRA in the family's key scheme, cadence saves, backup,
resume, validation PNGs), sampler CLI (PNG with embedded generation parameters, adapter overlay), manifests, presets."""
import json
import os
import subprocess
import sys

import pytest
import torch

from mojodiffusion_b200.io.png import load_png
from mojodiffusion_b200.io.safetensors_io import SafeTensors
from mojodiffusion_b200.runtime import ProductionGuard, ShapeProfile, default_manifest_by_id, manifest_ids
from mojodiffusion_b200.training.dataset import write_sample
from mojodiffusion_b200.training.presets import apply_preset, dry_run_report, lifecycle_paths, preset_entry, preset_ids

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# family -> (latent channels of the tiny architecture, text dim, text tokens, pooled dim)
TINY = {"flux": (16, 256, 16, 0), "klein": (8, 128, 16, 0), "zimage": (16, 128, 16, 0), "qwenimage": (16, 128, 16, 0),
        "sdxl": None}


def _run(mod, *args, env=None):
    e = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    e.update(env or {})
    r = subprocess.run([sys.executable, "-m", mod, *args], capture_output=True, text=True, env=e, cwd=ROOT, timeout=600)
    assert r.returncode == 0, f"{mod} {args} failed:\n{r.stdout[-2000:]}\n{r.stderr[-3000:]}"
    return json.loads(r.stdout.strip().splitlines()[-1])


def _tiny_dims(family):
    m = default_manifest_by_id(family)
    cfg = m.config(tiny=True)
    if family == "sdxl":
        return 4, cfg.context_dim, 8, cfg.adm_in_channels
    C = cfg.in_channels // (m.latent.patch ** 2) if m.latent.packed else cfg.in_channels
    from mojodiffusion_b200.runtime.adapters import adapter_for
    return C, adapter_for(m).text_dim(cfg), 16, 0


def _make_cache(d, family, n=4, hw=8):
    C, D, T, P = _tiny_dims(family)
    g = torch.Generator().manual_seed(0)
    os.makedirs(d, exist_ok=True)
    for i in range(n):
        write_sample(os.path.join(d, f"s{i:03d}.safetensors"), torch.randn(1, C, hw, hw, generator=g),
                     torch.randn(1, T, D, generator=g), torch.ones(1, T))


def _write_cfg(tmp, family, **over):
    ws = os.path.join(tmp, "ws")
    prompts = os.path.join(tmp, "prompts.json")
    json.dump({"schema": "serenity.sample_prompts.v1", "defaults": {"width": 64, "height": 64, "steps": 2, "cfg": 1.0, "seed": 7},
               "prompts": [{"id": "p0", "prompt": "a lighthouse at dusk"}, {"id": "p1", "prompt": "a red bicycle", "cfg": 2.0,
                                                                            "negative": "blurry"}]}, open(prompts, "w"))
    cfg = {"model_type": family, "training_method": "LORA", "lora_rank": 4, "lora_alpha": 4.0, "learning_rate": 1e-3,
           "batch_size": 2, "max_steps": 4, "save_every": 2, "save_every_unit": "STEP", "sample_every": 2, "sample_after_unit": "STEP",
           "cache_dir": os.path.join(tmp, "cache"), "workspace_dir": ws, "output_model_destination": "out/lora.safetensors",
           "validation_prompts_file": prompts, "gradient_checkpointing": "OFF", "backup_after": 2, "backup_after_unit": "STEP", "seed": 3}
    cfg.update(over)
    path = os.path.join(tmp, "config.json")
    json.dump(cfg, open(path, "w"))
    return path, ws, prompts


KEY_PREFIX = {"flux": "lora_transformer_", "klein": "transformer.", "zimage": "layers.", "qwenimage": "transformer.", "sdxl": "lora_unet_",
              "lens": "transformer_blocks.", "krea2": "blocks."}
KEY_SUFFIX = {"flux": ".lora_down.weight", "klein": ".lora_A.weight", "zimage": ".lora_A.weight", "qwenimage": ".lora_down.weight",
              "sdxl": ".lora_down.weight", "lens": ".lora_A.weight", "krea2": ".lora_A.weight"}


@pytest.mark.parametrize("family", ["flux", "klein", "zimage", "qwenimage", "sdxl", "lens", "krea2"])
def test_train_then_resume_then_sample(tmp_path, family):
    tmp = str(tmp_path)
    _make_cache(os.path.join(tmp, "cache"), family)
    cfg_path, ws, prompts = _write_cfg(tmp, family)
    rep = _run("mojodiffusion_b200.cli.train", cfg_path, "--tiny", "--quiet")
    assert rep["global_step"] == 4 and rep["weights"] == "random-init" and rep["adapters"] > 0
    assert rep["first_loss"] == rep["first_loss"] and rep["final_loss"] < 1e4
    lora = os.path.join(ws, "out", "lora.safetensors")
    st = SafeTensors(lora)
    keys = list(st.keys())
    st.close()
    assert any(k.startswith(KEY_PREFIX[family]) and k.endswith(KEY_SUFFIX[family]) for k in keys), keys[:4]
    side = SafeTensors(os.path.join(ws, "out", "lora.state.safetensors"))
    sk = set(side.keys())
    side.close()
    assert "__meta__" in sk and any(k.endswith(".lora_A.adam_m") for k in sk) and any(k.endswith(".lora_B.adam_v") for k in sk)
    saves = sorted(os.listdir(os.path.join(ws, "save")))
    assert len(saves) == 2 and "-save-2-" in saves[0] and "-save-4-" in saves[1]
    pngs = sorted(f for f in os.listdir(os.path.join(ws, "samples")) if f.endswith(".png"))
    assert len(pngs) == 4, pngs                                    # two prompts at steps 2 and 4
    img, _ = load_png(os.path.join(ws, "samples", pngs[0]))
    assert img.shape[:2] == (64, 64)
    assert os.path.isdir(os.path.join(ws, "backup"))
    # resume from the last backup and continue to step 6: the step counter and the optimizer state carry over
    cfg2, _, _ = _write_cfg(tmp, family, max_steps=6, continue_last_backup=True)
    rep2 = _run("mojodiffusion_b200.cli.train", cfg2, "--tiny", "--quiet")
    assert rep2["resumed"] is True and rep2["global_step"] == 6
    side = SafeTensors(os.path.join(ws, "out", "lora.state.safetensors"))
    assert int(side.tensor("__meta__")[0]) == 6
    side.close()
    # sampler CLI with the trained adapter as a runtime overlay
    out = os.path.join(tmp, "img", "p1.png")
    srep = _run("mojodiffusion_b200.cli.sample", family, cfg2, lora, prompts, "p1", out, "--tiny")
    assert srep["weights"] == "random-init" and "runtime overlay" in srep["lora"] and srep["text"] == "hash-embedding"
    img, _ = load_png(out)
    assert img.shape[:2] == (64, 64) and img.std() > 0
    gen = json.loads(load_png(out)[1]["serenity.genparams.v1"])
    assert gen["prompt"] == "a red bicycle" and gen["seed"] == 7 and gen["steps"] == 2 and gen["cfg"] == 2.0 and gen["prompt_id"] == "p1"
    # same seed, no adapter: a different image (the overlay is applied) of the same size
    out2 = os.path.join(tmp, "img", "p1_base.png")
    _run("mojodiffusion_b200.cli.sample", family, cfg2, "-", prompts, "p1", out2, "--tiny")
    img2, _ = load_png(out2)
    assert img2.shape == img.shape


def test_dry_run_reports_plan_and_cache_problems(tmp_path):
    tmp = str(tmp_path)
    _make_cache(os.path.join(tmp, "cache"), "flux", n=3)
    cfg_path, ws, _ = _write_cfg(tmp, "flux")
    e = dict(os.environ, PYTHONPATH=ROOT, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, "-m", "mojodiffusion_b200.cli.train", cfg_path, "--tiny", "--dry-run"], capture_output=True,
                       text=True, env=e, cwd=ROOT, timeout=300)
    plan = json.loads(r.stdout.strip().splitlines()[-1])
    assert plan["schema"] == "mdb200.train_plan.v1" and plan["family"] == "flux" and plan["steps_per_epoch"] == 1
    assert plan["lora"]["layout"] == "onetrainer" and plan["prompts"] == ["p0", "p1"] and plan["cache"]["samples"] == 3
    assert not os.path.exists(ws)                                  # a dry run writes nothing


def test_cadence_supervisor_trains_in_chunks_and_samples_between(tmp_path):
    tmp = str(tmp_path)
    _make_cache(os.path.join(tmp, "cache"), "klein")
    cfg_path, ws, _ = _write_cfg(tmp, "klein", max_steps=4, save_every=0)
    rep = _run("mojodiffusion_b200.cli.train_cadence", cfg_path, "--chunk", "2", "--tiny")
    assert rep["ok"] and rep["steps"] == 4
    chunks = [e for e in rep["events"] if e["event"] == "train_chunk"]
    samples = [e for e in rep["events"] if e["event"] == "sample"]
    assert [(c["from"], c["to"]) for c in chunks] == [(0, 2), (2, 4)] and len(samples) == 4
    assert all(s["rc"] == 0 and os.path.isfile(s["png"]) for s in samples)


def test_manifest_registry_and_guards():
    ids = manifest_ids()
    for want in ("flux1-dev", "flux2-klein-9b", "qwen-image", "z-image", "sd35-large", "chroma", "sdxl", "ltx2", "wan22-ti2v-5b"):
        assert want in ids
    assert default_manifest_by_id("flux").model_id == "flux1-dev"
    assert default_manifest_by_id("klein").family == "klein" and default_manifest_by_id("qwenimage").param_billions == 20.0
    assert default_manifest_by_id("flux1-dev-fp8.safetensors").model_id == "flux1-dev"
    with pytest.raises(KeyError):
        default_manifest_by_id("no-such-model")
    m = default_manifest_by_id("flux")
    sh = ShapeProfile.of(m, 1024, 1024)
    assert sh.image_tokens == 4096 and sh.text_tokens == 512 and sh.seq_len == 4608
    assert ShapeProfile.of(default_manifest_by_id("ltx2"), 768, 512, 121).image_tokens == 6144
    with pytest.raises(ValueError):
        ShapeProfile.of(m, 1000, 1024)
    with pytest.raises(PermissionError):
        ProductionGuard.check(default_manifest_by_id("chroma"), ShapeProfile.of(default_manifest_by_id("chroma"), 512, 512), serving=True)
    from mojodiffusion_b200.runtime import ExecutionConfig
    with pytest.raises(ValueError):
        ProductionGuard.check(m, sh, ExecutionConfig(sequence_parallel=5))
    ProductionGuard.check(m, sh, ExecutionConfig(sequence_parallel=8))
    # every manifest can build its tiny backbone and names an existing offload plan
    from mojodiffusion_b200.offload import plan as P
    for mid in ids:
        mm = default_manifest_by_id(mid)
        net = mm.build(tiny=True)
        assert sum(p.numel() for p in net.parameters()) > 0
        if mm.offload_plan:
            assert hasattr(P, mm.offload_plan), mm.offload_plan


def test_preset_catalogue_and_contracts(tmp_path):
    from mojodiffusion_b200.io.config import TrainConfig
    assert len(preset_ids()) == 29
    e = preset_entry("qwen")
    assert e.preset_id == "qwen_lora_16gb" and e.vram_tier_gb == 16 and e.optimizer == "ADAMW" and e.variant == "lora"
    assert preset_entry("zimage_deturbo_lora_8gb").variant == "deturbo_lora" and preset_entry("sdxl_1_0_inpaint_lora").variant == "inpaint_lora"
    assert preset_entry("qwen_finetune_24gb").optimizer == "ADAFACTOR" and preset_entry("qwen_finetune_24gb").training_method == "FINE_TUNE"
    with pytest.raises(ValueError):
        preset_entry("sd3")
    with pytest.raises(KeyError):
        preset_entry("nope")
    cfg = TrainConfig()
    apply_preset(cfg, "flux2_finetune_24gb")
    assert cfg.model_type == "klein" and cfg.training_method == "FINE_TUNE" and cfg.optimizer.optimizer == "ADAFACTOR"
    cfg.workspace_dir, cfg.output_model_destination, cfg.save_every = str(tmp_path), "out/my_lora.safetensors", 500
    p = lifecycle_paths(cfg, 500)
    assert p["final"].endswith("out/my_lora.safetensors") and p["state_sidecar"].endswith("out/my_lora.state.safetensors")
    assert p["step_file"].endswith("out/my_lora_step500.safetensors")
    rep = dry_run_report(cfg, "ernie_lora_8gb")
    assert not rep["ok"] and any("no runnable loop" in x for x in rep["problems"]) and any("cache" in x for x in rep["problems"])


@pytest.mark.parametrize("family", ["zimage_l2p", "sensenova_u1"])
def test_sample_cli_runs_the_pixel_space_families_without_a_vae(tmp_path, family):
    """Z-Image L2P and SenseNova-U1 produce pixels directly: the sampler entry point calls the model's own loop and writes the PNG."""
    tmp = str(tmp_path)
    cfg_path, ws, prompts = _write_cfg(tmp, family)
    out = os.path.join(tmp, "img", "p1.png")
    rep = _run("mojodiffusion_b200.cli.sample", family, cfg_path, "-", prompts, "p1", out, "--tiny")
    assert rep["family"] == family and rep["vae_weights"] == "none (pixel space)" and rep["text"] in ("hash-embedding", "hash-token-ids")
    img, meta = load_png(out)
    assert img.shape[:2] == (64, 64) and img.std() > 0 and json.loads(meta["serenity.genparams.v1"])["seed"] == 7


@pytest.mark.parametrize("family", ["lens", "krea2"])
def test_sample_cli_drives_lens_and_krea2_through_their_own_schedules(tmp_path, family):
    """The sampler entry point runs the two families whose text features are stacks of encoder layers: tiny architecture,
    hash text features of the stacked width, the family's exponential-shift time table and guidance rule, PNG out."""
    from mojodiffusion_b200.runtime.adapters import adapter_for, schedule_for
    from mojodiffusion_b200.sampling.family_schedules import krea2_timesteps, lens_sigmas
    tmp = str(tmp_path)
    cfg_path, ws, prompts = _write_cfg(tmp, family)
    out = os.path.join(tmp, "img", "p1.png")
    rep = _run("mojodiffusion_b200.cli.sample", family, cfg_path, "-", prompts, "p1", out, "--tiny")
    assert rep["family"] == family and rep["weights"] == "random-init" and rep["text"] == "hash-embedding" and rep["lora"] == "none"
    img, meta = load_png(out)
    assert img.shape[:2] == (64, 64) and img.std() > 0
    gen = json.loads(meta["serenity.genparams.v1"])
    assert gen["steps"] == 2 and gen["cfg"] == 2.0 and gen["prompt"] == "a red bicycle"
    m = default_manifest_by_id(family)
    a = adapter_for(m)
    tiny = m.config(tiny=True)
    if family == "lens":
        assert a.text_dim(tiny) == tiny.text_layers * tiny.text_hidden and m.schedule.cfg_rule == "textbook"
        assert schedule_for(m, 5, 4096) == list(lens_sigmas(5, 4096)) + [0.0]
    else:
        assert a.text_dim(tiny) == tiny.txtlayers * tiny.txtdim and m.schedule.cfg_rule == "cond_anchored"
        assert schedule_for(m, 5, 4096) == krea2_timesteps(4096, 5)
