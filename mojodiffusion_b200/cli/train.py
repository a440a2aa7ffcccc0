"""Trainer entry point:

    python -m mojodiffusion_b200.cli.train <config.json> [--max-steps N] [--tiny] [--device D] [--dry-run] [--preset ID]

Builds, from the reference's JSON run config: manifest -> backbone (checkpoint or seeded random weights) -> LoRA adapters
under the family's key scheme (``training_method`` LORA) or fp32-master full finetune (FINE_TUNE) -> latent cache and
bucketed batch loader -> one-step trainer -> the run loop with its cadence actions: validation samples (staged denoise ->
VAE decode -> PNG per prompt of the sample-prompt file), step saves, backups with optimizer state, final save plus the
``<name>.state.safetensors`` train-state sidecar, resume from the last complete backup (``continue_last_backup``).
Under ``torchrun`` (WORLD_SIZE > 1) the ranks train data-parallel: on GPUs with the fused reduce-scatter + AdamW +
all-gather kernels, on CPU ranks (gloo) with an all-reduce of the flat gradient buffer; every rank reads its own slice of
the batch list and draws its own noise. ``--dry-run`` validates config, cache and schedule and prints the plan without
touching a GPU.

Trainer mains this stands in for: serenitymojo/training/train_anima_ot.mojo:790-838 (argument handling), :855-1020
(set-up), :1027-1192 (loop, cadence, saves); naming policy serenitymojo/training/onetrainer_train_loop_policy.mojo:247-311;
dry-run / preflight serenitymojo/training/onetrainer_dry_run.mojo, onetrainer_cache_preflight.mojo.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from collections import OrderedDict

import torch

from ..io.config import guard_free_space, read_model_config, read_sample_prompts
from ..runtime import adapter_for
from ..training import lora as L
from ..training.dataset import BatchLoader, LatentCache
from ..training.family_trainer import FamilyTrainer
from ..training.loop import TrainRun
from ..training.trainer import StepConfig
from .common import attach_lora, build_model, manifest_from_config, pick_device


def preflight(cfg, m, cache: LatentCache, tiny: bool) -> dict:
    """Cache preflight: every bucket must sit on the family's latent grid and carry its channel count."""
    L_ = m.latent
    problems = []
    want_c = None if tiny else L_.channels
    for key, idx in cache.buckets().items():
        if want_c is not None and key.channels != want_c:
            problems.append(f"bucket {key}: {key.channels} latent channels, {m.model_id} expects {want_c}")
        if L_.packed and (key.height % L_.patch or key.width % L_.patch):
            problems.append(f"bucket {key}: latent size not divisible by the patch size {L_.patch}")
        if len(idx) < cfg.batch_size:
            problems.append(f"bucket {key}: {len(idx)} samples < batch size {cfg.batch_size} (dropped every epoch)")
    return {"samples": len(cache), "buckets": len(cache.buckets()), "problems": problems}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="mojodiffusion_b200.cli.train")
    ap.add_argument("config")
    ap.add_argument("--max-steps", type=int, default=0, help="stop after this many optimizer steps in THIS process (0: config)")
    ap.add_argument("--tiny", action="store_true", help="tiny architecture of the family (smoke runs without checkpoints)")
    ap.add_argument("--device", default="")
    ap.add_argument("--dry-run", action="store_true")
    ap.add_argument("--preset", default="", help="apply a catalogue preset on top of the config before anything else")
    ap.add_argument("--quiet", action="store_true")
    a = ap.parse_args(argv)

    cfg = read_model_config(a.config)
    if a.preset:
        from ..training.presets import apply_preset
        apply_preset(cfg, a.preset)
    tiny = a.tiny or str(cfg.extra.get("arch", "")) == "tiny"
    m = manifest_from_config(cfg)
    cache_dir = cfg.cache_dir or cfg.dataset_cache_dir or cfg.dataset_path
    if not cache_dir or not os.path.isdir(cache_dir):
        print(f"error: no latent cache directory (cache_dir / dataset_cache_dir / dataset_path): '{cache_dir}'", file=sys.stderr)
        return 2
    controlnet = cfg.training_method.upper() == "CONTROLNET"
    if controlnet and m.family != "zimage":
        print(f"error: training_method CONTROLNET is defined for the Z-Image family, not '{m.family}'", file=sys.stderr)
        return 2
    try:
        cache = LatentCache(cache_dir, require_control=controlnet)
    except Exception as e:                                  # a ControlNet run needs control_latent in every sample
        print(f"error: latent cache: {e}", file=sys.stderr)
        return 2
    pf = preflight(cfg, m, cache, tiny)
    prompts = None
    pfile = cfg.validation_prompts_file or cfg.sample_definition_file_name
    if pfile and os.path.isfile(pfile):
        prompts = read_sample_prompts(pfile)
        if cfg.sample_every == 250 and prompts.sample_every != 250:
            cfg.sample_every = prompts.sample_every
        cfg.sample_at_start = cfg.sample_at_start or prompts.sample_at_start
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    loader_probe = BatchLoader(cache, cfg.batch_size, cfg.seed, rank=rank, world=world, pin=False)
    plan = {"schema": "mdb200.train_plan.v1", "model": m.model_id, "family": m.family, "method": cfg.training_method,
            "tiny": tiny, "total_steps": cfg.total_steps, "steps_per_epoch": loader_probe.steps_per_epoch(),
            "batch_size": cfg.batch_size, "world": world, "save_every": [cfg.save_every, cfg.save_every_unit],
            "sample_every": [cfg.sample_after or cfg.sample_every, cfg.sample_after_unit],
            "prompts": [p.id for p in prompts.prompts] if prompts else [], "optimizer": cfg.optimizer.optimizer,
            "lora": {"rank": cfg.lora_rank, "alpha": cfg.lora_alpha, "layout": adapter_for(m).lora_layout} if cfg.training_method.upper() == "LORA" else None,
            "workspace": cfg.workspace_dir, "output": cfg.output_model_destination, "cache": pf}
    if a.dry_run:
        print(json.dumps(plan))
        return 1 if pf["problems"] and any("channels" in p or "divisible" in p for p in pf["problems"]) else 0
    if any("channels" in p or "divisible" in p for p in pf["problems"]):
        print("error: cache preflight failed:\n  " + "\n  ".join(pf["problems"]), file=sys.stderr)
        return 2
    if loader_probe.steps_per_epoch() == 0:
        print("error: the cache yields no full batch", file=sys.stderr)
        return 2

    dev = pick_device(a.device)
    if world > 1:
        from ..parallel import dist as pdist
        if dev.type == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        pdist.init_from_env("nccl" if dev.type == "cuda" else "gloo")
    is_main = rank == 0
    model, weights = build_model(m, cfg, dev, tiny)
    adapter = adapter_for(m)
    method = cfg.training_method.upper()
    ocfg = cfg.optimizer
    okw = dict(lr=cfg.learning_rate, betas=(ocfg.beta1, ocfg.beta2), eps=ocfg.eps, weight_decay=ocfg.weight_decay,
               max_grad_norm=cfg.max_grad_norm)
    dp = None
    inventory = None
    if method == "LORA":
        slots = attach_lora(m, model, cfg.lora_rank, cfg.lora_alpha, None)
        params = L.lora_parameters(slots)
        if world > 1:
            from ..parallel.dp import broadcast_parameters
            broadcast_parameters(params)
        if world > 1 and dev.type == "cuda" and ocfg.optimizer.upper() in ("ADAMW", "ADAMW_FUSED", "ADAM"):
            from ..parallel.fused_dp import FusedDPAdamW
            opt = FusedDPAdamW(params, **okw)
        else:
            from ..training.optim_extra import create_optimizer
            opt = create_optimizer(ocfg.optimizer, params, cfg.learning_rate, (ocfg.beta1, ocfg.beta2), ocfg.eps, ocfg.weight_decay,
                                   cfg.max_grad_norm, ocfg.stochastic_rounding)
            if world > 1:
                from ..parallel.dp import DataParallelGrads
                dp = DataParallelGrads(params)
    elif method in ("FINE_TUNE", "FINETUNE", "FULL"):
        from ..training.full_finetune import prepare_full_finetune
        slots = []
        inventory, opt = prepare_full_finetune(model, cfg.learning_rate, betas=(ocfg.beta1, ocfg.beta2), eps=ocfg.eps,
                                               weight_decay=ocfg.weight_decay, max_grad_norm=cfg.max_grad_norm)
        params = [p for _, p in inventory]
        if world > 1:
            from ..parallel.dp import DataParallelGrads, broadcast_parameters
            broadcast_parameters(params)
            dp = DataParallelGrads(params)
    elif method == "CONTROLNET":
        # frozen base + trainable control branch (copy-from-base blocks, zero projections); its own optimizer group
        from ..models.zimage_controlnet import ControlledZImage, ZImageControlNet, load_controlnet
        from ..training.full_finetune import prepare_full_finetune
        slots = []
        n_ctrl = cfg.controlnet_layers or max(1, model.cfg.depth // 5)
        net = ZImageControlNet(model.cfg, n_ctrl, dtype=next(model.parameters()).dtype, device=dev).init_from_base(model)
        ck = str(cfg.extra.get("controlnet_checkpoint", ""))
        if ck:
            load_controlnet(net, ck)
        model = ControlledZImage(model, net, cfg.controlnet_scale)
        inventory, opt = prepare_full_finetune(net, cfg.learning_rate, betas=(ocfg.beta1, ocfg.beta2), eps=ocfg.eps,
                                               weight_decay=ocfg.weight_decay, max_grad_norm=cfg.max_grad_norm)
        params = [p for _, p in inventory]
        if world > 1:
            from ..parallel.dp import DataParallelGrads, broadcast_parameters
            broadcast_parameters(params)
            dp = DataParallelGrads(params)
    else:
        print(f"error: training_method '{cfg.training_method}' is not LORA, FINE_TUNE or CONTROLNET", file=sys.stderr)
        return 2
    if cfg.gradient_checkpointing.upper() != "OFF":
        for mod in (model, getattr(model, "base", None)):
            if mod is not None and hasattr(mod, "gradient_checkpointing"):
                mod.gradient_checkpointing = True
    model.train()
    trainer = FamilyTrainer(adapter, model, params, opt, cfg, dp, StepConfig(seed=cfg.seed, rank=rank, world=world,
                                                                              guidance=float(cfg.extra.get("train_guidance", 1.0))))
    loader = BatchLoader(cache, cfg.batch_size, cfg.seed, rank=rank, world=world, pin=dev.type == "cuda",
                         dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32)

    # ---- state for checkpoints ---------------------------------------------------------------------------------
    def named_trainables():
        if method == "LORA":
            return L.lora_state_onetrainer(slots) if adapter.lora_layout == "onetrainer" else L.lora_state_peft(slots)
        return OrderedDict((n, p.detach().contiguous().cpu()) for n, p in inventory)

    def optimizer_state():
        sd = OrderedDict()
        for i, p in enumerate(params):
            mom = getattr(opt, "moments", None)
            if mom is not None:
                m_, v_ = opt.moments(p)
                sd[f"adam_m.{i}"] = m_.detach().float().cpu()
                sd[f"adam_v.{i}"] = v_.detach().float().cpu()
        sd["__meta__"] = torch.tensor([float(getattr(opt, "step_count", 0)), 0.0], dtype=torch.float32)
        return sd

    def load_trainables(sd):
        with torch.no_grad():
            if method == "LORA":
                for s in slots:
                    for dn, un in ((f"{s.key}.lora_down.weight", f"{s.key}.lora_up.weight"), (f"{s.key}.lora_A.weight", f"{s.key}.lora_B.weight")):
                        if dn in sd:
                            s.down.copy_(sd[dn].to(s.down.device, s.down.dtype))
                            s.up.copy_(sd[un].to(s.up.device, s.up.dtype))
                            break
                    else:
                        raise KeyError(f"resume: no adapter tensors for {s.key}")
            else:
                for n, p in inventory:
                    p.copy_(sd[n].to(p.device, p.dtype))
                    if getattr(opt, "masters", None) is not None:
                        opt.masters[[id(q) for q in params].index(id(p))].copy_(sd[n].float().to(p.device))

    def load_optimizer_state(sd):
        if hasattr(opt, "set_moments"):
            for i, p in enumerate(params):
                if f"adam_m.{i}" in sd:
                    opt.set_moments(p, sd[f"adam_m.{i}"].view_as(p), sd[f"adam_v.{i}"].view_as(p))
        if "__meta__" in sd:
            opt.step_count = int(sd["__meta__"][0].item())

    # ---- validation sampling -----------------------------------------------------------------------------------
    sample_fn = None
    sample_dir = os.path.join(cfg.workspace_dir or ".", "samples")
    if prompts is not None and prompts.prompts:
        from ..training.validation_sampler import ValidationSampler
        vs = ValidationSampler(m, model, dev, tiny=tiny, vae_path=cfg.vae, keep_vae=True)

        def sample_fn(progress, leaf):
            return vs.sample_all(prompts.prompts, sample_dir, leaf, {"global_step": progress.global_step})

    def step_fn(batch, lr):
        loss = trainer.step(batch, lr=lr)
        gn = getattr(opt, "norm_out", None)
        if gn is None:
            gl = getattr(opt, "last_grad_norm", None)
            gn = gl.float().sqrt() if gl is not None else torch.zeros(())
        return loss, gn

    hooks = {}
    if world > 1:
        import torch.distributed as dist
        from ..parallel import dist as pdist
        hooks["barrier_fn"] = pdist.barrier
        if hasattr(opt, "gather_state"):
            hooks["pre_save_fn"] = opt.gather_state

        def agree(bits: int) -> int:
            t = torch.tensor([bits], dtype=torch.int64, device=dev if dist.get_backend() == "nccl" else "cpu")
            dist.broadcast(t, src=0)
            return int(t.item())
        hooks["agree_fn"] = agree
    if dev.type == "cuda":
        from ..ops import native
        hooks["status_check_fn"] = native.check_status

    run = TrainRun(cfg, loader, step_fn, named_trainables, optimizer_state, load_trainables, load_optimizer_state,
                   sample_fn=sample_fn, display=not a.quiet, is_main=is_main, prefix=str(cfg.extra.get("save_filename_prefix", "")),
                   backup_after=int(cfg.extra.get("backup_after", 0)), backup_after_unit=str(cfg.extra.get("backup_after_unit", "NEVER")),
                   loss_sync_every=int(cfg.extra.get("loss_sync_every", 1)), **hooks)
    resumed = run.resume_if_requested()
    if resumed:
        trainer.step_index = run.progress.global_step
    if is_main and cfg.output_model_destination:
        nbytes = sum(t.numel() * t.element_size() for t in named_trainables().values())
        guard_free_space(cfg.workspace_dir or ".", 3 * nbytes)
    total = cfg.total_steps
    if a.max_steps > 0:
        total = min(total, run.progress.global_step + a.max_steps)
    progress = run.run(max_steps=total)

    if is_main:
        final = cfg.output_model_destination
        dst = ""
        if final:
            dst = final if os.path.isabs(final) else os.path.join(cfg.workspace_dir or ".", final)
            if method == "LORA":
                if hasattr(opt, "gather_state") and world == 1:
                    opt.gather_state()
                L.save_lora_state_sidecar(dst[:-len(".safetensors")] + ".state.safetensors" if dst.endswith(".safetensors") else dst + ".state.safetensors",
                                          slots, opt, getattr(opt, "step_count", progress.global_step))
            else:
                from ..training.full_finetune import save_state
                save_state(dst[:-len(".safetensors")] + ".state.safetensors", inventory, opt, getattr(opt, "step_count", progress.global_step))
        report = {"schema": "mdb200.train_result.v1", "model": m.model_id, "weights": weights, "resumed": resumed,
                  "global_step": progress.global_step, "epoch": progress.epoch, "final_loss": run.losses[-1] if run.losses else None,
                  "first_loss": run.losses[0] if run.losses else None, "saved": run.saved, "output": dst, "adapters": len(slots)}
        print(json.dumps(report))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
