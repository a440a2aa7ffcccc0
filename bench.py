#!/usr/bin/env python
"""Headline benchmark: FLUX.1-dev-shaped 12B MMDiT, 1024x1024 (4096 image tokens + 512 text tokens), bf16,
28-step Euler flow-matching denoise loop -> denoise iterations per second (one iteration = one full 57-block
forward + sampler update), plus LoRA (rank 16) training samples per second on the same backbone.

    python bench.py --gpus N --steps K --warmup W            # N > 1: launched by torch.distributed.run

Timing: W untimed warm-up steps, then exactly K steps between CUDA events on the launching stream, bracketed by a
barrier + synchronize; the reported time is the max over ranks. Inputs are synthetic N(0,1) tensors of the named
shapes and the weights are random-init from seed 0 (no datasets or checkpoints exist offline). Each step streams
24 GB of weights, far more than the 126 MB L2, so no explicit L2 flush is needed between iterations.

On N > 1 GPUs the headline value is throughput under weak scaling with every step crossing NVLink: a global batch of N
samples, each sample's tokens sharded over the N ranks (Ulysses sequence parallel, the all-to-alls fused into the QKV GEMM
and attention epilogues), so that every GPU does the work of one sample per step (N x S/N token rows in the linears, N
samples x H/N heads in attention). The same run also reports N independent replicas (one sample per GPU, no collective:
``replicas_no_comm``) and ONE sample sharded over the N GPUs (``strong_scaling_sp``). LoRA training is data parallel with
the gradient reduce-scatter, AdamW and parameter all-gather in one peer-memory pass.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

PUBLISHED_NEAREST = {"what": "Z-Image 6B 1024^2 denoise, RTX 3090 Ti (reference's nearest published analogue)",
                     "it_per_s": 0.23}


def _parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "torch"],
                    help="ours: the sm_100a kernels; reference: the upstream project (not installable offline); torch: the same "
                         "model code with every op routed to PyTorch library kernels (cuBLAS, SDPA, NCCL) as a same-box baseline")
    ap.add_argument("--batch", type=int, default=1, help="images per GPU")
    ap.add_argument("--model", default="flux1-dev", choices=["flux1-dev", "tiny"])
    ap.add_argument("--train-steps", type=int, default=-1, help="LoRA train steps to time (-1: min(steps, 4); 0: skip)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-train-graph", action="store_true", help="launch the training step's forward + backward eagerly instead of replaying one CUDA graph")
    ap.add_argument("--no-graph", action="store_true", help="launch the forward eagerly instead of replaying a CUDA graph")
    ap.add_argument("--sp-mode", default="fused", choices=["fused", "nccl"], help="Ulysses all-to-all: fused peer stores or NCCL baseline")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=3)
        except Exception:
            pass
        sm, mx, reasons, power = [], [], set(), []
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


def main():
    args = _parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference",
                          "unavailable": "reference is Mojo/MAX source with no setup.py/pyproject.toml: pip reports "
                                         "'Directory is not installable'; no mojo/pixi toolchain offline"}))
        return 0
    lib_baseline = args.impl == "torch"
    if lib_baseline:
        os.environ["MDB200_FORCE_REFERENCE"] = "1"
        args.sp_mode = "nccl"
        if args.train_steps < 0 or args.model != "tiny":
            # the library arm times the denoise loop. Its training step exists for the tiny model only: at the 12B shape the
            # backward pass of the PyTorch library kernels raised an illegal memory access twice on B200, so it is not offered
            args.train_steps = 0

    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from mojodiffusion_b200.models.mmdit import MMDiT, flux1_dev_config, tiny_mmdit_config
    from mojodiffusion_b200.ops import native
    from mojodiffusion_b200.parallel import dist as pdist
    from mojodiffusion_b200.pipeline import FluxPipeline
    from mojodiffusion_b200.sampling import flow_match as fm

    world = pdist.env_world()
    rank = pdist.env_rank()
    local = pdist.env_local_rank()
    assert torch.cuda.is_available(), "bench.py needs a GPU"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        pdist.init_from_env("nccl")
    native.load(True)
    launches = torch.ops.mdb200.launch_count
    if lib_baseline and world > 1 and args.train_steps != 0:
        args.no_e2e = True   # library baseline at N > 1: data-parallel training only (no library Ulysses path is kept)

    cfg = flux1_dev_config() if args.model == "flux1-dev" else tiny_mmdit_config()
    S_img, S_txt = (4096, 512) if args.model == "flux1-dev" else (256, 64)
    hw = (64, 64) if args.model == "flux1-dev" else (16, 16)
    B = args.batch
    model = MMDiT(cfg, dtype=torch.bfloat16, device=dev).init_weights(0)
    model.eval()
    sigmas = fm.flux1_sigmas(28, S_img)
    K, W = args.steps, max(args.warmup, 0)
    from mojodiffusion_b200 import ops
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ids = MMDiT.make_ids(hw[0], hw[1], S_txt, dev)

    def measure(sp, seed, shard, with_e2e, B=B):
        """Times K denoise steps (device events, max over ranks) and, optionally, K steps through the public API with the
        step's inputs coming from pinned host memory and its result read back. ``shard``: this rank holds 1/world of the
        tokens of each of the B shared samples (sequence parallel); otherwise every rank denoises its own B samples."""
        pipe = FluxPipeline(model, dev, sp=sp, use_cuda_graph=not args.no_graph)
        g = torch.Generator().manual_seed(seed)
        x_full = torch.randn(B, S_img, cfg.in_channels, generator=g)
        txt_full = torch.randn(B, S_txt, cfg.context_dim, generator=g).to(torch.bfloat16)
        y_full = torch.randn(B, cfg.vec_dim, generator=g).to(torch.bfloat16)
        if shard:
            Sl_img, Sl_txt = S_img // world, S_txt // world
            x_full = x_full[:, rank * Sl_img:(rank + 1) * Sl_img]
            txt_full = txt_full[:, rank * Sl_txt:(rank + 1) * Sl_txt]
        x_host, txt_host, y_host = x_full.contiguous().pin_memory(), txt_full.contiguous().pin_memory(), y_full.pin_memory()
        out_host = torch.empty_like(x_host).pin_memory()
        x, txt, y = x_host.to(dev), txt_host.to(dev), y_host.to(dev)
        xb = x.to(torch.bfloat16)
        gvec = torch.full((B,), 3.5, device=dev)
        tvec = torch.empty((B,), device=dev)

        def denoise_step(i):
            s_, s_next = sigmas[i % 28], sigmas[i % 28 + 1]
            tvec.fill_(float(s_))
            with torch.no_grad():
                v = pipe._forward(xb, txt, tvec, y, gvec, ids)
                ops.cfg_euler(x, v, None, dt=float(s_next - s_), mode=0, x_bf16=xb)

        for i in range(max(W, 1)):
            denoise_step(i)
        torch.cuda.synchronize()
        pdist.barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        n0 = launches()
        torch.cuda.synchronize()
        e0.record()
        for i in range(K):
            denoise_step(W + i)
        e1.record()
        torch.cuda.synchronize()
        pdist.barrier()
        res = {"n_launch": launches() - n0, "launches_per_step": None}
        res["clocks"] = sampler.stop() if rank == 0 else None
        res["ms"] = pdist.max_over_ranks(e0.elapsed_time(e1) / K)
        native.check_status()
        assert torch.isfinite(x).all(), "latents diverged"
        if not args.no_graph and not lib_baseline:
            # kernels inside the replayed graph are not re-counted by the host-side counter: count one eager step
            pipe_eager = FluxPipeline(model, dev, sp=sp, use_cuda_graph=False)
            nb = launches()
            with torch.no_grad():
                pipe_eager._forward(xb, txt, tvec, y, gvec, ids)
            torch.cuda.synchronize()
            pdist.barrier()
            res["launches_per_step"] = launches() - nb + 1
            res["n_launch"] = res["launches_per_step"] * K
        res["e2e"] = None
        if with_e2e:
            for i in range(min(max(W, 1), 2)):
                pipe.step_from_host(x_host, txt_host, y_host, sigmas[i], sigmas[i + 1], 3.5, out_host, hw)
            torch.cuda.synchronize()
            pdist.barrier()
            torch.cuda.synchronize()
            e0.record()
            bi = bo = 0
            for i in range(K):
                bi, bo = pipe.step_from_host(x_host, txt_host, y_host, sigmas[i % 28], sigmas[i % 28 + 1], 3.5, out_host, hw)
                torch.cuda.current_stream().synchronize()   # the caller reads the step's result on the host
                x_host.copy_(out_host)
            e1.record()
            torch.cuda.synchronize()
            ms_e2e = pdist.max_over_ranks(e0.elapsed_time(e1) / K)
            images = B if shard else B * world
            res["e2e"] = {"value": images * 1000.0 / ms_e2e, "unit": "it/s", "ms_per_step": ms_e2e,
                          "h2d_bytes_per_step": bi * world, "d2h_bytes_per_step": bo * world}
        del pipe
        return res

    # ------------------------------------------------------------------ denoise loop
    # N = 1: one sample on one GPU. N > 1, headline (weak scaling): global batch N x B, every sample's tokens sharded over the
    # N ranks (Ulysses sequence parallel, all-to-alls fused into the QKV GEMM and attention epilogues): per-GPU work equals
    # the one-GPU run and every attention layer crosses NVLink twice. Also reported: N replicas without communication, and
    # (strong scaling) ONE sample sharded over the ranks.
    do_denoise = not (lib_baseline and world > 1)
    ms = it_per_s = clocks = launches_per_step = e2e = strong = replicas = None
    n_launch = 0
    headline_sp = do_denoise and world > 1 and not lib_baseline
    if headline_sp:
        from mojodiffusion_b200.parallel.ulysses import UlyssesContext
        GB = B * world
        sp_w = UlyssesContext(GB, S_txt, S_img, cfg.heads, cfg.head_dim, mode=args.sp_mode, device=dev)
        head = measure(sp_w, 1234, True, not args.no_e2e, B=GB)
        ms, clocks, launches_per_step, n_launch, e2e = head["ms"], head["clocks"], head["launches_per_step"], head["n_launch"], head["e2e"]
        it_per_s = GB * 1000.0 / ms
        del sp_w
        torch.cuda.empty_cache()
        try:
            rep = measure(None, 1234 + rank, False, False)
            replicas = {"what": "one independent sample per GPU, no communication inside the step", "value": world * B * 1000.0 / rep["ms"],
                        "unit": "it/s", "ms_per_step": rep["ms"]}
        except Exception as ex:
            replicas = {"error": str(ex)[:300]}
    elif do_denoise:
        head = measure(None, 1234 + rank, False, not args.no_e2e)
        ms, clocks, launches_per_step, n_launch, e2e = head["ms"], head["clocks"], head["launches_per_step"], head["n_launch"], head["e2e"]
        it_per_s = world * B * 1000.0 / ms

    # ------------------------------------------------------------------ LoRA training samples/s
    train = None
    tsteps = min(K, 4) if args.train_steps < 0 else args.train_steps
    if tsteps > 0:
        from mojodiffusion_b200.parallel.dp import DataParallelGrads
        from mojodiffusion_b200.training import lora as L
        from mojodiffusion_b200.training.optim import FusedAdamW
        from mojodiffusion_b200.training.trainer import FlowMatchTrainer
        torch.cuda.empty_cache()
        slots = L.inject_flux_lora(model, rank=16, alpha=16.0)
        params = L.lora_parameters(slots)
        model.train()
        dp = None
        if lib_baseline:
            class _TorchAdamW:
                """torch.optim.AdamW (fused) + clip_grad_norm_ behind the trainer's optimizer interface."""

                def __init__(self, ps):
                    self.ps = ps
                    self.opt = torch.optim.AdamW(ps, lr=1e-4, betas=(0.9, 0.999), weight_decay=0.01, fused=True)

                def zero_grad(self, set_to_none=True):
                    self.opt.zero_grad(set_to_none=set_to_none)

                def step(self, grad_scale=1.0, lr=None):
                    if grad_scale != 1.0:
                        torch._foreach_mul_([p.grad for p in self.ps if p.grad is not None], grad_scale)
                    torch.nn.utils.clip_grad_norm_(self.ps, 1.0)
                    self.opt.step()

            opt = _TorchAdamW(params)
            dp = DataParallelGrads(params) if world > 1 else None
        elif world > 1:
            from mojodiffusion_b200.parallel.fused_dp import FusedDPAdamW
            opt = FusedDPAdamW(params, lr=1e-4, betas=(0.9, 0.999), weight_decay=0.01, max_grad_norm=1.0)
        else:
            opt = FusedAdamW(params, lr=1e-4, betas=(0.9, 0.999), weight_decay=0.01, max_grad_norm=1.0)
        gt = torch.Generator().manual_seed(99 + rank)   # data parallel: every rank trains on its own samples
        x0 = torch.randn(B, S_img, cfg.in_channels, generator=gt).to(dev)
        txt = torch.randn(B, S_txt, cfg.context_dim, generator=gt).to(dev, torch.bfloat16)
        y = torch.randn(B, cfg.vec_dim, generator=gt).to(dev, torch.bfloat16)

        def time_train(ckpt: bool):
            model.gradient_checkpointing = ckpt
            tr = FlowMatchTrainer(model, params, opt, dp, use_cuda_graph=not args.no_train_graph and not lib_baseline)
            want_graph = tr.use_cuda_graph
            tr.use_cuda_graph = False
            l0 = launches()
            tr.step(x0, txt, y, hw=hw)                       # one eager step: also counts the kernels of a step
            torch.cuda.synchronize()
            train_launches_per_step = launches() - l0
            if want_graph:
                ok_graph = 1
                tr.use_cuda_graph = True
                try:
                    tr.step(x0, txt, y, hw=hw)               # warms up, captures forward + backward, replays once
                    torch.cuda.synchronize()
                except Exception as ex:                      # capture refused: report it and time the eager step instead
                    ok_graph = 0
                    sys.stderr.write(f"[bench] training graph capture failed, timing the eager step: {ex}\n")
                if world > 1:
                    flag = torch.tensor([ok_graph], device=dev)
                    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                    ok_graph = int(flag.item())
                if not ok_graph:
                    tr.use_cuda_graph, tr._graphed = False, None
            for i in range(2):
                tr.step(x0, txt, y, hw=hw)
            torch.cuda.synchronize()
            pdist.barrier()
            t0n = launches()
            e0.record()
            for i in range(tsteps):
                loss = tr.step(x0, txt, y, hw=hw)
            e1.record()
            torch.cuda.synchronize()
            pdist.barrier()
            ms_t = pdist.max_over_ranks(e0.elapsed_time(e1) / tsteps)
            native.check_status()
            return {"metric": "lora_train_samples_per_s", "value": world * B * 1000.0 / ms_t, "unit": "samples/s",
                     "ms_per_step": ms_t, "steps": tsteps, "warmup": 3, "loss": float(loss), "rank": 16,
                     "gpu_launches": (train_launches_per_step * tsteps if tr._graphed is not None else launches() - t0n),
                     "launches_per_step": train_launches_per_step, "gradient_checkpointing": ckpt, "cuda_graph": bool(tr._graphed is not None),
                     "parallelism": f"dp{world}, NCCL all-reduce + torch AdamW" if (lib_baseline and world > 1) else (f"dp{world}, grad reduce-scatter + clip + AdamW + param all-gather fused in peer-memory "
                                     f"kernels (multicast {'on' if getattr(opt, 'symm', None) is not None and opt.symm.mc_ptr else 'off'})")
                     if world > 1 else "single"}

        # the reference's trainer recomputes every block in backward (24 GB cards); with 180 GB the activations of all 57
        # blocks stay resident, so the same step is also timed without recompute
        train = time_train(True)
        if not lib_baseline and args.model == "flux1-dev":
            try:
                nr = time_train(False)
                train["activations_resident"] = {k: nr[k] for k in ("value", "unit", "ms_per_step", "loss", "launches_per_step", "cuda_graph", "gradient_checkpointing")}
                train["activations_resident"]["peak_gib"] = round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)
            except torch.OutOfMemoryError as ex:
                train["activations_resident"] = {"error": str(ex)[:200]}

    # ------------------------------------------------------------------ one sample over all GPUs (strong scaling)
    # Runs last and guarded: a failure here must not cost the numbers above.
    if do_denoise and world > 1 and not lib_baseline:
        try:
            from mojodiffusion_b200.parallel.ulysses import UlyssesContext
            model.eval()
            for mod in model.modules():                   # drop the adapters the training section attached
                if hasattr(mod, "slots") and len(mod.slots):
                    mod.slots = torch.nn.ModuleList()
            torch.cuda.empty_cache()
            sp = UlyssesContext(B, S_txt, S_img, cfg.heads, cfg.head_dim, mode=args.sp_mode, device=dev)
            st = measure(sp, 1234, True, False)
            strong = {"what": "one sample sharded over the ranks (Ulysses sequence parallel, all-to-all " + args.sp_mode + ")",
                      "value": B * 1000.0 / st["ms"], "unit": "it/s", "ms_per_step": st["ms"], "scaling": "strong",
                      "launches_per_step": st["launches_per_step"], "e2e": st["e2e"]}
        except Exception as ex:
            strong = {"error": str(ex)[:300]}

    if rank == 0:
        line = {
            "metric": "flux1-dev-shape 1024^2 denoise it/s (+ LoRA r16 train samples/s in 'lora_train')",
            "value": it_per_s, "unit": "it/s", "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "torch library kernels (cuBLAS, SDPA, NCCL), eager" if lib_baseline else "ours",
            "config": {"model": f"{cfg.name} 12B MMDiT (19 double + 38 single, D=3072, 24x128)" if args.model == "flux1-dev" else cfg.name,
                       "global_batch": B * world, "seq_len": S_img + S_txt, "image_tokens": S_img, "text_tokens": S_txt,
                       "sampler": "euler flow-match, 28-step BFL-shifted schedule, guidance 3.5 (distilled)",
                       "parallelism": (f"ulysses sp{world}: global batch {B * world}, every sample's tokens sharded over the {world} GPUs, "
                                       f"all-to-all ({args.sp_mode}) inside the QKV GEMM and attention epilogues; replicas without "
                                       "communication in 'replicas_no_comm', one sample over all GPUs in 'strong_scaling_sp'"
                                       if headline_sp else (f"dp{world} replicas" if world > 1 else "single")),
                       "cuda_graph": not args.no_graph, "launches_per_step": launches_per_step,
                       "weights": "random-init seed 0",
                       "l2": "inputs larger than L2: 24 GB of weights stream every step"},
            "clocks": clocks, "gpu_launches": n_launch, "e2e": e2e, "replicas_no_comm": replicas, "strong_scaling_sp": strong,
            "lora_train": train,
            "published_nearest": PUBLISHED_NEAREST,
            "vs_published_nearest": it_per_s / PUBLISHED_NEAREST["it_per_s"] if it_per_s else None,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
