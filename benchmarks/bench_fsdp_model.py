#!/usr/bin/env python
"""Full finetune of a Qwen-Image-shaped MMDiT (60 blocks, 20 B parameters) with every large linear fully sharded over the
ranks: weight all-gather inside the consuming GEMM, dW reduce-scatter out of the producing GEMM's epilogue, fp32 master
shards with AdamW moments per rank. Device-timed (CUDA events, barrier + synchronize on both sides, max over ranks);
synthetic latents / text states of the 1024^2 shapes (4096 image + 512 text tokens), random-init weights from seed 0,
batch 1 per rank, gradient checkpointing per block.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_fsdp_model.py \
        [--mode fused|nccl] [--tiny] [--depth D] [--steps K] [--warmup W] [--json out.json]

The parameter, gradient, master and moment shards need about 18 bytes per parameter divided by N per GPU: the 20 B model
fits from N = 4 (about 90 GB per GPU); ``--depth`` cuts the block count for smaller N.
"""
import argparse
import dataclasses
import json
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojodiffusion_b200 import ops  # noqa: E402
from mojodiffusion_b200.ops import native  # noqa: E402
from mojodiffusion_b200.parallel import dist as pdist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--fuse-optimizer", action="store_true", help="AdamW of the sharded weights inside the reduce-scatter tail of backward")
    ap.add_argument("--offload-optimizer", action="store_true", help="fp32 masters and AdamW moments in pinned host memory, streamed per layer in step()")
    ap.add_argument("--depth", type=int, default=0, help="number of blocks (0: the architecture's own)")
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    world, rank, local = pdist.env_world(), pdist.env_rank(), pdist.env_local_rank()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        pdist.init_from_env("nccl")
    native.load(True)
    from mojodiffusion_b200.models.qwen_image import QwenImageDiT, qwen_image_config, tiny_qwen_image_config
    from mojodiffusion_b200.parallel.dp import DataParallelGrads
    from mojodiffusion_b200.parallel.fsdp import FSDPContext, shard_model
    from mojodiffusion_b200.training.optim import FusedAdamW

    cfg = tiny_qwen_image_config() if args.tiny else qwen_image_config()
    if args.depth > 0:
        cfg = dataclasses.replace(cfg, depth=args.depth)
    hw, S_txt = ((8, 8), 16) if args.tiny else ((64, 64), 512)
    t0 = time.time()
    model = QwenImageDiT(cfg, torch.bfloat16, dev).init_weights(0)
    n_params = sum(p.numel() for p in model.parameters())
    ctx = FSDPContext(mode=args.mode, device=dev, fuse_optimizer=args.fuse_optimizer and args.mode == "fused",
                      offload_optimizer=args.offload_optimizer)
    n_sharded = shard_model(model, ctx)
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()       # the peak of the training steps, not of building the unsharded model
    rest = [p for p in model.parameters() if p.numel() > 0]
    for p in rest:
        p.requires_grad_(True)
    dp = DataParallelGrads(rest) if world > 1 else None
    opt = FusedAdamW(rest, lr=1e-5, weight_decay=0.01, max_grad_norm=0.0, master_weights=True)
    model.gradient_checkpointing = True
    model.train()
    t_init = time.time() - t0

    g = torch.Generator().manual_seed(100 + rank)
    x0 = torch.randn(1, hw[0] * hw[1], cfg.in_channels, generator=g).to(dev)
    eps = torch.randn(1, hw[0] * hw[1], cfg.in_channels, generator=g).to(dev)
    txt = torch.randn(1, S_txt, cfg.context_dim, generator=g).to(dev, torch.bfloat16)
    t = torch.full((1,), 0.5, device=dev)

    def step():
        if dp is not None:
            dp.zero_grad()
        else:
            opt.zero_grad(set_to_none=True)
        if ctx.fused_active():
            ctx.begin_step(lr=1e-5)
        xt, target = ops.flow_match(x0, eps, t)
        loss = ops.mse_loss(model(xt.to(torch.bfloat16), txt, t, hw), target)
        loss.backward()
        scale = dp.sync() if dp is not None else 1.0
        opt.step(grad_scale=scale)
        ctx.step(lr=1e-5)
        return loss.detach()

    losses = []
    for _ in range(args.warmup):
        losses.append(step())
    torch.cuda.synchronize()
    pdist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        losses.append(step())
    e1.record()
    torch.cuda.synchronize()
    pdist.barrier()
    ms = pdist.max_over_ranks(e0.elapsed_time(e1) / args.steps)
    native.check_status()
    peak = torch.cuda.max_memory_allocated() / 2 ** 30
    if rank == 0:
        row = {"metric": "full-finetune samples/s", "value": world * 1000.0 / ms, "ms_per_step": ms, "n_gpus": world,
               "mode": args.mode + ("+optimizer-in-backward" if ctx.fused_active() else "") + ("+optimizer-state-on-host" if args.offload_optimizer else ""), "model": cfg.name, "depth": cfg.depth, "params_b": n_params / 1e9,
               "sharded_linears": n_sharded, "tokens": hw[0] * hw[1] + S_txt, "batch_per_gpu": 1,
               "gradient_checkpointing": True, "peak_gib_rank0": peak, "init_s": t_init,
               "losses": [float(l) for l in losses], "steps": args.steps, "warmup": args.warmup}
        print(json.dumps(row), flush=True)
        if args.json:
            json.dump(row, open(args.json, "w"), indent=1)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
