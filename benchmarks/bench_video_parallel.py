#!/usr/bin/env python
"""LTX-2-shaped 48-layer video DiT, 6144 latent tokens (8 x 24 x 32) + 256 context tokens, ONE sample with its tokens
sharded over N GPUs: Ulysses self-attention (inverse all-to-all fused into the attention epilogue) + tensor-parallel
feed-forward (all-gather inside GEMM 1, reduce-scatter out of GEMM 2's epilogue) against the same program on NCCL
collectives. Denoise iterations per second (forward + Euler update), CUDA events, barrier + synchronize on both sides,
max over ranks; random-init weights, synthetic inputs.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/bench_video_parallel.py [--json out.json]
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojodiffusion_b200.ops import native  # noqa: E402
from mojodiffusion_b200.parallel import dist as pdist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tiny", action="store_true")
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    world, rank, local = pdist.env_world(), pdist.env_rank(), pdist.env_local_rank()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        pdist.init_from_env("nccl")
    native.load(True)
    from mojodiffusion_b200.models.video_dit import VideoDiT, ltx2_config, tiny_video_dit_config
    from mojodiffusion_b200.parallel.video_parallel import ParallelVideoDiT
    cfg = tiny_video_dit_config() if args.tiny else ltx2_config()
    grid = (4, 8, 8) if args.tiny else (8, 24, 32)
    S = grid[0] * grid[1] * grid[2]
    model = VideoDiT(cfg, torch.bfloat16, dev).init_weights(0).eval()
    g = torch.Generator().manual_seed(7)
    x_full = torch.randn(1, S, cfg.in_channels, generator=g).to(dev)
    ctx = torch.randn(1, 16 if args.tiny else 256, cfg.context_dim, generator=g).to(dev, torch.bfloat16)
    t = torch.full((1,), 0.7, device=dev)
    rows = []
    for mode in ("fused", "nccl"):
        par = ParallelVideoDiT(model, grid, mode=mode, device=dev)
        x = par.shard(x_full).float()

        def step():
            with torch.no_grad():
                v = par.forward(x, ctx, t)
                x.add_(v.float(), alpha=-0.025)

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        pdist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        pdist.barrier()
        ms = pdist.max_over_ranks(e0.elapsed_time(e1) / args.steps)
        native.check_status()
        rows.append({"mode": mode, "n_gpus": world, "model": cfg.name, "tokens": S, "ms_per_step": ms, "it_per_s": 1000.0 / ms,
                     "finite": bool(torch.isfinite(x).all())})
        del par
        torch.cuda.empty_cache()
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.json:
            json.dump(rows, open(args.json, "w"), indent=1)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
