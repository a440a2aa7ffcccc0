#!/usr/bin/env python
"""Times each fused compute+collective path against its NCCL-only baseline and its roofline.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        benchmarks/bench_fused_paths.py [--json out.json]

Device-timed (CUDA events after warm-up, barrier + synchronize on both sides), max over ranks. Roofline of a path =
max(FLOPs / measured bf16 peak, bytes that must cross NVLink per GPU / 770 GB/s measured per direction).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mojodiffusion_b200.ops as O  # noqa: E402
from mojodiffusion_b200.ops import native  # noqa: E402
from mojodiffusion_b200.parallel import dist as pdist  # noqa: E402

LINK_GBS = 770.0


def timed(fn, iters=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    pdist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    pdist.barrier()
    return pdist.max_over_ranks(e0.elapsed_time(e1) / iters)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    pdist.init_from_env("nccl")
    rank, world = pdist.rank(), pdist.world_size()
    dev = torch.device("cuda", pdist.env_local_rank())
    native.load(True)
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    peak = peaks.get("bf16_tflops", 1590.0) * 1e12
    rows = []
    g = torch.Generator().manual_seed(rank)

    # ---- path 1: Ulysses attention layer, FLUX shape ---------------------------------------------------------
    from mojodiffusion_b200.parallel.ulysses import UlyssesContext
    B, S_txt, S_img, H, Dh = 1, 512, 4096, 24, 128
    D = H * Dh
    w = (torch.randn(3 * D, D, generator=g) * 0.02).bfloat16().to(dev)
    bq = torch.zeros(3 * D, dtype=torch.bfloat16, device=dev)
    wn = torch.ones(Dh, dtype=torch.bfloat16, device=dev)
    for mode in ("nccl", "fused"):
        sp = UlyssesContext(B, S_txt, S_img, H, Dh, mode=mode, device=dev)
        xt = torch.randn(B, sp.St, D, generator=g).bfloat16().to(dev)
        xi = torch.randn(B, sp.Si, D, generator=g).bfloat16().to(dev)
        pos = torch.zeros(sp.S, 3, device=dev)
        cos, sin = O.rope_table(pos, (16, 56, 56), 10000.0)

        def layer():
            with torch.no_grad():
                sp.scatter_qkv(xt, w, bq, "txt")
                sp.scatter_qkv(xi, w, bq, "img")
                sp.finish_scatter()
                sp.attention(wn, wn, wn, wn, cos, sin)
                sp.finish_attention()
        ms = timed(layer)
        S = S_txt + S_img
        flops = 2.0 * (S / world) * D * 3 * D + 4.0 * S * S * D / world
        nv_bytes = (S / world) * 3 * D * 2 * (world - 1) / world + S * (D / world) * 2 * (world - 1) / world
        roof = max(flops / peak, nv_bytes / (LINK_GBS * 1e9)) * 1e3
        rows.append({"path": "1 ulysses qkv-gemm + a2a + attention + a2a", "mode": mode, "ms": ms, "roofline_ms": roof,
                     "frac_of_roofline": roof / ms})
        del sp

    # ---- path 2: TP MLP, LTX shape --------------------------------------------------------------------------------
    from mojodiffusion_b200.parallel.tensor_parallel import TPContext, shard_mlp_weights
    R, Dm, F = 6144, 4096, 16384
    w1 = (torch.randn(F // world, Dm, generator=g) * 0.02).bfloat16().to(dev)
    b1 = torch.zeros(F // world, dtype=torch.bfloat16, device=dev)
    w2 = (torch.randn(Dm, F // world, generator=g) * 0.02).bfloat16().to(dev)
    b2 = torch.zeros(Dm, dtype=torch.bfloat16, device=dev)
    xl = torch.randn(R // world, Dm, generator=g).bfloat16().to(dev)
    for mode in ("nccl", "fused"):
        tp = TPContext(R, Dm, mode=mode, device=dev)
        ms = timed(lambda: tp.mlp(xl, w1, b1, w2, b2, "gelu_tanh", xl, None, R))
        flops = 2.0 * 2.0 * R * Dm * F / world
        nv_bytes = (R / world) * Dm * 2 * (world - 1) + R * Dm * 4 * (world - 1) / world
        roof = max(flops / peak, nv_bytes / (LINK_GBS * 1e9)) * 1e3
        rows.append({"path": "2 tp mlp ag->gemm, gemm->rs", "mode": mode, "ms": ms, "roofline_ms": roof,
                     "frac_of_roofline": roof / ms})
        del tp

    # ---- path 3: DP LoRA all-reduce + clip + AdamW -------------------------------------------------------------------
    from mojodiffusion_b200.parallel.fused_dp import FusedDPAdamW
    from mojodiffusion_b200.training.optim import FusedAdamW
    n_par = 65_000_000
    shapes = [(16, 3072)] * 300 + [(3072, 16)] * 300
    k = n_par // (2 * 300 * 16 * 3072) + 1
    shapes = shapes * k
    params = [torch.nn.Parameter(torch.zeros(*s, dtype=torch.bfloat16, device=dev)) for s in shapes]
    numel = sum(p.numel() for p in params)
    opt = FusedDPAdamW(params, lr=1e-4, max_grad_norm=1.0)
    opt.flat_grads.normal_()
    ms = timed(lambda: opt.step())
    nv_bytes = numel * 2 * (world - 1) / world * 2        # grads in + params out, per GPU
    hbm_bytes = numel / world * (4 * 5 + 2)
    roof = max(nv_bytes / (LINK_GBS * 1e9), hbm_bytes / (peaks.get("hbm_gbs", 6650.0) * 1e9)) * 1e3
    rows.append({"path": "3 dp reduce-scatter + clip + adamw + all-gather", "mode": "fused" + (" (multimem)" if opt.symm.mc_ptr else ""),
                 "ms": ms, "roofline_ms": roof, "frac_of_roofline": roof / ms, "numel": numel})
    params2 = [torch.nn.Parameter(torch.zeros(*s, dtype=torch.bfloat16, device=dev)) for s in shapes]
    flat = torch.zeros(numel, dtype=torch.bfloat16, device=dev).normal_()
    off = 0
    for p in params2:
        p.grad = flat[off:off + p.numel()].view_as(p)
        off += p.numel()
    base = FusedAdamW(params2, lr=1e-4, max_grad_norm=1.0)

    def nccl_step():
        dist.all_reduce(flat)
        base.step(grad_scale=1.0 / world)
    ms = timed(nccl_step)
    rows.append({"path": "3 dp all-reduce (NCCL) + fused AdamW on every rank", "mode": "nccl", "ms": ms})
    del opt, base, params, params2, flat

    # ---- path 4: FSDP linear fwd+bwd ---------------------------------------------------------------------------------
    from mojodiffusion_b200.parallel.fsdp import FSDPContext, FSDPLinear
    Rr, Di, Do = 4608, 3072, 12288
    for mode in ("nccl", "fused"):
        ctx = FSDPContext(mode=mode, device=dev)
        lay = FSDPLinear(ctx, Di, Do, bias=False, seed=1)
        ctx.finalize()
        x = torch.randn(Rr, Di, generator=g).bfloat16().to(dev).requires_grad_(True)
        dy = torch.randn(Rr, Do, generator=g).bfloat16().to(dev)

        def fb():
            y = lay(x)
            y.backward(dy)
            ctx.gathered_owner = None        # as in a real model: another layer has reused the buffer by then
        ms = timed(fb, iters=6)
        flops = 3 * 2.0 * Rr * Di * Do
        nv_bytes = Do * Di * 2 * (world - 1) / world * 2 + Do * Di * 4 * (world - 1) / world
        roof = max(flops / peak, nv_bytes / (LINK_GBS * 1e9)) * 1e3
        rows.append({"path": "4 fsdp linear: ag->gemm fwd, dx, dW gemm->rs", "mode": mode, "ms": ms, "roofline_ms": roof,
                     "frac_of_roofline": roof / ms})
        del ctx, lay
    native.check_status()
    if rank == 0:
        for r in rows:
            print(json.dumps({"n_gpus": world, **r}))
        if args.json:
            json.dump({"n_gpus": world, "rows": rows}, open(args.json, "w"), indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
