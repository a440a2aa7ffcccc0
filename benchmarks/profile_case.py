#!/usr/bin/env python
"""One small, self-terminating workload per kernel for profiler captures (a few launches, < 1 GB on the device).

    python benchmarks/profile_case.py --op gemm --shape 4608,3072,3072 --iters 3
    python benchmarks/profile_case.py --op attention --shape 1,4608,24,128
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mojodiffusion_b200.ops as O  # noqa: E402
from mojodiffusion_b200.ops import native  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "attention", "attention_bwd", "norm", "gemm_fp8", "flux_step", "flux_train_step"])
    ap.add_argument("--shape", default="")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    dev = "cuda"
    native.load(True)
    dims = [int(x) for x in a.shape.split(",")] if a.shape else []
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if a.op in ("flux_step", "flux_train_step"):
        from mojodiffusion_b200.models.mmdit import MMDiT, flux1_dev_config
        cfg = flux1_dev_config()
        model = MMDiT(cfg, dtype=torch.bfloat16, device=dev).init_weights(0)
        B, S_img, S_txt = 1, 4096, 512
        x = torch.randn(B, S_img, 64, device=dev)
        txt = torch.randn(B, S_txt, 4096, device=dev, dtype=torch.bfloat16)
        y = torch.randn(B, 768, device=dev, dtype=torch.bfloat16)
        g = torch.full((B,), 3.5, device=dev)
        ids = MMDiT.make_ids(64, 64, S_txt, dev)
        if a.op == "flux_step":
            xb = x.to(torch.bfloat16)

            def fn():
                with torch.no_grad():
                    v = model(xb, txt, torch.full((B,), 0.7, device=dev), y, g, ids=ids)
                    O.cfg_euler(x, v, None, dt=-0.03, mode=0, x_bf16=xb)
        else:
            from mojodiffusion_b200.training import lora as L
            from mojodiffusion_b200.training.optim import FusedAdamW
            from mojodiffusion_b200.training.trainer import FlowMatchTrainer
            slots = L.inject_flux_lora(model, rank=16, alpha=16.0)
            params = L.lora_parameters(slots)
            model.gradient_checkpointing = True
            tr = FlowMatchTrainer(model, params, FusedAdamW(params, lr=1e-4, max_grad_norm=1.0))
            fn = lambda: tr.step(x, txt, y, hw=(64, 64))
        torch.cuda.synchronize()
        print("MARK begin", torch.ops.mdb200.launch_count())
        for _ in range(a.iters):
            fn()
        torch.cuda.synchronize()
        native.check_status()
        print("MARK end", torch.ops.mdb200.launch_count())
        print("ok")
        return
    if a.op in ("gemm", "gemm_fp8"):
        M, N, K = dims or [4608, 3072, 3072]
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        if a.op == "gemm_fp8":
            wq, ws = O.fp8_quant_rows(w)
            fn = lambda: O.fp8_linear(x, wq, ws)
        else:
            fn = lambda: O.linear(x, w)
    elif a.op in ("attention", "attention_bwd"):
        B, S, H, Dh = dims or [1, 4608, 24, 128]
        q, k, v = [torch.randn(B, S, H, Dh, device=dev, dtype=torch.bfloat16, requires_grad=a.op == "attention_bwd")
                   for _ in range(3)]
        if a.op == "attention":
            fn = lambda: O.attention(q.detach(), k.detach(), v.detach())
        else:
            def fn():
                o = O.attention(q, k, v)
                o.backward(torch.ones_like(o))
    else:
        rows, D = dims or [36864, 3072]
        x = torch.randn(rows, D, device=dev, dtype=torch.bfloat16)
        mod = torch.randn(8, 2 * D, device=dev, dtype=torch.bfloat16)
        fn = lambda: O.norm_modulate(x, scale=mod[:, :D], shift=mod[:, D:], rows_per_group=rows // 8)
    for _ in range(a.iters):
        flush.zero_()
        fn()
    torch.cuda.synchronize()
    native.check_status()
    print("ok")


if __name__ == "__main__":
    main()
