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
    ap.add_argument("--op", default="gemm", choices=["gemm", "attention", "attention_bwd", "norm", "gemm_fp8"])
    ap.add_argument("--shape", default="")
    ap.add_argument("--iters", type=int, default=3)
    a = ap.parse_args()
    dev = "cuda"
    native.load(True)
    dims = [int(x) for x in a.shape.split(",")] if a.shape else []
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
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
