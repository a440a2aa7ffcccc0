#!/usr/bin/env python
"""Kernel micro-benchmarks (device-timed with CUDA events, warm-up, L2 flush between iterations):
tcgen05 GEMM vs torch.matmul (cuBLAS) on the DiT shapes, attention forward vs torch SDPA, norm+modulate bandwidth.
Counterpart of the reference's bench_matmul_vs_flame.mojo / bench_sdpa_vs_flame.mojo timing mains.

    python benchmarks/bench_kernels.py [--json out.json]
"""
import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import mojodiffusion_b200.ops as O  # noqa: E402
from mojodiffusion_b200.ops import native  # noqa: E402


def timeit(fn, iters=10, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--json", default=None)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--gemm-only", action="store_true")
    args = ap.parse_args()
    dev = "cuda"
    native.load(True)
    peaks = {}
    pk = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peaks = json.load(open(pk))
    peak_tf = peaks.get("bf16_tflops", 1590.0)
    peak_bw = peaks.get("hbm_gbs", 6650.0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    print("CTA pairs the device holds at once:", torch.ops.mdb200.gemm_pair_capacity(), flush=True)
    rows = []
    shapes = [(4608, 3072, 3072), (4608, 9216, 3072), (4608, 12288, 3072), (4608, 3072, 12288), (4608, 21504, 3072),
              (4608, 3072, 15360), (4096, 16384, 4096), (8192, 8192, 8192)]
    if args.quick:
        shapes = shapes[:3]
    for M, N, K in shapes:
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        from mojodiffusion_b200.ops.functional import _gemm
        t_ours = timeit(lambda: O.linear(x, w), flush=flush)
        t_one = timeit(lambda: _gemm([x], [w], bn=256), flush=flush)     # one CTA per 128 x 256 tile
        t_pair = timeit(lambda: _gemm([x], [w], bn=512), flush=flush)    # CTA pair per 256 x 256 tile, 6 stages
        t_lib = timeit(lambda: torch.matmul(x, w.t()), flush=flush)
        fl = 2.0 * M * N * K
        rows.append({"op": "gemm_bf16", "shape": [M, N, K], "ms": t_ours, "tflops": fl / t_ours / 1e9,
                     "frac_of_measured_peak": fl / t_ours / 1e9 / peak_tf, "one_cta_128x256_tflops": fl / t_one / 1e9,
                     "cta_pair_256x256_tflops": fl / t_pair / 1e9, "cublas_ms": t_lib,
                     "cublas_tflops": fl / t_lib / 1e9})
        print(rows[-1], flush=True)
    if args.gemm_only:
        native.check_status()
        if args.json:
            json.dump(rows, open(args.json, "w"), indent=1)
        return
    for B, S, H, Dh in [(1, 4608, 24, 128), (1, 6144, 32, 128), (2, 4096, 24, 128)][: 1 if args.quick else 3]:
        q, k, v = [torch.randn(B, S, H, Dh, device=dev, dtype=torch.bfloat16) for _ in range(3)]
        t_ours = timeit(lambda: O.attention(q, k, v), flush=flush)
        qt, kt, vt = [t.transpose(1, 2) for t in (q, k, v)]
        t_lib = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(qt, kt, vt), flush=flush)
        fl = 4.0 * B * H * S * S * Dh
        rows.append({"op": "attention_fwd", "shape": [B, S, H, Dh], "ms": t_ours, "tflops": fl / t_ours / 1e9,
                     "frac_of_measured_peak": fl / t_ours / 1e9 / peak_tf, "sdpa_ms": t_lib,
                     "sdpa_tflops": fl / t_lib / 1e9})
        print(rows[-1], flush=True)
    rows_n, D = 36864, 3072
    x = torch.randn(rows_n, D, device=dev, dtype=torch.bfloat16)
    mod = torch.randn(8, 2 * D, device=dev, dtype=torch.bfloat16)
    t = timeit(lambda: O.norm_modulate(x, scale=mod[:, :D], shift=mod[:, D:], rows_per_group=rows_n // 8), flush=flush)
    by = 2.0 * rows_n * D * 2
    rows.append({"op": "layernorm_modulate", "shape": [rows_n, D], "ms": t, "gbs": by / t / 1e6,
                 "frac_of_measured_copy_bw": by / t / 1e6 / peak_bw})
    print(rows[-1], flush=True)
    # QK-RMSNorm + RoPE in place on a packed [S, 3 * 24 * 128] projection buffer (q and k ranges: read + write)
    S, H, Dh = 4608, 24, 128
    qkv = torch.randn(1, S, 3 * H * Dh, device=dev, dtype=torch.bfloat16)
    wq = torch.ones(Dh, device=dev, dtype=torch.bfloat16)
    pos = torch.stack([torch.zeros(S), torch.arange(S).float(), torch.arange(S).float()], 1).to(dev)
    cos, sin = O.rope_table(pos, [16, 56, 56], 10000.0)
    t = timeit(lambda: O.qk_norm_rope(qkv, H, Dh, wq, wq, cos, sin), flush=flush)
    by = 2.0 * S * 2 * H * Dh * 2
    rows.append({"op": "qk_norm_rope", "shape": [S, H, Dh], "ms": t, "gbs": by / t / 1e6, "frac_of_measured_copy_bw": by / t / 1e6 / peak_bw})
    print(rows[-1], flush=True)
    # LoRA linear (rank 16): skinny down projection + the up projection as an extra K segment of the base GEMM, against the
    # chain it replaces (base GEMM, down GEMM, up GEMM accumulated into the base output), both on this package's GEMM and
    # on cuBLAS (addmm for the accumulation)
    for M, N, K in [(4608, 9216, 3072), (4608, 3072, 15360)][: 1 if args.quick else 2]:
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        A = torch.randn(16, K, device=dev, dtype=torch.bfloat16) * 0.02
        Bm = torch.randn(N, 16, device=dev, dtype=torch.bfloat16) * 0.02
        from mojodiffusion_b200.ops.functional import _gemm
        t_fused = timeit(lambda: O.lora_linear(x, w, None, A, Bm, 1.0), flush=flush)
        t_base = timeit(lambda: O.linear(x, w), flush=flush)

        def chain_ours():
            y = _gemm([x], [w])
            return _gemm([_gemm([x], [A])], [Bm], residual=y)

        def chain_lib():
            return torch.addmm(torch.matmul(x, w.t()), torch.matmul(x, A.t()), Bm.t())
        t_chain, t_chain_lib = timeit(chain_ours, flush=flush), timeit(chain_lib, flush=flush)
        rows.append({"op": "lora_linear_r16", "shape": [M, N, K], "fused_ms": t_fused, "base_gemm_ms": t_base,
                     "adapter_cost_ms": t_fused - t_base, "chain_ours_ms": t_chain, "chain_cublas_ms": t_chain_lib})
        print(rows[-1], flush=True)
    native.check_status()
    if args.json:
        json.dump(rows, open(args.json, "w"), indent=1)


if __name__ == "__main__":
    main()
