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


def summarize(path, first_marker, last_marker):
    """Device time per kernel group of one step out of an ncu launch list (serialised, cold-cache times: compare shares)."""
    import collections
    import csv
    import re
    rows = list(csv.reader(open(path, errors="ignore")))
    hdr_i = next(i for i, r in enumerate(rows) if "Kernel Name" in r)
    hdr = rows[hdr_i]
    ki, mi, ui = hdr.index("Kernel Name"), hdr.index("Metric Value"), hdr.index("Metric Unit")
    data = []
    for r in rows[hdr_i + 1:]:
        if len(r) <= mi:
            continue
        v = float(r[mi].replace(",", ""))
        v = v / 1000 if r[ui] == "ns" else v * 1000 if r[ui] == "ms" else v
        data.append((re.sub(r"\(.*", "", r[ki])[:110], v))
    firsts = [i for i, (k, _) in enumerate(data) if first_marker in k]
    lasts = [i for i, (k, _) in enumerate(data) if last_marker in k]
    if not firsts or not lasts or lasts[-1] < firsts[-1] and len(firsts) < 2:
        print(f"markers not found ({len(firsts)} x {first_marker}, {len(lasts)} x {last_marker}); capture more launches")
        return 1
    end = lasts[-1]
    begin = max(i for i in firsts if i < end)
    step = data[begin:end + 1]
    tot = sum(v for _, v in step)
    groups = collections.OrderedDict((g, [0, 0.0]) for g in ("base GEMMs, CTA-pair 256x256 tiles", "GEMMs, one-CTA 128-wide tiles",
                                                              "skinny (LoRA) GEMMs, 64-wide tiles", "attention backward", "attention forward",
                                                              "own norm / rope / pointwise / optimizer kernels", "torch copy / cat / fill / elementwise"))
    agg = collections.defaultdict(lambda: [0, 0.0])
    for k, v in step:
        agg[k][0] += 1
        agg[k][1] += v
        g = ("base GEMMs, CTA-pair 256x256 tiles" if "pair_kernel" in k else "skinny (LoRA) GEMMs, 64-wide tiles" if "gemm_tcgen05_kernel<64" in k
             else "GEMMs, one-CTA 128-wide tiles" if "gemm_tcgen05_kernel" in k else "attention backward" if ("attention_bwd" in k or "attn_delta" in k)
             else "attention forward" if "attention_fwd" in k else "own norm / rope / pointwise / optimizer kernels" if "mdb::" in k
             else "torch copy / cat / fill / elementwise")
        groups[g][0] += 1
        groups[g][1] += v
    print(f"one step = launches {begin}..{end}: {len(step)} launches, {tot / 1000:.1f} ms of device time (serialised)")
    for g, (n, v) in groups.items():
        print(f"  {v / 1000:8.2f} ms {100 * v / tot:5.1f} %  n={n:5d}  {g}")
    print("  top kernels:")
    for k, (n, v) in sorted(agg.items(), key=lambda t: -t[1][1])[:16]:
        print(f"  {v / 1000:8.2f} ms {100 * v / tot:5.1f} %  n={n:5d}  {k}")
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "gemm_prof", "gemm_trace", "attention_trace", "attention", "attention_bwd", "norm", "qk_norm_rope", "gemm_fp8", "gemm_mxfp8", "flux_step", "flux_train_step", "tp_fused_local", "ulysses_fused_local", "dp_fused_local"])
    ap.add_argument("--shape", default="")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--summarize", default="", help="no GPU work: read an `ncu --metrics gpu__time_duration.sum --csv` launch list and "
                    "print time per kernel group and per kernel, for the launches between --first-marker and --last-marker")
    ap.add_argument("--first-marker", default="flow_match_kernel")
    ap.add_argument("--last-marker", default="adamw")
    a = ap.parse_args()
    if a.summarize:
        return summarize(a.summarize, a.first_marker, a.last_marker)
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
    if a.op == "gemm_prof":
        # in-kernel cycle counters of both GEMM kernels (one CTA per 128 x 256 tile; CTA pair per 256 x 256 tile)
        from mojodiffusion_b200.ops.functional import _gemm
        M, N, K = dims or [4608, 3072, 3072]
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        print("CTA pairs the device holds at once:", torch.ops.mdb200.gemm_pair_capacity())
        names = ["mma_total", "producer_wait_empty", "mma_wait_full", "mma_wait_tmem_empty", "epi_wait_tmem_full", "epi_work", "tiles", "-"]
        for bn in (256, 512):
            for _ in range(2):
                _gemm([x], [w], bn=bn)
            prof = torch.zeros(torch.cuda.get_device_properties(0).multi_processor_count, 8, dtype=torch.int64, device=dev)
            flush.zero_()
            _gemm([x], [w], bn=bn, prof=prof)
            torch.cuda.synchronize()
            pr = prof.cpu().double()
            lead = pr[pr[:, 0] > 0]
            print(f"bn={bn} shape={M}x{N}x{K} CTAs with an MMA role: {lead.shape[0]}")
            for i, nm in enumerate(names[:7]):
                col = pr[:, i][pr[:, i] > 0]
                if col.numel():
                    print(f"  {nm:24s} mean {col.mean():12.0f}  max {col.max():12.0f}  (n={col.numel()})")
        native.check_status()
        print("ok")
        return
    if a.op == "attention_trace":
        # per-kv-tile time line of CTA (0,0,0): who waits for whom (MDB200_ATTN_ISSUE selects how the control warps issue)
        B, S, H, Dh = dims or [1, 4608, 24, 128]
        q, k, v = [torch.randn(B, S, H, Dh, device=dev, dtype=torch.bfloat16) for _ in range(3)]
        n_kv = (S + 127) // 128
        T = 4 * n_kv + 8
        for _ in range(2):
            O.attention(q, k, v)
        tr = torch.zeros(4, T, dtype=torch.int64, device=dev)
        torch.ops.mdb200.attention_set_trace(tr)
        flush.zero_()
        O.attention(q, k, v)
        torch.cuda.synchronize()
        torch.ops.mdb200.attention_set_trace(None)
        tr = tr.cpu()
        t0 = int(tr[2, 0])
        seen, issued = tr[0, :2 * n_kv] - t0, tr[1, :2 * n_kv] - t0
        wg = [(tr[2 + t, :4 * n_kv] - t0).view(n_kv, 4) for t in range(2)]
        print(f"attention B={B} S={S} H={H} Dh={Dh}: {n_kv} kv tiles; issue mode {os.environ.get('MDB200_ATTN_ISSUE', 'default')}")
        print("  kv | MMA: P0 seen, issued, P1 seen, issued | WG0: S seen, loaded, max, P out | WG1: same")
        for j in list(range(0, 6)) + list(range(n_kv - 3, n_kv)):
            print(f"  {j:3d} | {int(seen[2*j]):7d} {int(issued[2*j]):7d} {int(seen[2*j+1]):7d} {int(issued[2*j+1]):7d} | "
                  + " ".join(f"{int(x):7d}" for x in wg[0][j]) + " | " + " ".join(f"{int(x):7d}" for x in wg[1][j]))
        mid = slice(4, n_kv - 2)
        per = (wg[0][mid, 0][1:] - wg[0][mid, 0][:-1]).double()
        print(f"  steady state: period per kv tile {per.mean():.0f} cycles (ideal 2048); WG0 softmax span (S seen -> P out) "
              f"{(wg[0][mid, 3] - wg[0][mid, 0]).double().mean():.0f}, of which load {(wg[0][mid, 1] - wg[0][mid, 0]).double().mean():.0f}, "
              f"max {(wg[0][mid, 2] - wg[0][mid, 1]).double().mean():.0f}, exp+store {(wg[0][mid, 3] - wg[0][mid, 2]).double().mean():.0f}; "
              f"WG0 wait for S (P out -> next S seen) {(wg[0][mid, 0][1:] - wg[0][mid, 3][:-1]).double().mean():.0f}; "
              f"MMA issue time per (kv, q tile) {(issued[8:2*n_kv-4] - seen[8:2*n_kv-4]).double().mean():.0f}")
        native.check_status()
        print("ok")
        return
    if a.op == "gemm_trace":
        # per-K-block time line of CTA 0 (clock64): when the producer saw a free stage and issued its loads, when the MMA
        # issuer saw the operands, when the epilogue saw / drained each accumulator
        from mojodiffusion_b200.ops.functional import _gemm
        M, N, K = dims or [4608, 3072, 3072]
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        sms = torch.cuda.get_device_properties(0).multi_processor_count
        T = 2048
        kb_per_tile = (K + 63) // 64
        for bn in (256, 512):
            for _ in range(2):
                _gemm([x], [w], bn=bn)
            prof = torch.zeros(8 * sms + 6 * T, dtype=torch.int64, device=dev)
            flush.zero_()
            _gemm([x], [w], bn=bn, prof=prof)
            torch.cuda.synchronize()
            tr = prof[8 * sms:].view(2, 3, T).cpu()
            prod, mma, epi = tr[0, 0], tr[0, 1], tr[0, 2]
            n = int((mma > 0).sum())
            t0 = int(prod[0])
            print(f"bn={bn} shape={M}x{N}x{K}: {n} K blocks traced in CTA 0, {kb_per_tile} per tile")
            mm = (mma[:n] - t0).tolist()
            pp = (prod[:n] - t0).tolist()
            print("  first 24 K blocks: producer issue | operands seen | seen - issue")
            for i in range(min(24, n)):
                print(f"    kb {i:3d}  {pp[i]:8d}  {mm[i]:8d}  {mm[i] - pp[i]:6d}")
            for tile in range((n + kb_per_tile - 1) // kb_per_tile):
                lo, hi = tile * kb_per_tile, min(n, (tile + 1) * kb_per_tile)
                d = [mm[i + 1] - mm[i] for i in range(lo, hi - 1)]
                dp = [pp[i + 1] - pp[i] for i in range(lo, hi - 1)]
                lat = [mm[i] - pp[i] for i in range(lo, hi)]
                d.sort(); dp.sort(); lat.sort()
                print(f"  tile {tile}: span {mm[hi - 1] - mm[lo]} cycles for {hi - lo} blocks; MMA-seen step median {d[len(d) // 2]} "
                      f"p90 {d[int(len(d) * .9)]} max {d[-1]}; producer step median {dp[len(dp) // 2]} max {dp[-1]}; "
                      f"seen-issue median {lat[len(lat) // 2]} min {lat[0]} max {lat[-1]}")
            ne = int((epi > 0).sum())
            print("  epilogue (accumulator seen, drained) per tile:", [(int(epi[2 * i] - t0), int(epi[2 * i + 1] - t0)) for i in range(ne // 2)])
            pr = prof[:8 * sms].view(sms, 8).cpu()
            print("  CTA 0 counters: mma_total %d producer_wait %d mma_wait_full %d mma_wait_acc %d epi_wait %d epi_work %d" % tuple(int(v) for v in pr[0, :6]))
        native.check_status()
        print("ok")
        return
    if a.op in ("tp_fused_local", "ulysses_fused_local", "dp_fused_local"):
        # The fused compute+collective kernels of one rank of a 4-rank group, with every "peer" buffer living on this
        # GPU (a profiler is never put around a multi-rank run): same code paths, pointer tables and byte counts as
        # rank 0 of a real group; the transfers go through local memory instead of NVLink.
        from mojodiffusion_b200.ops.functional import _gemm
        world, r = 4, 0
        if a.op == "tp_fused_local":
            rows, D, Fh = dims or [6144, 4096, 16384]
            rl, fl = rows // world, Fh // world
            x_all = [torch.randn(rows, D, device=dev, dtype=torch.bfloat16) for _ in range(world)]
            stage = [torch.empty(world, rl, D, device=dev, dtype=torch.bfloat16) for _ in range(world)]
            w1 = torch.randn(fl, D, device=dev, dtype=torch.bfloat16) * 0.02
            w2 = torch.randn(D, fl, device=dev, dtype=torch.bfloat16) * 0.02
            ready = torch.zeros(8, dtype=torch.int32, device=dev)
            chunk = rl * D * 2
            gptrs = [x_all[c].data_ptr() + c * chunk for c in range(world)]

            def fn():
                h = _gemm([x_all[r]], [w1], act=1, gather_ptrs=gptrs, gather_cfg=[r, 0, rl, chunk], gather_dst=x_all[r], gather_ready=ready)
                _gemm([h], [w2], route_ptrs=[s_.data_ptr() for s_ in stage], route_cfg=[rl, D, r])
        elif a.op == "ulysses_fused_local":
            B, S_txt, S_img, H, Dh = 1, 512, 4096, 24, 128
            S, D, Hl = S_txt + S_img, 24 * 128, 24 // world
            Dl, Si = Hl * Dh, S_img // world
            qkv_g = [torch.zeros(B, S, 3 * Dl, device=dev, dtype=torch.bfloat16) for _ in range(world)]
            attn_x = [torch.zeros(B, (S_txt + S_img) // world, D, device=dev, dtype=torch.bfloat16) for _ in range(world)]
            x = torch.randn(Si, D, device=dev, dtype=torch.bfloat16)
            w = torch.randn(3 * D, D, device=dev, dtype=torch.bfloat16) * 0.02
            g = qkv_g[r]
            g.copy_(torch.randn_like(g))
            q, k, v = (g[..., i * Dl:(i + 1) * Dl].unflatten(-1, (Hl, Dh)) for i in range(3))
            St = S_txt // world
            ra = [t.data_ptr() + r * Dl * 2 for t in attn_x]
            rb = [t.data_ptr() + St * D * 2 + r * Dl * 2 for t in attn_x]

            def fn():
                _gemm([x], [w], route_ptrs=[t.data_ptr() for t in qkv_g], route_cfg=[Dl, D, S_txt + r * Si, Si, S, 3 * Dl])
                torch.ops.mdb200.attention_fwd(q, k, v, 1.0 / Dh ** 0.5, None, False, None, ra, rb,
                                               [St, S_txt, Si, (St + Si) * D, D, Dh])
        else:
            from mojodiffusion_b200.parallel.fused_dp import emulate_ranks, emulated_step
            numel = dims[0] if dims else 88473600
            sets = [[torch.nn.Parameter(torch.randn(numel, device=dev, dtype=torch.bfloat16))] for _ in range(world)]
            ranks = emulate_ranks(sets, lr=1e-4, max_grad_norm=1.0)
            for rk in ranks:
                rk.flat_grads.normal_()
            fn = lambda: emulated_step(ranks)
        for _ in range(a.iters):
            flush.zero_()
            fn()
        torch.cuda.synchronize()
        native.check_status()
        print("ok")
        return
    if a.op == "gemm_mxfp8":
        M, N, K = dims or [4608, 3072, 12288]
        x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
        w = torch.randn(N, K, device=dev, dtype=torch.bfloat16) * 0.02
        xq, xs = O.mxfp8_quant_rows(x, 128)
        wq, ws = O.mxfp8_quant_rows(w, 256)
        fn = lambda: O.gemm_mxfp8(xq, xs, wq, ws)
    elif a.op in ("gemm", "gemm_fp8"):
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
    elif a.op == "qk_norm_rope":
        B, S, H, Dh = dims or [8, 4608, 24, 128]                 # packed q | k | v buffer of 8 FLUX samples: 340 MB
        qkv = torch.randn(B, S, 3 * H * Dh, device=dev, dtype=torch.bfloat16)
        wq, wk = torch.ones(Dh, device=dev, dtype=torch.bfloat16), torch.ones(Dh, device=dev, dtype=torch.bfloat16)
        ids = torch.zeros(S, 3, device=dev)
        ids[:, 1], ids[:, 2] = torch.arange(S, device=dev) // 64, torch.arange(S, device=dev) % 64
        cos, sin = O.rope_table(ids, (16, 56, 56), 10000.0)
        fn = lambda: O.qk_norm_rope(qkv, H, Dh, wq, wk, cos, sin)
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
