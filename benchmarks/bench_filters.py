"""Times every image filter: the CUDA kernel (CUDA events, after warm-up, L2 flushed between iterations) against the
vectorised numpy statement on the host cores. ``python benchmarks/bench_filters.py [--size 2048]`` prints one JSON line
per filter; PSNR of kernel vs numpy is reported alongside."""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from mojodiffusion_b200.ops import filters as F  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--size", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    n = a.size
    rng = np.random.default_rng(0)
    ys, xs = np.mgrid[0:n, 0:n].astype(np.float32)
    img = np.stack([0.5 + 0.4 * np.sin(xs / 23.0), 0.5 + 0.4 * np.cos(ys / 17.0), (xs + ys) / (2 * n), np.ones_like(xs)], -1)
    img = np.clip(img + rng.normal(0, 0.02, img.shape).astype(np.float32) * np.array([1, 1, 1, 0], np.float32), 0, 1).astype(np.float32)
    dev = torch.from_numpy(img).cuda()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    small = img[:512, :512].copy()
    for name in sorted(F.OPS):
        for _ in range(3):
            F.image_filter(name, dev)
        times = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            torch.cuda.synchronize()
            e0.record()
            F.image_filter(name, dev)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        t0 = time.perf_counter()
        ref = F.REFERENCE[name](small)
        cpu_ms = (time.perf_counter() - t0) * 1e3 * (n * n) / (512 * 512)     # numpy time scaled to the full image
        got = F.image_filter(name, torch.from_numpy(small).cuda()).cpu().numpy()
        ms = float(np.median(times))
        print(json.dumps({"filter": name, "size": n, "gpu_ms": round(ms, 4), "mpix_per_s": round(n * n / ms / 1e3, 1),
                          "gbytes_per_s_rw": round(2 * n * n * 16 / ms / 1e6, 1), "numpy_ms_scaled": round(cpu_ms, 1),
                          "speedup": round(cpu_ms / ms, 1), "psnr_db_512": round(F.psnr_u8(got, ref), 2)}))


if __name__ == "__main__":
    main()
