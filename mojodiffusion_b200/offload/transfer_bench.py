"""Host<->device bandwidth sweep (pinned and pageable, both directions), timed with CUDA events on the copy stream
(serenitymojo/offload/transfer_benchmark.mojo:142-264). ``python -m mojodiffusion_b200.offload.transfer_bench``."""
from __future__ import annotations

import json
from typing import Dict, List

import torch


def transfer_sweep(sizes_mib=(1, 16, 64, 256, 1024), iters: int = 5, device=0) -> List[Dict]:
    dev = torch.device("cuda", device)
    stream = torch.cuda.Stream(dev)
    rows = []
    for mib in sizes_mib:
        n = mib << 20
        d = torch.empty(n, dtype=torch.uint8, device=dev)
        for pinned in (True, False):
            h = torch.empty(n, dtype=torch.uint8, pin_memory=pinned)
            for direction in ("h2d", "d2h"):
                with torch.cuda.stream(stream):
                    for _ in range(2):
                        (d.copy_(h, non_blocking=True) if direction == "h2d" else h.copy_(d, non_blocking=True))
                    stream.synchronize()
                    e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
                    e0.record(stream)
                    for _ in range(iters):
                        (d.copy_(h, non_blocking=True) if direction == "h2d" else h.copy_(d, non_blocking=True))
                    e1.record(stream)
                    stream.synchronize()
                ms = e0.elapsed_time(e1) / iters
                rows.append({"mib": mib, "pinned": pinned, "dir": direction, "ms": ms, "gib_per_s": (n / 2 ** 30) / (ms / 1e3)})
    return rows


if __name__ == "__main__":
    for r in transfer_sweep():
        print(json.dumps(r))
