"""Counters for the block streamer: how often a block was already there when asked for, how long the compute stream had
to wait for copies, bytes moved (serenitymojo/offload/telemetry.mojo:10-131)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict


@dataclass
class OffloadTelemetry:
    prefetch_calls: int = 0
    await_calls: int = 0
    await_hits: int = 0            # block was already in a slot (prefetched or still there)
    await_misses: int = 0          # copy had to be issued at await time
    resident_hits: int = 0
    h2d_bytes: int = 0
    h2d_copies: int = 0
    await_wait_ns: int = 0
    pack_ns: int = 0

    def hit_rate(self) -> float:
        n = self.await_hits + self.await_misses
        return self.await_hits / n if n else 1.0

    def summary(self) -> Dict[str, float]:
        return {"prefetch_calls": self.prefetch_calls, "await_calls": self.await_calls, "hit_rate": round(self.hit_rate(), 4),
                "resident_hits": self.resident_hits, "h2d_gib": self.h2d_bytes / 2 ** 30, "h2d_copies": self.h2d_copies,
                "await_wait_ms": self.await_wait_ns / 1e6, "pack_ms": self.pack_ns / 1e6}

    def line(self) -> str:
        s = self.summary()
        return "[offload] " + " ".join(f"{k}={v:.4g}" if isinstance(v, float) else f"{k}={v}" for k, v in s.items())
